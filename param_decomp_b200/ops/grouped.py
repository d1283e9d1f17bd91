"""Grouped (per-expert) decomposed sites on the tcgen05 engine.

Jobs (token, slot) are sorted by expert and each expert's run is padded to a multiple of 128 rows,
so every 128-row block of the job matrix belongs to exactly one expert. The GEMM kernel then takes a
per-row-block map to pick the expert's weight matrix (forward and input gradients), and per-expert
K ranges over the shared job axis for the weight gradients (`dW[e] = sum_{j in e} lhs_j^T dout_j`);
experts with no jobs produce all-zero gradients without touching the tensor core.

This replaces the reference's ragged-dot kernels: tokamax `ragged_dot` for forward / dlhs and the
Pallas-Triton transposed grouped matmul for the weight gradient
(param_decomp/routed/experts.py:209-323), with the mask epilogues of the dense site kernel fused in.
"""

from __future__ import annotations

import os
import weakref
from dataclasses import dataclass

import torch
from torch import Tensor

from param_decomp_b200.ops import elementwise as ew
from param_decomp_b200.ops import native as nv

BLOCK = 128  # rows per entry of `bgroup` (one output row block of the grouped kernels)
# Rows every expert's job group is padded to (`PD_GROUP_PAD`). 256 lets a CTA pair share one expert's tile
# (both row blocks of the pair belong to the same expert) at the price of more padding rows; measured on
# the 42-expert top-8 step (65,536 jobs per layer) it is 2% slower than 128 (50.4 vs 49.2 ms), so 128 stays.
PAD = int(os.environ.get("PD_GROUP_PAD", "128"))
assert PAD in (128, 256)
PAIR = 2 if PAD == 256 else 0  # `cta_group` request of the grouped products
_LAYOUTS: dict[tuple[int, int], tuple[weakref.ref, "JobLayout"]] = {}


@dataclass
class JobLayout:
    """Sorted-and-padded job order. `pos[j]` = row of job `j` in the padded matrix."""

    pos: Tensor  # [J] int64
    n_rows: int  # padded row count (multiple of 128)
    bgroup: Tensor  # [n_rows / 128] int32: expert of each row block, -1 for unused tail blocks
    krange: Tensor  # [E, 2] int32: 64-row K-block range of each expert
    counts: Tensor  # [E] int64

    @classmethod
    def cached(cls, indices: Tensor, n_experts: int) -> "JobLayout":
        """The layout of the jobs `indices.reshape(-1)` (token-major, slot-minor), built once per
        routing decision: the clean pass, every masked pass and the CI function of a layer all see the
        same pinned `indices` tensor, so they share one sort."""
        key = (id(indices), n_experts)
        hit = _LAYOUTS.get(key)
        if hit is not None and hit[0]() is indices:
            return hit[1]
        for k in [k for k, (ref, _) in _LAYOUTS.items() if ref() is None]:
            del _LAYOUTS[k]
        layout = cls.build(indices.reshape(-1), n_experts)
        _LAYOUTS[key] = (weakref.ref(indices), layout)
        return layout

    @classmethod
    def cached_local(cls, indices: Tensor, lo: int, n_local: int) -> "JobLayout":
        """The layout one rank of an expert group uses when every rank sees all tokens: the jobs of its own
        experts `[lo, lo + n_local)` form groups `0 .. n_local - 1`, all other jobs are parked in a last group
        whose row blocks carry owner -1, so the grouped products skip them and `combine` leaves them out."""
        key = (id(indices), -(lo * 65536 + n_local) - 1)
        hit = _LAYOUTS.get(key)
        if hit is not None and hit[0]() is indices:
            return hit[1]
        e = indices.reshape(-1)
        mine = (e >= lo) & (e < lo + n_local)
        layout = cls.build(torch.where(mine, e - lo, torch.full_like(e, n_local)), n_local + 1)
        layout.bgroup = torch.where(layout.bgroup == n_local, torch.full_like(layout.bgroup, -1), layout.bgroup)
        layout.krange = layout.krange[:n_local].contiguous()
        layout.foreign = True
        _LAYOUTS[key] = (weakref.ref(indices), layout)
        return layout

    @property
    def skip(self) -> Tensor | None:
        """Row-block owners for the combine kernels when some rows are never computed."""
        return self.bgroup if getattr(self, "foreign", False) else None

    @classmethod
    def build(cls, expert_of_job: Tensor, n_experts: int) -> "JobLayout":
        J = expert_of_job.numel()
        # (a scatter-add, not bincount: bincount sizes its output from the data and synchronises)
        counts = torch.zeros(n_experts, dtype=torch.int64, device=expert_of_job.device).scatter_add_(
            0, expert_of_job, torch.ones_like(expert_of_job))
        padded = (counts + PAD - 1) // PAD * PAD
        starts = torch.cumsum(padded, 0) - padded
        order = expert_of_job.argsort(stable=True)
        sorted_e = expert_of_job[order]
        first = torch.cumsum(counts, 0) - counts
        rank_in_group = torch.arange(J, device=expert_of_job.device) - first[sorted_e]
        pos = torch.empty(J, dtype=torch.int64, device=expert_of_job.device)
        pos[order] = starts[sorted_e] + rank_in_group
        # static upper bound on rows so shapes do not depend on the routing (no host sync)
        n_rows = (J + n_experts * (PAD - 1) + PAD - 1) // PAD * PAD
        blocks = torch.arange(n_rows // BLOCK, device=pos.device) * BLOCK
        ends = starts + padded
        owner = torch.searchsorted(ends, blocks, right=True)
        valid = (owner < n_experts) & (blocks < ends[-1])
        bgroup = torch.where(valid, owner, torch.full_like(owner, -1)).to(torch.int32)
        krange = torch.stack([starts // 64, (starts + padded) // 64], dim=1).to(torch.int32).contiguous()
        return cls(pos, n_rows, bgroup, krange, counts)

    def rowmap(self, k: int, c: int) -> Tensor:
        """`[n_rows, 4]` int32 for the mask epilogues on job rows: padded row -> (token, first column of
        its slot in the narrow `[tokens, k * c]` layout); jobs are token-major, slot-minor. Padding
        rows carry token -1."""
        key = (k, c)
        cache = self.__dict__.setdefault("_rowmaps", {})
        if key not in cache:
            J = self.pos.numel()
            j = torch.arange(J, device=self.pos.device)
            rm = torch.zeros(self.n_rows, 4, dtype=torch.int32, device=self.pos.device)
            rm[:, 0] = -1
            rm[self.pos, 0] = (j // k).to(torch.int32)
            rm[self.pos, 1] = ((j % k) * c).to(torch.int32)
            cache[key] = rm
        return cache[key]

    def expand_tokens(self, x: Tensor, k: int) -> Tensor:
        """`x [N, d]` -> padded sorted job rows `[n_rows, d]`, token `n` feeding its `k` jobs."""
        if _fast_rows(x):
            return _TokensToRows.apply(x, self, k)
        return self.scatter_rows(repeat_rows(x, k))

    def combine(self, padded: Tensor, route_w: Tensor) -> Tensor:
        """`y[n] = sum_s route_w[n, s] * padded[row of job (n, s)]`: job rows back to tokens with the
        routing weights applied. `route_w [N, k]`."""
        N, k = route_w.shape
        if _fast_rows(padded):
            return _RowsToTokens.apply(padded, route_w.float().contiguous(), self)
        y = self.gather_rows(padded).reshape(N, k, -1)
        return (y * route_w.reshape(N, k, 1).to(y.dtype)).sum(1)

    def scatter_rows(self, x_jobs: Tensor) -> Tensor:
        """Job order -> padded sorted rows (zeros in the padding)."""
        return _ScatterRows.apply(x_jobs, self.pos, self.n_rows, self)

    def gather_rows(self, padded: Tensor) -> Tensor:
        """Padded sorted rows -> job order."""
        return _GatherRows.apply(padded, self.pos, self.n_rows, self)


def _fast_rows(t: Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.shape[1] % 8 == 0


class _TokensToRows(torch.autograd.Function):
    """One pass each way: rows are copied in 16-byte pieces through the row map (forward) and summed
    over a token's `k` jobs through its inverse (backward); nothing is cleared or accumulated."""

    @staticmethod
    def forward(ctx, x: Tensor, layout: "JobLayout", k: int) -> Tensor:  # type: ignore[override]
        ctx.layout, ctx.k, ctx.n = layout, k, x.shape[0]
        return ew.rows_expand(x.contiguous(), layout.rowmap(k, 1), None, layout.n_rows, k, rep=1, use_slot=False)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        return ew.rows_combine(g.contiguous(), ctx.layout.pos, None, ctx.n, ctx.k, ctx.layout.skip), None, None


class _RowsToTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, padded: Tensor, route_w: Tensor, layout: "JobLayout") -> Tensor:  # type: ignore[override]
        ctx.layout = layout
        padded = padded.contiguous()
        ctx.save_for_backward(route_w, padded if ctx.needs_input_grad[1] else None)
        N, k = route_w.shape
        return ew.rows_combine(padded, layout.pos, route_w, N, k, layout.skip)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        route_w, padded = ctx.saved_tensors
        layout, (N, k) = ctx.layout, route_w.shape
        g = g.contiguous()
        d_padded = ew.rows_expand(g, layout.rowmap(k, 1), route_w, layout.n_rows, k, rep=1, use_slot=False)
        d_w = None
        if padded is not None:  # routing weights recomputed from the live activations
            d_w = (padded.index_select(0, layout.pos).reshape(N, k, -1).float() * g.float()[:, None, :]).sum(-1)
            if layout.skip is not None:  # rows of jobs this rank never computed hold no data
                owned = layout.skip[(layout.pos >> 7)].reshape(N, k) >= 0
                d_w = torch.where(owned, d_w, torch.zeros((), device=d_w.device))
        return d_padded, d_w, None


def _place_rows(x_jobs: Tensor, pos: Tensor, n_rows: int, layout: "JobLayout") -> Tensor:
    """Job-order rows to their padded positions, zeros elsewhere."""
    if _fast_rows(x_jobs):
        return ew.rows_expand(x_jobs.contiguous(), layout.rowmap(1, 1), None, n_rows, 1, rep=1, use_slot=False)
    out = x_jobs.new_zeros(n_rows, x_jobs.shape[-1])
    out.index_copy_(0, pos, x_jobs)
    return out


class _ScatterRows(torch.autograd.Function):
    """`pos` is injective, so the adjoint of the row scatter is a plain row gather (the generic
    indexing backward would sort the indices to accumulate duplicates that cannot occur)."""

    @staticmethod
    def forward(ctx, x_jobs: Tensor, pos: Tensor, n_rows: int, layout: "JobLayout") -> Tensor:  # type: ignore[override]
        ctx.pos = pos
        return _place_rows(x_jobs, pos, n_rows, layout)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        return g.index_select(0, ctx.pos), None, None, None


class _GatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, padded: Tensor, pos: Tensor, n_rows: int, layout: "JobLayout") -> Tensor:  # type: ignore[override]
        ctx.pos, ctx.n_rows, ctx.layout = pos, n_rows, layout
        return padded.index_select(0, pos)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        return _place_rows(g, ctx.pos, ctx.n_rows, ctx.layout), None, None, None


def repeat_rows(x: Tensor, k: int) -> Tensor:
    """`x [N, d] -> [N * k, d]`, row `n` repeated `k` times in place (token-major jobs); the adjoint
    is a sum over the `k` copies rather than an index accumulation."""
    return x.unsqueeze(1).expand(x.shape[0], k, x.shape[1]).reshape(x.shape[0] * k, x.shape[1])


class _GroupedSite(torch.autograd.Function):
    """Blocked site on padded sorted jobs. `x [R, d_in]`, `V [E, d_in, c]`, `U [E, c, d_out]`,
    `W [E, d_out, d_in]`, `mask [R, c]` (materialised, may require grad), `delta/d_eff/rowscale [R]`."""

    @staticmethod
    def forward(ctx, x, mask, delta, V, U, W, gV, gU, layout: JobLayout, rowscale, d_eff, need_wgrad: bool):  # type: ignore[override]
        R = x.shape[0]
        E, _, c = V.shape
        d_out = U.shape[-1]
        A = torch.empty(R, c, device=x.device, dtype=torch.bfloat16)
        need_H = mask is not None and mask.requires_grad
        H = torch.empty_like(A) if need_H else None
        ci = mask if mask is not None else torch.ones(1, c, device=x.device, dtype=torch.bfloat16).expand(R, c)
        nv.gemm(x, V, A, b_mn=True, epi=nv.EPI_MASK_FWD, out1=H, ci=ci, delta=delta, rowscale=rowscale, mask_mode=1,
                bgroup_of_mblock=layout.bgroup, cta_group=PAIR)
        y = torch.empty(R, d_out, device=x.device, dtype=torch.bfloat16)
        if d_eff is not None:
            xd = ew.rowscale(x, d_eff)
            nv.gemm(A, U, y, b_mn=True, a1=xd, b1=W, bgroup_of_mblock=layout.bgroup, cta_group=PAIR)
        else:
            nv.gemm(A, U, y, b_mn=True, bgroup_of_mblock=layout.bgroup, cta_group=PAIR)
        ctx.save_for_backward(x, mask, delta, rowscale, d_eff, A, H, V, U, W)
        ctx.layout, ctx.sinks, ctx.need_wgrad = layout, (gV, gU), need_wgrad
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x, mask, delta, rowscale, d_eff, A, H, V, U, W = ctx.saved_tensors
        layout: JobLayout = ctx.layout
        gV, gU = ctx.sinks
        R, d_in = x.shape
        E, _, c = V.shape
        dy = dy.contiguous()
        dH = torch.empty(R, c, device=x.device, dtype=torch.bfloat16)
        dm = torch.empty(R, c, device=x.device, dtype=torch.bfloat16) if H is not None else None
        ci = mask if mask is not None else torch.ones(1, c, device=x.device, dtype=torch.bfloat16).expand(R, c)
        nv.gemm(dy, U, dH, epi=nv.EPI_MASK_BWD, ci=ci, h=H, delta=delta, rowscale=rowscale, dci=dm, mask_mode=1,
                bgroup_of_mblock=layout.bgroup, cta_group=PAIR)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(R, d_in, device=x.device, dtype=torch.bfloat16)
            if d_eff is not None:
                dyd = ew.rowscale(dy, d_eff)
                nv.gemm(dH, V, dx, a1=dyd, b1=W, b1_mn=True, bgroup_of_mblock=layout.bgroup, cta_group=PAIR)
            else:
                nv.gemm(dH, V, dx, bgroup_of_mblock=layout.bgroup, cta_group=PAIR)
        if ctx.need_wgrad:
            # dV[e] += x_e^T dH_e ; dU[e] += A_e^T dy_e  (ragged K ranges over the job axis)
            nv.gemm(x, dH, gV, a_mn=True, b_mn=True, accumulate=True, kblock_range=layout.krange, a_bcast=True,
                    b_bcast=True)
            nv.gemm(A, dy, gU, a_mn=True, b_mn=True, accumulate=True, kblock_range=layout.krange, a_bcast=True,
                    b_bcast=True)
        dmask = dm if (dm is not None and ctx.needs_input_grad[1]) else None
        return dx, dmask, None, None, None, None, None, None, None, None, None, None


def grouped_site(x: Tensor, V: Tensor, U: Tensor, W: Tensor | None, layout: JobLayout, mask: Tensor | None,
                 delta: Tensor | None, route: Tensor | None, grad_V: Tensor | None, grad_U: Tensor | None,
                 need_wgrad: bool) -> Tensor:
    """All arguments already in padded sorted-job order (`layout.scatter_rows`)."""
    rowscale = d_eff = None
    if route is not None:
        rowscale = route.float()
        d_eff = (rowscale * delta + (1 - rowscale)) if delta is not None else (1 - rowscale)
    elif delta is not None:
        d_eff = delta
    if mask is not None and mask.dtype != torch.bfloat16:
        mask = mask.to(torch.bfloat16)
    return _GroupedSite.apply(x.contiguous(), mask, delta, V, U, W, grad_V, grad_U, layout, rowscale, d_eff, need_wgrad)


def grouped_linear(x: Tensor, W: Tensor, layout: JobLayout) -> Tensor:
    """Frozen expert bank `y_j = x_j W[e(j)]^T` (clean forward)."""
    y = torch.empty(x.shape[0], W.shape[1], device=x.device, dtype=torch.bfloat16)
    nv.gemm(x.contiguous(), W, y, bgroup_of_mblock=layout.bgroup, cta_group=PAIR)
    return y


class _GroupedLinearTrainable(torch.autograd.Function):
    """`y_j = x_j W[e(j)] + b[e(j)]` on padded sorted jobs with gradients for `x`, `W [E, K, N]`
    (fp32 master, read through a bf16 copy) and `b [E, N]`."""

    @staticmethod
    def forward(ctx, x: Tensor, W: Tensor, b: Tensor | None, layout: JobLayout) -> Tensor:  # type: ignore[override]
        from param_decomp_b200.ops.elementwise import cast_bf16

        Wb = cast_bf16(W.detach().contiguous()) if W.dtype != torch.bfloat16 else W.detach().contiguous()
        R, _ = x.shape
        N = W.shape[-1]
        x = x.contiguous()
        y = torch.empty(R, N, device=x.device, dtype=torch.bfloat16)
        nv.gemm(x, Wb, y, b_mn=True, bgroup_of_mblock=layout.bgroup, cta_group=PAIR)
        if b is not None:
            # rows of padding blocks carry expert -1: they are never read back, any bias row will do
            row_e = layout.bgroup.clamp_min(0).long().repeat_interleave(BLOCK)
            y = y + b.detach().to(torch.bfloat16)[row_e]
        ctx.save_for_backward(x, Wb)
        ctx.layout, ctx.has_bias, ctx.w_dtype = layout, b is not None, W.dtype
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        x, Wb = ctx.saved_tensors
        layout: JobLayout = ctx.layout
        dy = dy.contiguous()
        E, K, N = Wb.shape
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            nv.gemm(dy, Wb, dx, bgroup_of_mblock=layout.bgroup, cta_group=PAIR)  # W_e [K, N] as the K-major B of dx = dy W_e^T
        dW = torch.zeros(E, K, N, device=x.device, dtype=torch.float32)
        nv.gemm(x, dy, dW, a_mn=True, b_mn=True, accumulate=True, kblock_range=layout.krange, a_bcast=True, b_bcast=True)
        db = None
        if ctx.has_bias:
            # every 128-row block belongs to one expert: reduce inside blocks first, then add the few
            # hundred block sums into their experts (a row-wise index_add would serialise on E rows)
            blocks = dy.float().view(-1, BLOCK, N).sum(1)
            be = layout.bgroup.long()
            db = torch.zeros(E, N, device=x.device, dtype=torch.float32)
            db.index_add_(0, be.clamp_min(0), blocks * (be >= 0)[:, None])
        return dx, dW.to(ctx.w_dtype), db, None


def grouped_linear_trainable(x: Tensor, W: Tensor, b: Tensor | None, layout: JobLayout) -> Tensor:
    """Per-expert trainable linear on padded sorted job rows (`layout.scatter_rows`)."""
    return _GroupedLinearTrainable.apply(x, W, b, layout)


class _GroupedSiteMapped(torch.autograd.Function):
    """Blocked site whose mask inputs stay in their source layout: `ci [N, k c]` (narrow CI or a
    materialised mask), `delta`, `rowscale [N]`; the kernels reach them through `rowmap`, draw the
    stochastic mask in the epilogue (`mode 0`) and write the CI gradient back in the narrow layout."""

    @staticmethod
    def forward(ctx, x, ci, delta, V, U, W, gV, gU, layout: JobLayout, rowscale, d_eff_rows, need_wgrad: bool,
                rowmap: Tensor, mode: int, seed: int, stream: int, row_offset: int):  # type: ignore[override]
        R = x.shape[0]
        E, _, c = V.shape
        d_out = U.shape[-1]
        A = torch.empty(R, c, device=x.device, dtype=torch.bfloat16)
        need_H = ci.requires_grad
        H = torch.empty_like(A) if need_H else None
        rng = dict(seed=seed, rng_stream=stream, row_offset=row_offset, mask_mode=mode, rowmap=rowmap)
        nv.gemm(x, V, A, b_mn=True, epi=nv.EPI_MASK_FWD, out1=H, ci=ci, delta=delta, rowscale=rowscale,
                bgroup_of_mblock=layout.bgroup, cta_group=PAIR, **rng)
        y = torch.empty(R, d_out, device=x.device, dtype=torch.bfloat16)
        if d_eff_rows is not None:
            xd = ew.rowscale(x, d_eff_rows)
            nv.gemm(A, U, y, b_mn=True, a1=xd, b1=W, bgroup_of_mblock=layout.bgroup, cta_group=PAIR)
        else:
            nv.gemm(A, U, y, b_mn=True, bgroup_of_mblock=layout.bgroup, cta_group=PAIR)
        ctx.save_for_backward(x, ci, delta, rowscale, d_eff_rows, A, H, V, U, W, rowmap)
        ctx.layout, ctx.sinks, ctx.need_wgrad, ctx.rng = layout, (gV, gU), need_wgrad, (mode, seed, stream, row_offset)
        return y

    @staticmethod
    def backward(ctx, dy):  # type: ignore[override]
        x, ci, delta, rowscale, d_eff_rows, A, H, V, U, W, rowmap = ctx.saved_tensors
        layout: JobLayout = ctx.layout
        gV, gU = ctx.sinks
        mode, seed, stream, row_offset = ctx.rng
        R, d_in = x.shape
        c = V.shape[-1]
        dy = dy.contiguous()
        dH = torch.empty(R, c, device=x.device, dtype=torch.bfloat16)
        dci = torch.zeros_like(ci) if H is not None else None
        nv.gemm(dy, U, dH, epi=nv.EPI_MASK_BWD, ci=ci, h=H, delta=delta, rowscale=rowscale, dci=dci,
                bgroup_of_mblock=layout.bgroup, cta_group=PAIR, seed=seed, rng_stream=stream, row_offset=row_offset, mask_mode=mode,
                rowmap=rowmap)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(R, d_in, device=x.device, dtype=torch.bfloat16)
            if d_eff_rows is not None:
                nv.gemm(dH, V, dx, a1=ew.rowscale(dy, d_eff_rows), b1=W, b1_mn=True, bgroup_of_mblock=layout.bgroup, cta_group=PAIR)
            else:
                nv.gemm(dH, V, dx, bgroup_of_mblock=layout.bgroup, cta_group=PAIR)
        if ctx.need_wgrad:
            nv.gemm(x, dH, gV, a_mn=True, b_mn=True, accumulate=True, kblock_range=layout.krange, a_bcast=True,
                    b_bcast=True)
            nv.gemm(A, dy, gU, a_mn=True, b_mn=True, accumulate=True, kblock_range=layout.krange, a_bcast=True,
                    b_bcast=True)
        return (dx, dci if ctx.needs_input_grad[1] else None) + (None,) * 15


def grouped_site_mapped(x: Tensor, V: Tensor, U: Tensor, W: Tensor, layout: JobLayout, ci: Tensor, mode: int,
                        seed: int, stream: int, row_offset: int, delta: Tensor | None, route: Tensor | None, k: int,
                        grad_V: Tensor | None, grad_U: Tensor | None, need_wgrad: bool) -> Tensor:
    """`x` padded job rows; `ci [N, k c]` bf16 in token order; `delta`, `route [N]` per token."""
    c = V.shape[-1]
    rowmap = layout.rowmap(k, c)
    rowscale = d_tok = None
    if route is not None:
        rowscale = route.float().contiguous()
        d_tok = (rowscale * delta + (1 - rowscale)) if delta is not None else (1 - rowscale)
    elif delta is not None:
        d_tok = delta
    d_rows = None
    if d_tok is not None:
        tok = rowmap[:, 0].long()
        d_rows = torch.where(tok >= 0, d_tok[tok.clamp_min(0)], torch.zeros((), device=x.device)).contiguous()
    return _GroupedSiteMapped.apply(x.contiguous(), ci, delta, V, U, W, grad_V, grad_U, layout, rowscale, d_rows,
                                    need_wgrad, rowmap, mode, seed, stream, row_offset)
