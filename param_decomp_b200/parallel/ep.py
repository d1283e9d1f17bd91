"""Expert parallelism for the MoE target: experts (frozen weights + their component blocks) are
sharded over the expert group, tokens stay data-parallel, and jobs travel to their expert's owner.

Two modes
  * `all_to_all` (default): each job's activation row and its per-job mask rows are sent to the
    owning rank (variable counts, exchanged first), the owner runs its experts' gate/up/down sites on
    the received jobs, and the output rows return by the reverse all-to-all. Differentiable: the
    backward of a dispatch is a combine and vice versa.
  * `allreduce`: the reference's scheme ("EP by activation slicing", param_decomp/routed/
    experts.py:28-40,864-885): every rank sees all tokens of its data shard's group, computes only
    its local experts' jobs, partial outputs are summed over the group. Kept for parity and as the
    baseline the all-to-all path is measured against.

Experts are padded with never-routed dummies so their count tiles the group (the analogue of stack
padding): `E_pad = ceil(E / W) * W`, rank `r` owns experts `[r E_loc, (r+1) E_loc)`.

Transports of the all-to-all mode
  * `collective`: `torch.distributed.all_to_all_single` (NCCL on GPUs, gloo on CPU).
  * `p2p` (GPUs of one NVLink domain): `ops/csrc/collectives_sm100.cu::pd_ep_scatter_rows`. Every job
    row is read through the router's permutation and stored straight into its owner's receive buffer
    (symmetric memory, 16-byte peer stores), grouped by source rank in job order, so the result is
    bit-identical to the collective transport; the kernel ends with a bounded cross-GPU barrier. The
    combine is the same kernel with the maps reversed, writing each output row at its source job index.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor

from param_decomp_b200.core.masking import SiteMask


def _tie(y: Tensor, shipped: list[Tensor]) -> Tensor:
    """`y` with an autograd edge to every received tensor. The adjoint of each exchange is itself an exchange that
    every rank must enter; a rank whose local expert computation happens not to depend on one of its received
    tensors (it received no job at all, or a site ignores an input) would otherwise skip that exchange in the
    backward pass and leave the other ranks waiting in it. Adds exact zeros."""
    for t in shipped:
        y = y + (t.sum() * 0.0).to(y.dtype)
    return y


def padded_experts(n_experts: int, world: int) -> int:
    return (n_experts + world - 1) // world * world


def local_expert_range(n_experts: int, rank: int, world: int) -> tuple[int, int]:
    e_loc = padded_experts(n_experts, world) // world
    return rank * e_loc, (rank + 1) * e_loc


def shard_expert_weights(weights: dict[str, Tensor], n_experts: int, rank: int, world: int) -> dict[str, Tensor]:
    """Keep this rank's slice of every `experts_*` weight (zero-padded dummies at the tail)."""
    lo, hi = local_expert_range(n_experts, rank, world)
    out = {}
    for k, w in weights.items():
        if ".experts_" in k and w.dim() == 3:
            pad = padded_experts(n_experts, world) - w.shape[0]
            if pad:
                w = torch.cat([w, w.new_zeros(pad, *w.shape[1:])], dim=0)
            out[k] = w[lo:hi].contiguous()
        else:
            out[k] = w
    return out


class _AllToAll(torch.autograd.Function):
    """Variable-count all-to-all of rows; backward is the transposed exchange."""

    @staticmethod
    def forward(ctx, x: Tensor, send: list[int], recv: list[int], group) -> Tensor:  # type: ignore[override]
        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = x.new_empty(sum(recv), *x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        out = g.new_empty(sum(ctx.send), *g.shape[1:])
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv,
                               group=ctx.group)
        return out, None, None, None


from param_decomp_b200.parallel.group_ops import CopyToGroup as _CopyToGroup  # noqa: E402
from param_decomp_b200.parallel.group_ops import ReduceFromGroup as _ReduceFromGroup  # noqa: E402


class P2PRows:
    """Symmetric receive buffers + flags of one expert group for `pd_ep_scatter_rows`.

    Buffers are keyed by row size and double-buffered: an exchange may only overwrite a buffer whose
    previous content every rank has already copied out, which the barrier of the exchange in between
    guarantees (stream order on each rank: copy-out, then the next exchange's kernel)."""

    def __init__(self, group: Any, device: torch.device, wait_limit_s: float = 2.0) -> None:
        from param_decomp_b200.parallel.sharded_optim import symmetric_empty

        self.group, self.device, self.limit = group, device, wait_limit_s
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self._alloc = symmetric_empty
        self.flags, self.flag_ptrs = symmetric_empty(8, torch.int32, device, group)
        self.flags.zero_()
        self.ticket = torch.zeros(1, device=device, dtype=torch.int32)
        self.seq = 0
        self.bufs: dict[int, list] = {}
        self.turn: dict[int, int] = {}
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def _buffer(self, row_bytes: int, cap_rows: int):
        need = row_bytes * cap_rows
        cur = self.bufs.get(row_bytes)
        if cur is None or cur[0][0].numel() < need:  # collective: every rank reaches this with the same sizes
            self.bufs[row_bytes] = [self._alloc(need, torch.uint8, self.device, self.group) for _ in range(2)]
            self.turn[row_bytes] = 0
        t = self.turn[row_bytes]
        self.turn[row_bytes] = 1 - t
        return self.bufs[row_bytes][t]

    def exchange(self, rows: Tensor, gather: Tensor | None, dest_rank: Tensor, dest_row: Tensor, n_out: int,
                 cap_rows: int) -> Tensor:
        """Row `j` (or `rows[gather[j]]`) lands at row `dest_row[j]` of rank `dest_rank[j]`'s buffer;
        returns the `n_out` rows this rank received."""
        import ctypes as C

        from param_decomp_b200.ops import native as nv
        from param_decomp_b200.parallel.sharded_optim import PdPeerPtrs, _peer_table

        assert rows.dim() == 2 and rows.is_contiguous()
        row_bytes = rows.shape[1] * rows.element_size()
        assert row_bytes % 16 == 0, "payload rows must be a multiple of 16 bytes"
        buf, ptrs = self._buffer(row_bytes, cap_rows)

        class Call(C.Structure):
            _fields_ = [("src", C.c_void_p * 2), ("row_bytes", C.c_int * 2), ("dst", PdPeerPtrs * 2),
                        ("gather", C.c_void_p), ("dest_rank", C.c_void_p), ("dest_row", C.c_void_p),
                        ("n", C.c_longlong), ("flags", PdPeerPtrs), ("rank", C.c_int), ("world", C.c_int),
                        ("seq", C.c_uint), ("ticket", C.c_void_p), ("status", C.c_void_p), ("limit_s", C.c_double)]

        c = Call()
        c.src[0], c.row_bytes[0] = rows.data_ptr() if rows.numel() else buf.data_ptr(), row_bytes
        c.dst[0] = _peer_table(ptrs)
        c.gather = gather.data_ptr() if gather is not None else None
        c.dest_rank, c.dest_row = dest_rank.data_ptr(), dest_row.data_ptr()
        c.n = dest_rank.numel()
        c.flags = _peer_table(self.flag_ptrs)
        c.rank, c.world = self.rank, self.world
        self.seq += 1
        c.seq, c.ticket, c.status, c.limit_s = self.seq, self.ticket.data_ptr(), nv.status_word().data_ptr(), self.limit
        lib = nv.lib()
        lib.pd_ep_scatter_rows.argtypes = [C.c_void_p, C.c_void_p]
        rc = lib.pd_ep_scatter_rows(C.byref(c), nv.current_stream_ptr())
        nv.count_launch()
        if rc != 0:
            raise nv.NativeError(f"pd_ep_scatter_rows failed (code {rc})")
        return buf[: n_out * row_bytes].view(rows.dtype).view(n_out, rows.shape[1]).clone()


class _P2PExchange(torch.autograd.Function):
    """Differentiable row exchange: the backward sends gradient rows along the reversed maps."""

    @staticmethod
    def forward(ctx, rows: Tensor, p2p: P2PRows, gather, fwd_rank, fwd_row, n_out: int, bwd_rank, bwd_row,
                cap_rows: int) -> Tensor:  # type: ignore[override]
        ctx.p2p, ctx.gather, ctx.maps, ctx.cap = p2p, gather, (bwd_rank, bwd_row), cap_rows
        ctx.n_src, ctx.n_jobs = rows.shape[0], fwd_rank.numel()
        return p2p.exchange(rows.contiguous(), gather, fwd_rank, fwd_row, n_out, cap_rows)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        bwd_rank, bwd_row = ctx.maps
        gj = ctx.p2p.exchange(g.contiguous(), None, bwd_rank, bwd_row, ctx.n_jobs, ctx.cap)
        if ctx.gather is not None:
            gj = gj.new_zeros(ctx.n_src, gj.shape[1]).index_add_(0, ctx.gather, gj)
        return gj, None, None, None, None, None, None, None, None


@dataclass
class ExpertParallel:
    group: Any
    n_experts: int  # the model's true expert count (before padding)
    mode: str = "all_to_all"
    transport: str = "collective"  # or "p2p": direct peer stores over NVLink (GPUs only)

    def __post_init__(self) -> None:
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.e_loc = padded_experts(self.n_experts, self.world) // self.world
        self._p2p: P2PRows | None = None

    # ---------------------------------------------------------------------------------------------
    def run_experts(self, model, layer: int, xt: Tensor, expert_of_job: Tensor, token_of_job: Tensor,
                    slot_of_job: Tensor, weights, masks) -> Tensor:
        """`xt [N, d]` local tokens; returns `[J, d]` outputs in job order (token-major, slot-minor)."""
        if self.mode == "allreduce":
            return self._allreduce(model, layer, xt, expert_of_job, token_of_job, slot_of_job, weights, masks)
        if self.transport == "p2p":
            return self._all_to_all_p2p(model, layer, xt, expert_of_job, token_of_job, slot_of_job, weights, masks)
        J = expert_of_job.numel()
        dest = expert_of_job // self.e_loc
        order = dest.argsort(stable=True)
        send = torch.bincount(dest, minlength=self.world)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        send_l, recv_l = send.tolist(), recv.tolist()

        shipped: list[Tensor] = []  # received tensors whose adjoint is a collective (see `_tie`)

        def ship(rows: Tensor) -> Tensor:
            out = _AllToAll.apply(rows[order], send_l, recv_l, self.group)
            if out.requires_grad:
                shipped.append(out)
            return out

        x_recv = ship(xt[token_of_job])
        e_recv = _AllToAll.apply((expert_of_job % self.e_loc)[order], send_l, recv_l, self.group)
        # per-job mask payload of the three expert sites
        names = model.expert_site_names(layer)
        job_masks: dict[str, SiteMask] = {}
        if masks is not None:
            for name in names:
                if name not in masks:
                    continue
                sm = masks[name].materialize()
                spec = next(s for s in model.sites if s.name == name)
                c = spec.C_block
                m = d = r = None
                if sm.mask is not None:
                    flat = sm.mask.reshape(-1, sm.mask.shape[-1])
                    m = ship(flat.reshape(flat.shape[0], flat.shape[1] // c, c)[token_of_job, slot_of_job])
                if sm.delta is not None:
                    d = ship(sm.delta.reshape(-1, 1)[token_of_job])
                if sm.route is not None:
                    r = ship(sm.route.reshape(-1, 1)[token_of_job].float())[:, 0] > 0.5
                job_masks[name] = SiteMask(mask=m, delta=d, route=r)
        Jr = x_recv.shape[0]
        ar = torch.arange(Jr, device=xt.device)
        y_recv = self._local(model, layer, x_recv, e_recv, weights, job_masks if masks is not None else None, ar)
        y_recv = _tie(y_recv, shipped)
        y_sorted = _AllToAll.apply(y_recv, recv_l, send_l, self.group)
        inv = torch.empty_like(order)
        inv[order] = torch.arange(J, device=order.device)
        return y_sorted[inv]

    def fast_allreduce(self, model, xt: Tensor) -> bool:
        """Whether `run_tokens_allreduce` applies: all-reduce mode on the fused backend with mask inputs
        read through the row map."""
        return self.mode == "allreduce" and model._fused(xt) and getattr(model, "use_row_map", False)

    def run_tokens_allreduce(self, model, layer: int, xt: Tensor, indices: Tensor, route_w: Tensor, weights, masks,
                             token_of_job: Tensor, slot_of_job: Tensor) -> Tensor:
        """All-reduce mode on the grouped kernels, tokens in and tokens out. The job layout parks every other
        rank's jobs in row blocks without an owner, so the grouped products touch this rank's experts only and
        the routing-weighted combine leaves the rest out; the mask inputs stay in token order (read through the
        row map). No host synchronisation: shapes do not depend on the routing."""
        from dataclasses import replace

        from param_decomp_b200.ops.grouped import JobLayout
        from param_decomp_b200.parallel.group_ops import copy_to_group

        layout = JobLayout.cached_local(indices, self.rank * self.e_loc, self.e_loc)
        shared = dict(masks) if masks is not None else None
        if shared is not None:
            for name in model.expert_site_names(layer):
                sm = shared.get(name)
                if sm is None:
                    continue
                cut = lambda t: None if t is None else copy_to_group(t, self.group)  # noqa: E731
                shared[name] = replace(sm, ci=cut(sm.ci), mask=cut(sm.mask), delta=cut(sm.delta))
        y = model.expert_tokens(layer, copy_to_group(xt, self.group), indices, copy_to_group(route_w, self.group),
                                weights, shared, token_of_job, slot_of_job, layout=layout)
        return _ReduceFromGroup.apply(y, self.group)

    def _all_to_all_p2p(self, model, layer: int, xt: Tensor, expert_of_job: Tensor, token_of_job: Tensor,
                        slot_of_job: Tensor, weights, masks) -> Tensor:
        """Same result as the collective transport; rows move by `pd_ep_scatter_rows`."""
        if self._p2p is None:
            self._p2p = P2PRows(self.group, xt.device)
        p2p, W = self._p2p, self.world
        J = expert_of_job.numel()
        cap = W * J  # every rank sends J jobs; an owner can receive at most all of them
        dest = (expert_of_job // self.e_loc).to(torch.int32)
        send = torch.bincount(dest, minlength=W)
        cm = torch.empty(W, W, dtype=send.dtype, device=send.device)  # cm[s, r]: jobs rank s sends to rank r
        dist.all_gather_into_tensor(cm, send, group=self.group)
        base = cm[: self.rank].sum(0)  # my first row in each owner's buffer (rows grouped by source rank)
        order = dest.argsort(stable=True)
        first = torch.cumsum(send, 0) - send
        slot = torch.empty(J, dtype=torch.int64, device=dest.device)
        slot[order] = torch.arange(J, device=dest.device) - first[dest[order].long()]
        dest_row = base[dest.long()] + slot
        recv_from = cm[:, self.rank]
        R = int(recv_from.sum())  # one host read per layer call, as on the collective path
        src_rank_of_row = torch.repeat_interleave(torch.arange(W, device=dest.device, dtype=torch.int32), recv_from,
                                                  output_size=R)
        # metadata rides along first: (source job index, local expert id) per received row
        meta = torch.zeros(J, 4, dtype=torch.int32, device=dest.device)
        meta[:, 0] = torch.arange(J, device=dest.device, dtype=torch.int32)
        meta[:, 1] = (expert_of_job % self.e_loc).to(torch.int32)
        meta_recv = p2p.exchange(meta, None, dest, dest_row, R, cap)
        src_job = meta_recv[:, 0].long()
        e_recv = meta_recv[:, 1].long()

        def pad16(rows: Tensor) -> tuple[Tensor, int]:
            cols = rows.shape[1]
            per16 = 16 // rows.element_size()
            extra = (-cols) % per16
            return (torch.nn.functional.pad(rows, (0, extra)) if extra else rows), cols

        shipped: list[Tensor] = []

        def ship(rows: Tensor, gather: Tensor | None) -> Tensor:
            rows, cols = pad16(rows)
            out = _P2PExchange.apply(rows, p2p, gather, dest, dest_row, R, src_rank_of_row, src_job, cap)
            if out.requires_grad:
                shipped.append(out)
            return out[:, :cols]

        x_recv = ship(xt, token_of_job)  # the router's gather is applied by the kernel
        names = model.expert_site_names(layer)
        job_masks: dict[str, SiteMask] = {}
        if masks is not None:
            for name in names:
                if name not in masks:
                    continue
                sm = masks[name].materialize()
                c = next(s for s in model.sites if s.name == name).C_block
                m = d = r = None
                if sm.mask is not None:
                    flat = sm.mask.reshape(-1, sm.mask.shape[-1])
                    m = ship(flat.reshape(flat.shape[0], flat.shape[1] // c, c)[token_of_job, slot_of_job], None)
                if sm.delta is not None:
                    d = ship(sm.delta.reshape(-1, 1), token_of_job)
                if sm.route is not None:
                    r = ship(sm.route.reshape(-1, 1).float(), token_of_job)[:, 0] > 0.5
                job_masks[name] = SiteMask(mask=m, delta=d, route=r)
        ar = torch.arange(R, device=xt.device)
        y_recv = self._local(model, layer, x_recv, e_recv, weights, job_masks if masks is not None else None, ar)
        y_recv = _tie(y_recv, shipped)
        y_rows, cols = pad16(y_recv)
        y = _P2PExchange.apply(y_rows, p2p, None, src_rank_of_row, src_job, J, dest, dest_row, cap)
        return y[:, :cols]

    def _local(self, model, layer: int, x_jobs: Tensor, e_local: Tensor, weights, masks, ar: Tensor) -> Tensor:
        order, bounds = e_local, [0]
        if not model._fused(x_jobs):
            order = e_local.argsort(stable=True)
            for n in torch.bincount(e_local, minlength=self.e_loc).tolist():
                bounds.append(bounds[-1] + n)
        return model.expert_jobs(layer, x_jobs, e_local, order, bounds, weights, masks, ar, torch.zeros_like(ar))

    def _allreduce(self, model, layer, xt, expert_of_job, token_of_job, slot_of_job, weights, masks) -> Tensor:
        """Tokens are replicated over the group; this rank runs the jobs of its own experts and the
        partial outputs are summed. Gradients are exact on every rank: inputs shared by the ranks
        (activations, mask inputs) pass through `_CopyToGroup`, the sum through `_ReduceFromGroup`, so
        replicated parameters upstream see the full gradient and local expert blocks see their own."""
        lo = self.rank * self.e_loc
        mine = (expert_of_job >= lo) & (expert_of_job < lo + self.e_loc)
        idx = mine.nonzero()[:, 0]
        share = lambda t: _CopyToGroup.apply(t, self.group) if t.requires_grad else t  # noqa: E731
        xt = share(xt)
        y = xt.new_zeros(expert_of_job.numel(), xt.shape[-1])
        keep_alive = xt.sum() * 0  # every rank must reach the same backward collectives, jobs or not
        sub_masks = None
        if masks is not None:
            sub_masks = {}
            for name in model.expert_site_names(layer):
                if name not in masks:
                    continue
                sm = masks[name].materialize()
                c = next(s for s in model.sites if s.name == name).C_block
                m = d = None
                if sm.mask is not None:
                    flat = share(sm.mask.reshape(-1, sm.mask.shape[-1]))
                    keep_alive = keep_alive + flat.sum() * 0
                    m = flat.reshape(flat.shape[0], flat.shape[1] // c, c)[token_of_job[idx], slot_of_job[idx]]
                if sm.delta is not None:
                    dl = share(sm.delta.reshape(-1, 1))
                    keep_alive = keep_alive + dl.sum() * 0
                    d = dl[token_of_job[idx]]
                r = None if sm.route is None else sm.route.reshape(-1)[token_of_job[idx]]
                sub_masks[name] = SiteMask(mask=m, delta=d, route=r)
        if idx.numel():
            ar = torch.arange(idx.numel(), device=xt.device)
            y_local = self._local(model, layer, xt[token_of_job[idx]], expert_of_job[idx] - lo, weights, sub_masks, ar)
            y = y.index_copy(0, idx, y_local.to(y.dtype))
        return _ReduceFromGroup.apply(y + keep_alive.to(y.dtype), self.group)
