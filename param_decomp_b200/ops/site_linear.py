"""Fused decomposed-linear site on the tcgen05 GEMM engine (forward and backward).

Contract (identical to `core.decomposed_linear.site_forward`):
    y = ((x V) * coef) U + d_eff * (x W^T),   coef = r * (m - d),   d_eff = r * d + (1 - r)
with `r` the routing indicator (1 = routed), `d` the delta mask, `m` the component mask which is
either drawn in the kernel epilogue from Philox counters (`StochasticSpec`) or supplied.

Launches per forward:  (1) H = x V with the mask epilogue -> A = H * coef (and H if a backward
will need it)   (2) y = A U + (d_eff * x) W^T as ONE GEMM with two K-phases sharing the accumulator.
Backward:  (3) dA = dy U^T with the backward mask epilogue -> dH = dA * coef, dci / dm
(4) dx = dH V^T + (d_eff * dy) W   (two K-phases)   (5) dV += x^T dH   (6) dU += A^T dy, both
accumulated in fp32 straight into the master gradient buffers with TMA reduce-add (split-K).
No operand is ever transposed in memory: the kernel reads MN-major tiles directly.

Weight gradients bypass autograd: `grad_V` / `grad_U` are fp32 views into the stacked masters'
`.grad`, so several uses of a site in one step (draws, terms) accumulate in place.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor

from param_decomp_b200.core.masking import SiteMask
from param_decomp_b200.ops import elementwise as ew
from param_decomp_b200.ops import native as nv


@dataclass
class SiteWeights:
    """bf16 operands of one site plus (optional) fp32 gradient sinks."""

    V: Tensor  # [d_in, C] bf16
    U: Tensor  # [C, d_out] bf16
    W: Tensor | None  # [d_out, d_in] bf16 frozen
    grad_V: Tensor | None = None  # [d_in, C] fp32, accumulated into
    grad_U: Tensor | None = None  # [C, d_out] fp32


def _split_k_for(M: int, N: int, K: int, sms: int = 148) -> int:
    """Split count for a weight-gradient GEMM (`K` = tokens): few output tiles leave SMs idle and
    an unlucky tile count wastes most of its last wave, so take the split (<= 8, >= 1024 tokens per
    split) whose tile count fills its waves best."""
    tiles = ((M + 127) // 128) * ((N + 255) // 256)
    best, best_eff = 1, 0.0
    for s in range(1, 9):
        if s > 1 and K // s < 1024:
            break
        waves = tiles * s / sms
        eff = waves / -(-tiles * s // sms)
        if eff > best_eff + 0.03:
            best, best_eff = s, eff
    return best


class _FusedSite(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, ci_or_mask: Tensor | None, delta: Tensor | None, w: SiteWeights,
                rowscale: Tensor | None, d_eff: Tensor | None, seed: int, stream: int, mask_mode: int,
                row_offset: int, need_weight_grads: bool, col_offset: int = 0,
                target_term: bool = True) -> Tensor:  # type: ignore[override]
        """`col_offset`: place of mask column 0 in the site's Philox counter space (a rank holding a column
        slice of the components draws the uniforms the whole site would). `target_term=False`: the
        `d_eff * x W^T` part is left to another rank of a component-split site."""
        if not target_term:
            d_eff = None
        N = x.shape[0]
        C, d_out = w.U.shape
        A = torch.empty(N, C, device=x.device, dtype=torch.bfloat16)
        need_bwd = x.requires_grad or (ci_or_mask is not None and ci_or_mask.requires_grad) or need_weight_grads
        need_H = need_bwd and ((ci_or_mask is not None and ci_or_mask.requires_grad)
                               or (delta is not None and delta.requires_grad))
        H = torch.empty_like(A) if need_H else None
        if ci_or_mask is None:
            # all-ones mask: coef = rowscale * (1 - delta); reuse the materialised-mask mode on a
            # broadcast row of ones (stride 0 rows are fine for the epilogue's plain loads)
            ones = torch.ones(1, C, device=x.device, dtype=torch.bfloat16).expand(N, C)
            ci_arg, mode = ones, 1
        else:
            ci_arg, mode = ci_or_mask, mask_mode
        nv.gemm(x, w.V, A, b_mn=True, epi=nv.EPI_MASK_FWD, out1=H, ci=ci_arg, delta=delta, rowscale=rowscale,
                seed=seed, rng_stream=stream, mask_mode=mode, row_offset=row_offset, philox_col0=col_offset)
        y = torch.empty(N, d_out, device=x.device, dtype=torch.bfloat16)
        if d_eff is not None:
            xd = ew.rowscale(x, d_eff)
            nv.gemm(A, w.U, y, b_mn=True, a1=xd, b1=w.W)
        else:
            nv.gemm(A, w.U, y, b_mn=True)
        ctx.save_for_backward(x, ci_or_mask, delta, rowscale, d_eff, A, H)
        ctx.w = w
        ctx.rng = (seed, stream, mode, row_offset, col_offset)
        ctx.target_term = target_term
        ctx.need_weight_grads = need_weight_grads
        ctx.ci_arg_is_ones = ci_or_mask is None
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        x, ci_or_mask, delta, rowscale, d_eff, A, H = ctx.saved_tensors
        w: SiteWeights = ctx.w
        seed, stream, mode, row_offset, col_offset = ctx.rng
        N, d_in = x.shape
        C, d_out = w.U.shape
        dy = dy.contiguous()
        need_dci = H is not None
        dH = torch.empty(N, C, device=x.device, dtype=torch.bfloat16)
        # the mask gradient leaves the kernel in the dtype autograd wants (bf16 for LM CI values)
        dci_dtype = ci_or_mask.dtype if (ci_or_mask is not None and ci_or_mask.dtype == torch.bfloat16) else torch.float32
        dci = torch.empty(N, C, device=x.device, dtype=dci_dtype) if need_dci else None
        if ctx.ci_arg_is_ones:
            ci_arg = torch.ones(1, C, device=x.device, dtype=torch.bfloat16).expand(N, C)
        else:
            ci_arg = ci_or_mask
        nv.gemm(dy, w.U, dH, epi=nv.EPI_MASK_BWD, ci=ci_arg, h=H, delta=delta, rowscale=rowscale, dci=dci,
                seed=seed, rng_stream=stream, mask_mode=mode, row_offset=row_offset, philox_col0=col_offset)
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty(N, d_in, device=x.device, dtype=torch.bfloat16)
            if d_eff is not None:
                dyd = ew.rowscale(dy, d_eff)
                nv.gemm(dH, w.V, dx, a1=dyd, b1=w.W, b1_mn=True)
            else:
                nv.gemm(dH, w.V, dx)
        if ctx.need_weight_grads:
            assert w.grad_V is not None and w.grad_U is not None
            nv.gemm(x, dH, w.grad_V, a_mn=True, b_mn=True, accumulate=True, split_k=_split_k_for(d_in, C, N))
            nv.gemm(A, dy, w.grad_U, a_mn=True, b_mn=True, accumulate=True, split_k=_split_k_for(C, d_out, N))
        d_delta = None
        if delta is not None and ctx.needs_input_grad[2]:
            # d/d(delta) = -sum_c dA*H*r + r * <dy, x W^T>; only adversarial delta sources need it
            d_delta = torch.zeros(N, device=x.device, dtype=torch.float32)
            if ctx.target_term:
                xw = torch.empty(N, d_out, device=x.device, dtype=torch.bfloat16)
                nv.gemm(x, w.W, xw)
                r = rowscale if rowscale is not None else 1.0
                d_delta = (dy.float() * xw.float()).sum(-1) * r
            if dci is not None:
                d_delta = d_delta - dci.float().sum(-1)  # mask_mode 1: dci holds dA*H*r
        dci_out = None
        if dci is not None and ctx.needs_input_grad[1]:
            dci_out = dci if dci.dtype == ci_or_mask.dtype else dci.to(ci_or_mask.dtype)
        return dx, dci_out, d_delta, None, None, None, None, None, None, None, None, None, None


def fused_site_forward(x: Tensor, w: SiteWeights, sm: SiteMask, need_weight_grads: bool,
                       target_term: bool = True) -> Tensor:
    """`x [..., d_in]` bf16 -> `[..., d_out]` bf16. Stochastic specs stay lazy (drawn in-kernel)."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    N = x2.shape[0]
    delta = None if sm.delta is None else sm.delta.reshape(N).float()
    rowscale = d_eff = None
    if sm.route is not None:
        rowscale = sm.route.reshape(N).float()
        d_eff = (rowscale * delta + (1 - rowscale)) if delta is not None else (1 - rowscale)
    elif delta is not None:
        d_eff = delta
    col_offset = 0
    if sm.stochastic is not None:
        assert sm.ci is not None
        mask_t, mode = sm.ci.reshape(N, -1), 0
        seed, stream, row_offset = sm.stochastic.seed64, sm.stochastic.stream, sm.stochastic.row_offset
        col_offset = sm.stochastic.col_offset
    else:
        mask_t = None if sm.mask is None else sm.mask.reshape(N, -1)
        mode, seed, stream, row_offset = 1, 0, 0, 0
    if mask_t is not None:
        if mask_t.dtype != torch.bfloat16:
            mask_t = mask_t.to(torch.bfloat16)
        if mask_t.stride(-1) != 1 or mask_t.stride(0) % 8 != 0 or mask_t.data_ptr() % 16 != 0:
            mask_t = mask_t.contiguous()  # (a column slice of a wider tensor is read in place through its row pitch)
    y = _FusedSite.apply(x2, mask_t, delta, w, rowscale, d_eff, seed, stream, mode, row_offset, need_weight_grads,
                         col_offset, target_term)
    return y.reshape(*lead, -1)
