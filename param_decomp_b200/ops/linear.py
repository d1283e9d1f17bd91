"""Autograd wrappers that put the target's linears and the decomposed sites on the tcgen05 engine."""

from __future__ import annotations

from dataclasses import replace

import torch
from torch import Tensor

from param_decomp_b200.core.components import ComputeWeights
from param_decomp_b200.core.masking import SiteMask
from param_decomp_b200.ops import native as nv
from param_decomp_b200.ops.site_linear import SiteWeights, fused_site_forward


class _FrozenLinear(torch.autograd.Function):
    """`y = x W^T` with a frozen `W [d_out, d_in]`: the backward is `dx = dy W` (W read MN-major)."""

    @staticmethod
    def forward(ctx, x: Tensor, W: Tensor) -> Tensor:  # type: ignore[override]
        y = torch.empty(x.shape[0], W.shape[0], device=x.device, dtype=torch.bfloat16)
        nv.gemm(x, W, y)
        ctx.save_for_backward(W)
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        (W,) = ctx.saved_tensors
        dx = torch.empty(dy.shape[0], W.shape[1], device=dy.device, dtype=torch.bfloat16)
        nv.gemm(dy.contiguous(), W, dx, b_mn=True)
        return dx, None


def linear(x: Tensor, W: Tensor) -> Tensor:
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    if x2.requires_grad:
        y = _FrozenLinear.apply(x2, W)
    else:
        y = torch.empty(x2.shape[0], W.shape[0], device=x.device, dtype=torch.bfloat16)
        nv.gemm(x2, W, y)
    return y.reshape(*lead, -1)


def site(x: Tensor, weights: ComputeWeights, name: str, W: Tensor, sm: SiteMask) -> Tensor:
    V, U = weights.site(name)
    sw = SiteWeights(V, U, W, weights.grad_V.get(name), weights.grad_U.get(name))
    return fused_site_forward(x, sw, sm, need_weight_grads=weights.direct_grads)


def site_split(x: Tensor, weights: ComputeWeights, name: str, W: Tensor, sm: SiteMask, group) -> Tensor:
    """The site with its component axis split over `group` (this rank holds `V[:, C/W]`, `U[C/W, :]`): the
    rank's columns of the replicated mask, the fused kernels on the local slice, partial outputs summed
    over the group; the first rank carries the target term."""
    import torch.distributed as dist

    from param_decomp_b200.parallel.group_ops import ReduceFromGroup, copy_to_group

    V, U = weights.site(name)
    sw = SiteWeights(V, U, W, weights.grad_V.get(name), weights.grad_U.get(name))
    sm = sm.column_shard(group)
    if sm.delta is not None and sm.delta.requires_grad:
        sm = replace(sm, delta=copy_to_group(sm.delta, group))
    part = fused_site_forward(copy_to_group(x, group), sw, sm, need_weight_grads=weights.direct_grads,
                              target_term=dist.get_rank(group) == 0)
    return ReduceFromGroup.apply(part, group)


class _BmmBias(torch.autograd.Function):
    """`y[g] = x[g] W[g] + b[g]` for a stack of `g` independent linears with TRAINABLE fp32 masters.

    bf16 operands on the batched tcgen05 kernel, fp32 weight/bias gradients. `x [g, N, K]` bf16,
    `W [g, K, M]` fp32, `b [g, 1, M]` fp32 -> `[g, N, M]` bf16.
    """

    @staticmethod
    def forward(ctx, x: Tensor, W: Tensor, b: Tensor) -> Tensor:  # type: ignore[override]
        from param_decomp_b200.ops.elementwise import cast_bf16

        Wb = cast_bf16(W.detach().contiguous())
        g, N, K = x.shape
        M = W.shape[-1]
        x = x.contiguous()
        y = torch.empty(g, N, M, device=x.device, dtype=torch.bfloat16)
        nv.gemm(x, Wb, y, b_mn=True, bias=b.detach().reshape(g, M).contiguous())
        ctx.save_for_backward(x, Wb)
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        x, Wb = ctx.saved_tensors
        dy = dy.contiguous()
        g, N, K = x.shape
        M = Wb.shape[-1]
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            nv.gemm(dy, Wb, dx)  # Wb [g, K, M] read as the K-major B operand of dx = dy W^T
        dW = torch.zeros(g, K, M, device=x.device, dtype=torch.float32)
        tiles = ((K + 127) // 128) * ((M + 255) // 256) * g
        split = max(1, min(148 // max(tiles, 1), N // 512))
        nv.gemm(x, dy, dW, a_mn=True, b_mn=True, accumulate=True, split_k=split)
        from param_decomp_b200.ops.elementwise import colsum_bf16

        db = colsum_bf16(dy).unsqueeze(1) if M % 8 == 0 else dy.float().sum(1, keepdim=True)
        return dx, dW, db


def bmm_bias(x: Tensor, W: Tensor, b: Tensor) -> Tensor:
    return _BmmBias.apply(x, W, b)


class _TrainableLinear(torch.autograd.Function):
    """`y = x W^T + b` for ONE linear with trainable fp32 masters (`W [d_out, d_in]`, torch's layout): bf16
    operands on the tcgen05 kernel, fp32 weight / bias gradients, the transformer CI functions' linears."""

    @staticmethod
    def forward(ctx, x: Tensor, W: Tensor, b: Tensor | None) -> Tensor:  # type: ignore[override]
        from param_decomp_b200.ops.elementwise import cast_bf16

        Wb = cast_bf16(W.detach().contiguous())
        y = torch.empty(x.shape[0], W.shape[0], device=x.device, dtype=torch.bfloat16)
        nv.gemm(x, Wb, y, bias=None if b is None else b.detach().float().contiguous())
        ctx.save_for_backward(x, Wb)
        ctx.has_bias = b is not None
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        from param_decomp_b200.ops.elementwise import colsum_bf16

        x, Wb = ctx.saved_tensors
        dy = dy.contiguous()
        N, d_in = x.shape
        d_out = Wb.shape[0]
        dx = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            nv.gemm(dy, Wb, dx, b_mn=True)  # dx = dy W
        dW = torch.zeros(d_out, d_in, device=x.device, dtype=torch.float32)
        tiles = ((d_out + 127) // 128) * ((d_in + 255) // 256)
        nv.gemm(dy, x, dW, a_mn=True, b_mn=True, accumulate=True, split_k=max(1, min(148 // max(tiles, 1), N // 512)))
        db = colsum_bf16(dy) if ctx.has_bias else None
        return dx, dW, db


def trainable_linear_supported(x: Tensor, W: Tensor) -> bool:
    return x.is_cuda and W.shape[0] % 8 == 0 and W.shape[1] % 8 == 0


def trainable_linear(x: Tensor, W: Tensor, b: Tensor | None) -> Tensor:
    """`x [..., d_in]` (any float dtype; computed in bf16) -> `[..., d_out]` bf16."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.dtype != torch.bfloat16:
        x2 = x2.to(torch.bfloat16)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    return _TrainableLinear.apply(x2, W, b).reshape(*lead, -1)
