"""Bindings of the gated-delta-rule and causal-conv kernels (`csrc/delta_rule.cu`).

The recurrence runs in fp32 with the state on chip; the backward replays 64-token chunks from
checkpointed states. Parity: param_decomp/target_ports/qwen3_5_moe.py:65-74,89-158.
"""

from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor

from param_decomp_b200.ops import native as nv

_SHAPES = {(64, 64), (128, 128), (64, 128), (32, 32)}
_configured = False


def _lib():
    global _configured
    lib = nv.lib()
    if not _configured:
        P, I = C.c_void_p, C.c_int
        lib.pd_delta_rule_fwd.argtypes = [P] * 7 + [I] * 5 + [P]
        lib.pd_delta_rule_bwd.argtypes = [P] * 13 + [I] * 5 + [P]
        lib.pd_conv1d_silu_fwd.argtypes = [P, P, P, I, I, I, I, P]
        lib.pd_conv1d_silu_bwd.argtypes = [P, P, P, P, P, I, I, I, I, P]
        _configured = True
    return lib


def supported(q: Tensor, v: Tensor) -> bool:
    return (q.is_cuda and nv.available() and nv.has_symbol("pd_delta_rule_fwd")
            and (q.shape[-1], v.shape[-1]) in _SHAPES)


def conv_supported(x: Tensor, w: Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.shape[-1] <= 8 and nv.available()
            and nv.has_symbol("pd_conv1d_silu_fwd"))


class _DeltaRule(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor) -> Tensor:  # type: ignore[override]
        q, k, v, g, beta = (t.float().contiguous() for t in (q, k, v, g, beta))
        B, T, H, dk = q.shape
        dv = v.shape[-1]
        o = torch.empty_like(v)
        need = any(ctx.needs_input_grad)
        ckpt = torch.empty(B * H, (T + 63) // 64, dk, dv, device=q.device, dtype=torch.float32) if need else None
        rc = _lib().pd_delta_rule_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                                      o.data_ptr(), ckpt.data_ptr() if need else None, B, T, H, dk, dv,
                                      nv.current_stream_ptr())
        nv.count_launch()
        if rc != 0:
            raise nv.NativeError(f"pd_delta_rule_fwd failed (code {rc})")
        if need:
            ctx.save_for_backward(q, k, v, g, beta, ckpt)
        return o

    @staticmethod
    def backward(ctx, d_o: Tensor):  # type: ignore[override]
        q, k, v, g, beta, ckpt = ctx.saved_tensors
        B, T, H, dk = q.shape
        dv = v.shape[-1]
        d_o = d_o.float().contiguous()
        dq, dk_, dv_ = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dg, dbeta = torch.empty_like(g), torch.empty_like(beta)
        scratch = torch.empty(B * H, 64, dk, dv, device=q.device, dtype=torch.float32)
        rc = _lib().pd_delta_rule_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
                                      d_o.data_ptr(), ckpt.data_ptr(), scratch.data_ptr(), dq.data_ptr(), dk_.data_ptr(),
                                      dv_.data_ptr(), dg.data_ptr(), dbeta.data_ptr(), B, T, H, dk, dv,
                                      nv.current_stream_ptr())
        nv.count_launch()
        if rc != 0:
            raise nv.NativeError(f"pd_delta_rule_bwd failed (code {rc})")
        return dq, dk_, dv_, dg, dbeta


def gated_delta_rule(q: Tensor, k: Tensor, v: Tensor, g: Tensor, beta: Tensor) -> Tensor:
    """Inputs as the recurrence sees them: q already l2-normalised and scaled, k l2-normalised, fp32."""
    return _DeltaRule.apply(q, k, v, g, beta)


class _ConvSilu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, w: Tensor) -> Tensor:  # type: ignore[override]
        x = x.contiguous()
        wb = w.to(torch.bfloat16).contiguous()
        B, T, D = x.shape
        y = torch.empty_like(x)
        rc = _lib().pd_conv1d_silu_fwd(x.data_ptr(), wb.data_ptr(), y.data_ptr(), B, T, D, wb.shape[1],
                                       nv.current_stream_ptr())
        nv.count_launch()
        if rc != 0:
            raise nv.NativeError(f"pd_conv1d_silu_fwd failed (code {rc})")
        ctx.save_for_backward(x, wb)
        ctx.w_dtype = w.dtype
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        x, wb = ctx.saved_tensors
        B, T, D = x.shape
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dw = torch.zeros(D, wb.shape[1], device=x.device, dtype=torch.float32)
        rc = _lib().pd_conv1d_silu_bwd(x.data_ptr(), wb.data_ptr(), dy.data_ptr(), dx.data_ptr(), dw.data_ptr(), B, T,
                                       D, wb.shape[1], nv.current_stream_ptr())
        nv.count_launch()
        if rc != 0:
            raise nv.NativeError(f"pd_conv1d_silu_bwd failed (code {rc})")
        return dx, dw.to(ctx.w_dtype)


def causal_conv1d_silu(x: Tensor, w: Tensor) -> Tensor:
    """`x [B, T, D]` bf16, `w [D, K]`: per-channel causal filter then SiLU."""
    return _ConvSilu.apply(x, w)
