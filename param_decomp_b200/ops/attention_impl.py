"""Autograd binding of the tcgen05 flash-attention kernels (`csrc/attention_sm100.cu`).

`q [B, T, H, hd]`, `k, v [B, T, Hkv, hd]` bf16 contiguous, `hd` 64 or 128, `T % 128 == 0`; causal
and / or document-segmented masks; grouped-query attention. Forward keeps the base-2 log-sum-exp
per row; backward recomputes the probabilities tile by tile.
Parity: param_decomp/attention.py:51-137 (the dispatcher's `flash` arm).
"""

from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor

from param_decomp_b200.ops import native as nv

_configured = False


def _lib():
    global _configured
    lib = nv.lib()
    if not _configured:
        P, I = C.c_void_p, C.c_int
        lib.pd_flash_attention_fwd.argtypes = [P, P, P, P, P, P, I, I, I, I, I, I, P, P]
        lib.pd_flash_attention_bwd.argtypes = [P, P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, P, P]
        _configured = True
    return lib


def _c(t: Tensor) -> Tensor:
    return t if t.is_contiguous() else t.contiguous()


class FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q: Tensor, k: Tensor, v: Tensor, causal: bool, segment_ids: Tensor | None = None) -> Tensor:  # type: ignore[override]
        q, k, v = _c(q), _c(k), _c(v)
        B, T, H, hd = q.shape
        Hkv = k.shape[2]
        out = torch.empty_like(q)
        lse = torch.empty(B, H, T, device=q.device, dtype=torch.float32)
        seg = None
        if segment_ids is not None:
            seg = _c(segment_ids.to(torch.int32))
        rc = _lib().pd_flash_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                           seg.data_ptr() if seg is not None else None, B, T, H, Hkv, hd, int(causal),
                                           nv.status_word().data_ptr(), nv.current_stream_ptr())
        nv.count_launch()
        if rc != 0:
            raise nv.NativeError(f"pd_flash_attention_fwd failed (code {rc})")
        ctx.save_for_backward(q, k, v, out, lse, seg)
        ctx.causal = causal
        return out

    @staticmethod
    def backward(ctx, d_out: Tensor):  # type: ignore[override]
        q, k, v, out, lse, seg = ctx.saved_tensors
        d_out = _c(d_out)
        B, T, H, hd = q.shape
        Hkv = k.shape[2]
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        delta = torch.empty(B, H, T, device=q.device, dtype=torch.float32)
        dq_acc = torch.zeros(B, T, H, hd, device=q.device, dtype=torch.float32)
        rc = _lib().pd_flash_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), d_out.data_ptr(),
                                           lse.data_ptr(), delta.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(),
                                           dk.data_ptr(), dv.data_ptr(), seg.data_ptr() if seg is not None else None,
                                           B, T, H, Hkv, hd, int(ctx.causal), nv.status_word().data_ptr(),
                                           nv.current_stream_ptr())
        nv.count_launch(3)
        if rc != 0:
            raise nv.NativeError(f"pd_flash_attention_bwd failed (code {rc})")
        return dq, dk, dv, None, None
