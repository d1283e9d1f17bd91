"""Attention-pattern KL: `KL(softmax(S_clean) || softmax(S_masked))` per (row, head, query), mean.

`scores [B, H, T, T]` carry `-inf` at masked keys. The eager form materialises the patterns; the
reference streams 64-wide tiles with online base-2 softmax statistics so `[T, T]` never exists
(param_decomp/attention_kl.py:93-264) - the same tiling is what `csrc/attention_kl_sm100.cu` does.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor


@dataclass
class AttnQK:
    """What the streamed kernel needs instead of a `[B, H, T, T]` score tensor: the pass's post-RoPE
    queries and keys (`[B, T, H, hd]`, `[B, T, Hkv, hd]`) and its mask description."""

    q: Tensor
    k: Tensor
    causal: bool = True
    segment_ids: Tensor | None = None


def capture_scores(q: Tensor, k: Tensor, causal: bool, segment_ids: Tensor | None, fused: bool):
    """The `attn_scores` capture of a block: `AttnQK` when the streamed kernel can take it, else the
    materialised masked scores."""
    if fused and streamed_supported(q, k):
        return AttnQK(q, k, causal, segment_ids)
    from param_decomp_b200.models import ports

    s = ports.attention_scores(q, k)
    m = ports.attention_mask(q.shape[1], causal, segment_ids, q.device)
    return s if m is None else s.masked_fill(~m, float("-inf"))


def attention_pattern_kl(clean_scores, masked_scores) -> Tensor:
    if isinstance(clean_scores, AttnQK):
        assert isinstance(masked_scores, AttnQK)
        return attention_pattern_kl_streamed(clean_scores.q, clean_scores.k, masked_scores.q, masked_scores.k,
                                             masked_scores.causal, masked_scores.segment_ids)
    lc = torch.log_softmax(clean_scores.float(), dim=-1)
    lm = torch.log_softmax(masked_scores.float(), dim=-1)
    p = lc.exp()
    term = torch.where(p > 0, p * (lc - lm), torch.zeros_like(p))
    return term.sum(-1).mean()


# ---- streamed form on the tcgen05 kernels (csrc/attention_kl_sm100.cu) -------------------------------


def streamed_supported(q: Tensor, k: Tensor) -> bool:
    from param_decomp_b200.ops import native as nv

    return (q.is_cuda and q.dtype == torch.bfloat16 and q.dim() == 4 and q.shape[-1] in (64, 128)
            and q.shape[1] % 128 == 0 and k.shape[1] == q.shape[1] and nv.available()
            and nv.has_symbol("pd_attention_kl_fwd"))


class _StreamedKL(torch.autograd.Function):
    """Per-row KL `[B, H, T]` from post-RoPE `q [B,T,H,hd]`, `k [B,T,Hkv,hd]` of both passes.
    Gradients flow to the masked pass only (the clean pattern is the target)."""

    @staticmethod
    def forward(ctx, qc: Tensor, kc: Tensor, qm: Tensor, km: Tensor, causal: bool, seg: Tensor | None) -> Tensor:  # type: ignore[override]
        import ctypes as C

        from param_decomp_b200.ops import native as nv

        qc, kc, qm, km = (t.contiguous() for t in (qc, kc, qm, km))
        B, T, H, hd = qm.shape
        Hkv = km.shape[2]
        kl = torch.empty(B, H, T, device=qm.device, dtype=torch.float32)
        lc, lm = torch.empty_like(kl), torch.empty_like(kl)
        seg32 = seg.to(torch.int32).contiguous() if seg is not None else None
        lib = nv.lib()
        P, I = C.c_void_p, C.c_int
        lib.pd_attention_kl_fwd.argtypes = [P] * 8 + [I] * 6 + [P, P]
        rc = lib.pd_attention_kl_fwd(qc.data_ptr(), kc.data_ptr(), qm.data_ptr(), km.data_ptr(), kl.data_ptr(),
                                     lc.data_ptr(), lm.data_ptr(), seg32.data_ptr() if seg32 is not None else None,
                                     B, T, H, Hkv, hd, int(causal), nv.status_word().data_ptr(), nv.current_stream_ptr())
        nv.count_launch()
        if rc != 0:
            raise nv.NativeError(f"pd_attention_kl_fwd failed (code {rc})")
        ctx.save_for_backward(qc, kc, qm, km, lc, lm, seg32)
        ctx.causal = causal
        return kl

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        import ctypes as C

        from param_decomp_b200.ops import native as nv

        qc, kc, qm, km, lc, lm, seg32 = ctx.saved_tensors
        B, T, H, hd = qm.shape
        Hkv = km.shape[2]
        g = g.float().contiguous()
        dq_acc = torch.zeros(B, T, H, hd, device=qm.device, dtype=torch.float32)
        dq, dk = torch.empty_like(qm), torch.empty_like(km)
        lib = nv.lib()
        P, I = C.c_void_p, C.c_int
        lib.pd_attention_kl_bwd.argtypes = [P] * 11 + [I] * 6 + [P, P]
        rc = lib.pd_attention_kl_bwd(qc.data_ptr(), kc.data_ptr(), qm.data_ptr(), km.data_ptr(), lc.data_ptr(),
                                     lm.data_ptr(), g.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                     seg32.data_ptr() if seg32 is not None else None, B, T, H, Hkv, hd,
                                     int(ctx.causal), nv.status_word().data_ptr(), nv.current_stream_ptr())
        nv.count_launch(2)
        if rc != 0:
            raise nv.NativeError(f"pd_attention_kl_bwd failed (code {rc})")
        return None, None, dq, dk, None, None


def attention_pattern_kl_streamed(qc: Tensor, kc: Tensor, qm: Tensor, km: Tensor, causal: bool = True,
                                  segment_ids: Tensor | None = None) -> Tensor:
    """Mean over (batch, head, query) of the pattern KL, from the two passes' post-RoPE q and k."""
    return _StreamedKL.apply(qc.detach(), kc.detach(), qm, km, causal, segment_ids).mean()
