"""Flash attention on sm_100a (tcgen05 QK^T and PV with TMEM accumulators). See csrc/attention_sm100.cu.

The kernel itself takes bf16 `[B, T, H, hd]` with `hd` 64 or 128 and `T % 128 == 0`. Other shapes are brought
to that form here instead of being handed to a library kernel: the head dimension is zero-padded to 64 / 128
(scores are unchanged; the query is pre-scaled so the kernel's `1 / sqrt(hd_padded)` becomes `1 / sqrt(hd)`),
the sequence is padded to a multiple of 128 with positions of their own segment (`-1`) that no real query
attends. Head dimensions above 128 are refused.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F
from torch import Tensor

from param_decomp_b200.ops import native as nv


def supported(q: Tensor, k: Tensor, v: Tensor, segment_ids: Tensor | None) -> bool:
    """Shapes the kernel takes as they are: bf16, head_dim 64 or 128, sequence a multiple of 128."""
    if not (q.is_cuda and nv.available() and nv.has_symbol("pd_flash_attention_fwd")):
        return False
    return (q.dtype == torch.bfloat16 and q.dim() == 4 and q.shape[-1] in (64, 128) and q.shape[1] % 128 == 0
            and k.shape[1] == q.shape[1] and q.shape[2] % k.shape[2] == 0)


def flash_attention(q: Tensor, k: Tensor, v: Tensor, causal: bool, segment_ids: Tensor | None = None) -> Tensor:
    from param_decomp_b200.ops.attention_impl import FlashAttention

    if not (q.is_cuda and nv.available()):
        raise nv.NativeError("flash attention needs a CUDA device and the native library")
    B, T, H, hd = q.shape
    if hd > 128 or k.shape[1] != T or H % k.shape[2] != 0:
        raise NotImplementedError(f"flash attention: head_dim {hd} / shapes {tuple(q.shape)}, {tuple(k.shape)} "
                                  "are outside the kernel's range (head_dim <= 128, equal lengths, grouped heads)")
    dtype = q.dtype
    if dtype != torch.bfloat16:
        q, k, v = q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16)
    hd_p = 64 if hd <= 64 else 128
    if hd_p != hd:
        q = F.pad(q * math.sqrt(hd_p / hd), (0, hd_p - hd))
        k, v = F.pad(k, (0, hd_p - hd)), F.pad(v, (0, hd_p - hd))
    T_p = (T + 127) // 128 * 128
    if T_p != T:
        pad = (0, 0, 0, 0, 0, T_p - T)  # (hd, heads, T)
        q, k, v = F.pad(q, pad), F.pad(k, pad), F.pad(v, pad)
        if segment_ids is None:
            segment_ids = torch.zeros(B, T, dtype=torch.int32, device=q.device)
        segment_ids = F.pad(segment_ids.to(torch.int32), (0, T_p - T), value=-1)
    out = FlashAttention.apply(q, k, v, causal, segment_ids)
    if T_p != T or hd_p != hd:
        out = out[:, :T, :, :hd]
    return out if dtype == torch.bfloat16 else out.to(dtype)
