"""Flash attention on sm_100a (tcgen05 QK^T and PV with TMEM accumulators). See csrc/attention_sm100.cu."""

from __future__ import annotations

import torch
from torch import Tensor

from param_decomp_b200.ops import native as nv


def supported(q: Tensor, k: Tensor, v: Tensor, segment_ids: Tensor | None) -> bool:
    """bf16, head_dim 64 or 128, sequence a multiple of 128, same length for queries and keys."""
    if not (q.is_cuda and nv.available() and nv.has_symbol("pd_flash_attention_fwd")):
        return False
    return (q.dtype == torch.bfloat16 and q.dim() == 4 and q.shape[-1] in (64, 128) and q.shape[1] % 128 == 0
            and k.shape[1] == q.shape[1] and q.shape[2] % k.shape[2] == 0)


def flash_attention(q: Tensor, k: Tensor, v: Tensor, causal: bool, segment_ids: Tensor | None = None) -> Tensor:
    from param_decomp_b200.ops.attention_impl import FlashAttention

    return FlashAttention.apply(q, k, v, causal, segment_ids)
