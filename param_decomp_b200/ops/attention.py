"""Flash attention on sm_100a (tcgen05 QK^T and PV with TMEM accumulators). See csrc/attention_sm100.cu."""

from __future__ import annotations

import torch
from torch import Tensor

from param_decomp_b200.ops import native as nv


def supported(q: Tensor, k: Tensor, v: Tensor, segment_ids: Tensor | None) -> bool:
    """The kernel covers bf16, head_dim 64 or 128, causal or full, no document segments."""
    if not nv.has_symbol("pd_flash_attention_fwd"):
        return False
    return (q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and segment_ids is None
            and q.shape[1] % 128 == 0)


def flash_attention(q: Tensor, k: Tensor, v: Tensor, causal: bool) -> Tensor:
    from param_decomp_b200.ops.attention_impl import FlashAttention

    return FlashAttention.apply(q, k, v, causal)
