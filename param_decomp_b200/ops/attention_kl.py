"""Attention-pattern KL: `KL(softmax(S_clean) || softmax(S_masked))` per (row, head, query), mean.

`scores [B, H, T, T]` carry `-inf` at masked keys. The eager form materialises the patterns; the
reference streams 64-wide tiles with online base-2 softmax statistics so `[T, T]` never exists
(param_decomp/attention_kl.py:93-264) - the same tiling is what `csrc/attention_kl_sm100.cu` does.
"""

from __future__ import annotations

import torch
from torch import Tensor


def attention_pattern_kl(clean_scores: Tensor, masked_scores: Tensor) -> Tensor:
    lc = torch.log_softmax(clean_scores.float(), dim=-1)
    lm = torch.log_softmax(masked_scores.float(), dim=-1)
    p = lc.exp()
    term = torch.where(p > 0, p * (lc - lm), torch.zeros_like(p))
    return term.sum(-1).mean()
