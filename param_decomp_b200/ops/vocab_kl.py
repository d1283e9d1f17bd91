"""Vocabulary-wide KL reconstruction loss from final hidden states.

`KL(softmax(h_c W^T) || softmax(h_m W^T))` averaged over positions, computed per chunk of positions
with both logit products on the tcgen05 engine and the chunk recomputed in backward, so logits
`[positions, vocab]` exist only one chunk at a time (the reference streams vocab chunks with online
softmax accumulators for the same reason: param_decomp/targets/losses.py:102-162).
"""

from __future__ import annotations

import torch
from torch import Tensor

from param_decomp_b200.ops import native as nv


def _padded(n: int, v: int, device) -> Tensor:
    """`[n, v]` bf16 view whose row pitch is a multiple of 16 bytes (TMA stores need it)."""
    vp = (v + 7) // 8 * 8
    return torch.empty(n, vp, device=device, dtype=torch.bfloat16)[:, :v]


def _logits(h: Tensor, head: Tensor) -> Tensor:
    out = _padded(h.shape[0], head.shape[0], h.device)
    nv.gemm(h.contiguous(), head, out)
    return out


class _ChunkKL(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hc: Tensor, hm: Tensor, head: Tensor) -> Tensor:  # type: ignore[override]
        lc, lm = _logits(hc, head).float(), _logits(hm, head).float()
        logp_c = torch.log_softmax(lc, dim=-1)
        logp_m = torch.log_softmax(lm, dim=-1)
        ctx.save_for_backward(hc, hm, head)
        return (logp_c.exp() * (logp_c - logp_m)).sum()

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        hc, hm, head = ctx.saved_tensors
        p_c = torch.softmax(_logits(hc, head).float(), dim=-1)
        p_m = torch.softmax(_logits(hm, head).float(), dim=-1)
        dlogits = _padded(hm.shape[0], head.shape[0], hm.device)
        dlogits.copy_((p_m - p_c) * g)
        dh = torch.empty_like(hm)
        nv.gemm(dlogits, head, dh, b_mn=True)  # [n, V] x [V, d]: head read MN-major
        return None, dh, None


def kl_from_hidden(hc: Tensor, hm: Tensor, head: Tensor, chunk: int) -> Tensor:
    n = hc.shape[0]
    total = torch.zeros((), device=hm.device, dtype=torch.float32)
    for s in range(0, n, chunk):
        total = total + _ChunkKL.apply(hc[s:s + chunk], hm[s:s + chunk], head)
    return total / n
