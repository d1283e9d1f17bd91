"""Vocabulary-wide KL reconstruction loss from final hidden states on the fused backend.

Clean logits are formed once per step (`clean_logits`) and kept in bf16; each masked forward forms
its logits with one tcgen05 GEMM, one kernel pass computes the per-position KL *and* the gradient
`softmax(masked) - softmax(clean)`, and the backward is a single GEMM `dlogits @ head` whose
`alpha` carries the upstream gradient over the number of positions. Nothing is recomputed and no
fp32 `[positions, vocab]` tensor exists. (The reference streams vocabulary chunks with online
softmax accumulators to bound memory, param_decomp/targets/losses.py:102-162; a B200 holds the bf16
logits of the whole batch, so time is spent on one GEMM + one bandwidth pass instead.)
"""

from __future__ import annotations

import torch
from torch import Tensor

from param_decomp_b200.ops import native as nv
from param_decomp_b200.ops.elementwise import vocab_kl_rows


def padded_logits(h: Tensor, head: Tensor) -> Tensor:
    """`h [n, d] @ head[V, d]^T -> [n, V]` bf16 view with a 16-byte-multiple row pitch."""
    n, V = h.shape[0], head.shape[0]
    vp = (V + 7) // 8 * 8
    out = torch.empty(n, vp, device=h.device, dtype=torch.bfloat16)[:, :V]
    nv.gemm(h.contiguous(), head, out)
    return out


class _KLFromLogits(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hm: Tensor, clean_logits: Tensor, head: Tensor) -> Tensor:  # type: ignore[override]
        lm = padded_logits(hm, head)
        kl, dlm = vocab_kl_rows(clean_logits, lm, want_grad=hm.requires_grad)
        ctx.save_for_backward(dlm, head)
        ctx.n = hm.shape[0]
        return kl.mean()

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        dlm, head = ctx.saved_tensors
        dh = torch.empty(ctx.n, head.shape[1], device=head.device, dtype=torch.bfloat16)
        nv.gemm(dlm, head, dh, b_mn=True, alpha=1.0 / ctx.n)
        return dh * g.to(dh.dtype), None, None  # upstream gradient stays on the device (no host sync)


def kl_from_hidden(clean_logits: Tensor, hm: Tensor, head: Tensor) -> Tensor:
    return _KLFromLogits.apply(hm, clean_logits, head)
