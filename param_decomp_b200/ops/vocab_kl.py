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


class _StreamedKLFromHidden(torch.autograd.Function):
    """The same loss without any `[positions, vocab]` tensor: positions are processed in chunks of `rows`; per
    chunk the clean and masked logits are formed (two tcgen05 GEMMs into re-used buffers), one kernel pass gives
    the chunk's KL and `softmax(masked) - softmax(clean)`, and the chunk's gradient with respect to the masked
    hidden state, `dlogits @ head / n`, is taken at once - so the backward pass only scales a `[positions, d]`
    tensor. Peak extra memory is `3 x rows x vocab` bf16 whatever the batch; the price is one more logits GEMM
    per call for the clean side (param_decomp/targets/losses.py:63-162 streams vocabulary chunks with online
    softmax accumulators to the same end)."""

    @staticmethod
    def forward(ctx, hc: Tensor, hm: Tensor, head: Tensor, rows: int) -> Tensor:  # type: ignore[override]
        n, d = hm.shape
        V = head.shape[0]
        vp = (V + 7) // 8 * 8
        rows = max(128, min(rows, n))
        lc_buf = torch.empty(rows, vp, device=hm.device, dtype=torch.bfloat16)
        lm_buf = torch.empty(rows, vp, device=hm.device, dtype=torch.bfloat16)
        want_grad = hm.requires_grad
        dl_buf = torch.empty(rows, vp, device=hm.device, dtype=torch.bfloat16) if want_grad else None
        dh = torch.empty(n, d, device=hm.device, dtype=torch.bfloat16) if want_grad else None
        total = torch.zeros((), device=hm.device, dtype=torch.float32)
        hc, hm = hc.contiguous(), hm.contiguous()
        for s in range(0, n, rows):
            r = min(rows, n - s)
            lc, lm = lc_buf[:r, :V], lm_buf[:r, :V]
            nv.gemm(hc[s:s + r], head, lc)
            nv.gemm(hm[s:s + r], head, lm)
            kl, dlm = vocab_kl_rows(lc, lm, want_grad=want_grad, grad_out=dl_buf)
            total = total + kl.sum()
            if want_grad:
                nv.gemm(dlm, head, dh[s:s + r], b_mn=True, alpha=1.0 / n)
        ctx.save_for_backward(dh)
        return total / n

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        (dh,) = ctx.saved_tensors
        return None, dh * g.to(dh.dtype), None, None


def kl_from_hidden_streamed(hc: Tensor, hm: Tensor, head: Tensor, rows: int) -> Tensor:
    """`hc`, `hm [n, d]` bf16 final hidden states (clean, masked), `head [V, d]`; `rows` positions per chunk."""
    return _StreamedKLFromHidden.apply(hc, hm, head, rows)
