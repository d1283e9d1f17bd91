"""Leaky-hard sigmoids that turn CI pre-activations into importances in [0, 1].

`lower` (used for masks): forward `clamp(x, 0, 1)`; backward passes the gradient on (0, 1], blocks
it above 1, and below 0 lets through `alpha * g` only when `g < 0` (i.e. only when descent would
push the pre-activation up, back into range). `upper` (used by the minimality loss): plain autodiff
of `x > 1 ? 1 + alpha (x - 1) : clamp(x, 0, 1)`.

Parity: param_decomp/core/ci_fn/squashing.py:8-45; nano_param_decomp/run.py:143-188.
"""

from __future__ import annotations

import torch
from torch import Tensor

LEAKY_ALPHA = 0.01


class _LowerLeakyHardSigmoid(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, alpha: float) -> Tensor:  # type: ignore[override]
        ctx.save_for_backward(x)
        ctx.alpha = alpha
        return x.clamp(0.0, 1.0)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        (x,) = ctx.saved_tensors
        below = x <= 0
        inside = (x > 0) & (x <= 1)
        leak = torch.where(g < 0, ctx.alpha * g, torch.zeros_like(g))
        return torch.where(inside, g, torch.where(below, leak, torch.zeros_like(g))), None


def lower_leaky_hard_sigmoid(x: Tensor, alpha: float = LEAKY_ALPHA) -> Tensor:
    return _LowerLeakyHardSigmoid.apply(x, alpha)


def upper_leaky_hard_sigmoid(x: Tensor, alpha: float = LEAKY_ALPHA) -> Tensor:
    return torch.where(x > 1, 1 + alpha * (x - 1), x.clamp(0.0, 1.0))


def symmetric_leaky_hard_sigmoid(x: Tensor, alpha: float = LEAKY_ALPHA) -> Tensor:
    """Leaks on both sides with plain autodiff (available for ablations)."""
    return torch.where(x > 1, 1 + alpha * (x - 1), torch.where(x < 0, alpha * x, x))
