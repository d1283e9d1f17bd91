"""Fused AdamW with device-side global-norm clipping (no host synchronisation in the step)."""

from __future__ import annotations

import torch
from torch import Tensor

from param_decomp_b200.ops import native as nv
from param_decomp_b200.ops.elementwise import _check, _lib, _s


def grad_norm_and_scale(grads: list[Tensor], max_norm: float | None) -> tuple[Tensor, Tensor]:
    """Returns device scalars `(norm, scale)`, `scale = min(max_norm / (norm + 1e-6), 1)`."""
    dev = grads[0].device
    buf = torch.zeros(3, device=dev, dtype=torch.float32)  # sumsq, scale, norm
    lib = _lib()
    for g in grads:
        assert g.dtype == torch.float32 and g.is_contiguous()
        _check(lib.pd_sumsq(g.data_ptr(), g.numel(), buf.data_ptr(), _s()), "sumsq")
    _check(lib.pd_clip_scale(buf.data_ptr(), float(max_norm) if max_norm is not None else 0.0,
                             buf[1:].data_ptr(), buf[2:].data_ptr(), _s()), "clip_scale")
    return buf[2], buf[1]


def adamw_step(params: list[Tensor], grads: list[Tensor], mus: list[Tensor], nus: list[Tensor], *, lr: float,
               b1: float, b2: float, eps: float, wd: float, bc1: float, bc2: float, grad_scale: Tensor) -> None:
    lib = _lib()
    assert grad_scale.dtype == torch.float32 and grad_scale.is_cuda
    for p, g, m, v in zip(params, grads, mus, nus):
        assert p.is_contiguous() and g.is_contiguous() and p.dtype == torch.float32
        _check(lib.pd_adamw(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), lr, b1, b2, eps, wd,
                            bc1, bc2, grad_scale.data_ptr(), _s()), "adamw")
