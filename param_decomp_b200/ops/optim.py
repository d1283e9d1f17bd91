"""Fused AdamW with device-side global-norm clipping (no host synchronisation in the step)."""

from __future__ import annotations

import torch
from torch import Tensor

import ctypes as C

from param_decomp_b200.ops.elementwise import _check, _lib, _s

_REFS: dict[tuple, Tensor] = {}


def tensor_refs(params: list[Tensor], grads: list[Tensor], mus: list[Tensor] | None = None,
                nus: list[Tensor] | None = None) -> Tensor:
    """Device table `{p, g, m, v, n}` per leaf for the multi-tensor kernels, built once per set of buffers
    (optimizer state and the direct-gradient buffers keep their addresses from step to step)."""
    key = tuple((p.data_ptr(), g.data_ptr(), m.data_ptr() if m is not None else 0, v.data_ptr() if v is not None else 0,
                 p.numel()) for p, g, m, v in zip(params, grads, mus or [None] * len(params), nus or [None] * len(params)))
    t = _REFS.get(key)
    if t is None:
        for p, g in zip(params, grads):
            assert p.dtype == torch.float32 and g.dtype == torch.float32 and p.is_contiguous() and g.is_contiguous()
        if len(_REFS) > 64:
            _REFS.clear()
        t = torch.tensor([list(k) for k in key], dtype=torch.int64).to(params[0].device)
        _REFS[key] = t
    return t


def grad_norm_and_scale_multi(params: list[Tensor], grads: list[Tensor], max_norm: float | None) -> tuple[Tensor, Tensor]:
    """As `grad_norm_and_scale`, with one launch for the whole group."""
    refs = tensor_refs(params, grads)
    buf = torch.zeros(3, device=grads[0].device, dtype=torch.float32)  # sumsq, scale, norm
    lib = _lib()
    lib.pd_sumsq_multi.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    _check(lib.pd_sumsq_multi(refs.data_ptr(), len(grads), buf.data_ptr(), _s()), "sumsq_multi")
    _check(lib.pd_clip_scale(buf.data_ptr(), float(max_norm) if max_norm is not None else 0.0,
                             buf[1:].data_ptr(), buf[2:].data_ptr(), _s()), "clip_scale")
    return buf[2], buf[1]


def adamw_step_multi(params: list[Tensor], grads: list[Tensor], mus: list[Tensor], nus: list[Tensor], *, lr: float,
                     b1: float, b2: float, eps: float, wd: float, bc1: float, bc2: float, grad_scale: Tensor,
                     hyper: Tensor | None = None) -> None:
    """One launch for every leaf of the group. `hyper` (`[3]` fp32 on the device: lr, 1/bc1, 1/bc2) overrides the
    by-value numbers at run time (a slot of the step-scalar table)."""
    refs = tensor_refs(params, grads, mus, nus)
    lib = _lib()
    F = C.c_float
    lib.pd_adamw_multi.argtypes = [C.c_void_p, C.c_int, F, F, F, F, F, F, F, C.c_void_p, C.c_void_p, C.c_void_p]
    _check(lib.pd_adamw_multi(refs.data_ptr(), len(params), lr, b1, b2, eps, wd, bc1, bc2,
                              hyper.data_ptr() if hyper is not None else None, grad_scale.data_ptr(), _s()),
           "adamw_multi")


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
