"""Bindings + autograd wrappers of the bandwidth-bound kernels (`csrc/elementwise.cu`)."""

from __future__ import annotations

import ctypes as C

import torch
from torch import Tensor

from param_decomp_b200.ops import native as nv

_configured = False


def _lib():
    global _configured
    lib = nv.lib()
    if not _configured:
        P, LL, I, F = C.c_void_p, C.c_longlong, C.c_int, C.c_float
        lib.pd_sumsq.argtypes = [P, LL, P, P]
        lib.pd_clip_scale.argtypes = [P, F, P, P, P]
        lib.pd_adamw.argtypes = [P, P, P, P, LL, F, F, F, F, F, F, F, P, P]
        lib.pd_cast_bf16.argtypes = [P, P, LL, P]
        lib.pd_rmsnorm_fwd.argtypes = [P, P, P, P, LL, I, F, P]
        lib.pd_rmsnorm_bwd.argtypes = [P, P, P, P, P, LL, I, P]
        lib.pd_rope.argtypes = [P, P, P, LL, I, I, I, I, P]
        lib.pd_rope_to.argtypes = [P, P, P, P, LL, I, I, I, I, P]
        lib.pd_swiglu_fwd.argtypes = [P, P, P, LL, P]
        lib.pd_swiglu_bwd.argtypes = [P, P, P, P, P, LL, P]
        lib.pd_rowscale.argtypes = [P, P, P, LL, I, P]
        lib.pd_ci_squash.argtypes = [P, P, P, LL, F, P]
        _configured = True
    return lib


def _check(rc: int, what: str) -> None:
    nv.count_launch()
    if rc != 0:
        raise nv.NativeError(f"{what} failed to launch (code {rc})")


def _s() -> int:
    return nv.current_stream_ptr()


def _scalar_arg(x) -> tuple[float, int | None]:
    """A scalar kernel argument given as a python number or as a 0-d fp32 device tensor (a slot of the
    step-scalar table): `(by-value placeholder, device address or None)`."""
    if isinstance(x, Tensor):
        assert x.dtype == torch.float32 and x.is_cuda and x.numel() == 1
        return 0.0, x.data_ptr()
    return float(x), None


def cast_bf16(src: Tensor, out: Tensor | None = None) -> Tensor:
    assert src.dtype == torch.float32 and src.is_contiguous()
    out = out if out is not None else torch.empty_like(src, dtype=torch.bfloat16)
    _check(_lib().pd_cast_bf16(src.data_ptr(), out.data_ptr(), src.numel(), _s()), "cast_bf16")
    return out


def rowscale(x: Tensor, s: Tensor) -> Tensor:
    """`y[r, :] = x[r, :] * s[r]` (bf16 rows, fp32 scales), one vectorised pass."""
    assert x.dtype == torch.bfloat16 and s.dtype == torch.float32
    x = x if x.is_contiguous() else x.contiguous()
    s = s if s.is_contiguous() else s.contiguous()
    if x.shape[1] % 8 != 0 or x.data_ptr() % 16 != 0:
        return (x.float() * s[:, None]).to(torch.bfloat16)
    y = torch.empty_like(x)
    _check(_lib().pd_rowscale(x.data_ptr(), s.data_ptr(), y.data_ptr(), x.shape[0], x.shape[1], _s()), "rowscale")
    return y


def rows_expand(x: Tensor, rowmap: Tensor, w: Tensor | None, n_rows: int, k: int, rep: int, use_slot: bool) -> Tensor:
    """`out[r] = w[token, slot] * x[token * rep + slot * use_slot]` for the `(token, slot)` that `rowmap`
    gives padded row `r`; zero rows where the map holds token -1. bf16 rows, fp32 weights."""
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and rowmap.dtype == torch.int32 and rowmap.shape[1] == 4
    out = torch.empty(n_rows, x.shape[1], device=x.device, dtype=torch.bfloat16)
    lib = _lib()
    lib.pd_rows_expand.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int,
                                   C.c_int, C.c_int, C.c_void_p]
    _check(lib.pd_rows_expand(x.data_ptr(), rowmap.data_ptr(), w.data_ptr() if w is not None else None, out.data_ptr(),
                              n_rows, x.shape[1], k, rep, int(use_slot), _s()), "rows_expand")
    return out


def rows_combine(padded: Tensor, pos: Tensor, w: Tensor | None, tokens: int, k: int,
                 bgroup: Tensor | None = None) -> Tensor:
    """`y[n] = sum_s w[n, s] * padded[pos[n * k + s]]` (fp32 accumulation, bf16 rows). `bgroup` (int32, one
    entry per 128 rows): jobs whose row block has owner -1 are skipped (rows this rank never computed)."""
    assert padded.dtype == torch.bfloat16 and padded.is_contiguous() and pos.dtype == torch.int64
    assert pos.numel() == tokens * k
    y = torch.empty(tokens, padded.shape[1], device=padded.device, dtype=torch.bfloat16)
    lib = _lib()
    lib.pd_rows_combine.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int,
                                    C.c_int, C.c_void_p]
    _check(lib.pd_rows_combine(padded.data_ptr(), pos.data_ptr(), w.data_ptr() if w is not None else None,
                               bgroup.data_ptr() if bgroup is not None else None, y.data_ptr(), tokens,
                               padded.shape[1], k, _s()), "rows_combine")
    return y


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: Tensor, w: Tensor | None, eps: float) -> Tensor:  # type: ignore[override]
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        rows, d = x2.shape
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        _check(_lib().pd_rmsnorm_fwd(x2.data_ptr(), w.data_ptr() if w is not None else None, y.data_ptr(),
                                     rstd.data_ptr(), rows, d, eps, _s()), "rmsnorm_fwd")
        ctx.save_for_backward(x2, w, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        x2, w, rstd = ctx.saved_tensors
        dy2 = dy.reshape(x2.shape)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dx = torch.empty_like(x2)
        _check(_lib().pd_rmsnorm_bwd(x2.data_ptr(), w.data_ptr() if w is not None else None, dy2.data_ptr(),
                                     rstd.data_ptr(), dx.data_ptr(), x2.shape[0], x2.shape[1], _s()), "rmsnorm_bwd")
        return dx.view(ctx.shape), None, None


def rms_norm(x: Tensor, w: Tensor | None, eps: float) -> Tensor:
    return _RMSNorm.apply(x, w, eps)


class _Rope(torch.autograd.Function):
    """Rotary embedding on `[B, T, H, hd]` (full head_dim). Out of place; backward = inverse rotation."""

    @staticmethod
    def forward(ctx, x: Tensor, cos_half: Tensor, sin_half: Tensor) -> Tensor:  # type: ignore[override]
        B, T, H, hd = x.shape
        x = x.contiguous()
        y = torch.empty_like(x)  # rotated straight from `x` into `y`: no copy first
        _check(_lib().pd_rope_to(x.data_ptr(), y.data_ptr(), cos_half.data_ptr(), sin_half.data_ptr(), B * T, T, H, hd, 0,
                                 _s()), "rope")
        ctx.save_for_backward(cos_half, sin_half)
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):  # type: ignore[override]
        cos_half, sin_half = ctx.saved_tensors
        B, T, H, hd = dy.shape
        dy = dy.contiguous()
        dx = torch.empty_like(dy)
        _check(_lib().pd_rope_to(dy.data_ptr(), dx.data_ptr(), cos_half.data_ptr(), sin_half.data_ptr(), B * T, T, H, hd, 1,
                                 _s()), "rope_bwd")
        return dx, None, None


def rope(x: Tensor, cos_half: Tensor, sin_half: Tensor) -> Tensor:
    """`cos_half/sin_half [T, hd/2]` fp32 contiguous (positions shared by every batch row)."""
    return _Rope.apply(x, cos_half, sin_half)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate: Tensor, up: Tensor) -> Tensor:  # type: ignore[override]
        gate, up = gate.contiguous(), up.contiguous()
        out = torch.empty_like(gate)
        _check(_lib().pd_swiglu_fwd(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), _s()), "swiglu_fwd")
        ctx.save_for_backward(gate, up)
        return out

    @staticmethod
    def backward(ctx, dout: Tensor):  # type: ignore[override]
        gate, up = ctx.saved_tensors
        dout = dout.contiguous()
        dg, du = torch.empty_like(gate), torch.empty_like(up)
        _check(_lib().pd_swiglu_bwd(gate.data_ptr(), up.data_ptr(), dout.data_ptr(), dg.data_ptr(), du.data_ptr(),
                                    gate.numel(), _s()), "swiglu_bwd")
        return dg, du


def swiglu(gate: Tensor, up: Tensor) -> Tensor:
    return _SwiGLU.apply(gate, up)


class _SquashActivity(torch.autograd.Function):
    """`pre [rows, C]` bf16 -> (`lower` bf16, `activity [C]` fp32 = mean over rows of the smooth-L0
    penalty of the upper-leaky importance). One read of `pre` in forward, one fused pass in backward
    that applies the lower-leaky gradient rule and the minimality gradient together."""

    @staticmethod
    def forward(ctx, pre: Tensor, gamma, normalize_at_one: bool, alpha: float):  # type: ignore[override]
        """`gamma`: a float, or a 0-d fp32 device tensor (the schedule's slot in the step-scalar table)."""
        rows, Cn = pre.shape
        pre = pre.contiguous()
        lower = torch.empty_like(pre)
        colsum = torch.zeros(Cn, device=pre.device, dtype=torch.float32)
        lib = _lib()
        lib.pd_ci_squash_activity.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_float,
                                              C.c_int, C.c_float, C.c_void_p, C.c_void_p]
        g_val, g_ptr = _scalar_arg(gamma)
        _check(lib.pd_ci_squash_activity(pre.data_ptr(), lower.data_ptr(), colsum.data_ptr(), rows, Cn, g_val,
                                         int(normalize_at_one), alpha, g_ptr, _s()), "ci_squash_activity")
        ctx.save_for_backward(pre)
        ctx.cfg = (gamma, normalize_at_one, alpha)
        ctx.mark_non_differentiable()
        return lower, colsum / rows

    @staticmethod
    def backward(ctx, dlower: Tensor | None, dact: Tensor | None):  # type: ignore[override]
        (pre,) = ctx.saved_tensors
        gamma, norm, alpha = ctx.cfg
        rows, Cn = pre.shape
        dcol = (dact.float() / rows).contiguous() if dact is not None else torch.zeros(Cn, device=pre.device)
        dpre = torch.empty_like(pre)
        lib = _lib()
        lib.pd_ci_squash_activity_bwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int,
                                                  C.c_float, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
        dl = None if dlower is None else dlower.contiguous()
        g_val, g_ptr = _scalar_arg(gamma)
        _check(lib.pd_ci_squash_activity_bwd(pre.data_ptr(), dl.data_ptr() if dl is not None else None, dcol.data_ptr(),
                                             dpre.data_ptr(), rows, Cn, g_val, int(norm), alpha, g_ptr, _s()),
               "ci_squash_activity_bwd")
        return dpre, None, None, None


def squash_activity(pre: Tensor, gamma: float, normalize_at_one: bool, alpha: float = 0.01) -> tuple[Tensor, Tensor]:
    lead = pre.shape[:-1]
    lower, act = _SquashActivity.apply(pre.reshape(-1, pre.shape[-1]), gamma, normalize_at_one, alpha)
    return lower.reshape(*lead, -1), act


class _SquashActivityJobs(torch.autograd.Function):
    """Narrow CI of an expert-blocked site: `pre [tokens, k * c]` bf16 with the selected experts
    `experts [tokens, k]` -> (`lower` bf16 in the same layout, `activity [n_blocks * c]` fp32 = the
    per-component sum of the smooth-L0 penalty over the tokens that selected its expert, divided by
    the number of tokens). The forward walks the padded sorted job layout so every thread block sums
    one expert's rows; the backward is pointwise in token order."""

    @staticmethod
    def forward(ctx, pre: Tensor, experts: Tensor, layout, n_blocks: int, gamma: float,  # type: ignore[override]
                normalize_at_one: bool, alpha: float):
        tokens, kc = pre.shape
        k = experts.shape[-1]
        c = kc // k
        pre = pre.contiguous()
        experts = experts.reshape(tokens, k).contiguous()
        lower = torch.empty_like(pre)
        colsum = torch.zeros(n_blocks * c, device=pre.device, dtype=torch.float32)
        rowmap = layout.rowmap(k, c)
        lib = _lib()
        lib.pd_ci_squash_activity_jobs.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                   C.c_longlong, C.c_int, C.c_longlong, C.c_float, C.c_int,
                                                   C.c_float, C.c_void_p, C.c_void_p]
        g_val, g_ptr = _scalar_arg(gamma)
        _check(lib.pd_ci_squash_activity_jobs(pre.data_ptr(), lower.data_ptr(), colsum.data_ptr(), rowmap.data_ptr(),
                                              layout.bgroup.data_ptr(), layout.n_rows, c, kc, g_val,
                                              int(normalize_at_one), alpha, g_ptr, _s()), "ci_squash_activity_jobs")
        ctx.save_for_backward(pre, experts)
        ctx.cfg = (gamma, normalize_at_one, alpha, k, c)
        ctx.n_blocks = n_blocks
        return lower, colsum / tokens

    @staticmethod
    def backward(ctx, dlower: Tensor | None, dact: Tensor | None):  # type: ignore[override]
        pre, experts = ctx.saved_tensors
        gamma, norm, alpha, k, c = ctx.cfg
        tokens = pre.shape[0]
        dcol = (dact.float() / tokens).contiguous() if dact is not None else torch.zeros(
            ctx.n_blocks * c, device=pre.device)
        dpre = torch.empty_like(pre)
        lib = _lib()
        lib.pd_ci_squash_activity_jobs_bwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                                       C.c_longlong, C.c_int, C.c_int, C.c_float, C.c_int, C.c_float,
                                                       C.c_void_p, C.c_void_p]
        dl = None if dlower is None else dlower.contiguous()
        g_val, g_ptr = _scalar_arg(gamma)
        _check(lib.pd_ci_squash_activity_jobs_bwd(pre.data_ptr(), dl.data_ptr() if dl is not None else None,
                                                  dcol.data_ptr(), experts.data_ptr(), dpre.data_ptr(), tokens, k, c,
                                                  g_val, int(norm), alpha, g_ptr, _s()), "ci_squash_activity_jobs_bwd")
        return dpre, None, None, None, None, None, None


def squash_activity_selected(values: Tensor, experts: Tensor, n_blocks: int, gamma: float, normalize_at_one: bool,
                             alpha: float = 0.01) -> tuple[Tensor, Tensor]:
    """`values [..., k * c]`, `experts [..., k]` (the pinned selection tensor, which also keys the cached
    job layout) -> (`lower` like `values`, `activity [n_blocks * c]`)."""
    from param_decomp_b200.ops.grouped import JobLayout

    layout = JobLayout.cached(experts, n_blocks)
    lead = values.shape[:-1]
    lower, act = _SquashActivityJobs.apply(values.reshape(-1, values.shape[-1]), experts, layout, n_blocks, gamma,
                                           normalize_at_one, alpha)
    return lower.reshape(*lead, -1), act


def vocab_kl_rows(lc: Tensor, lm: Tensor, want_grad: bool, grad_out: Tensor | None = None) -> tuple[Tensor, Tensor | None]:
    """Per-row `KL(softmax(lc) || softmax(lm))` and (optionally) `softmax(lm) - softmax(lc)`.
    `lc`, `lm`: `[rows, V]` bf16 views whose row pitch is a multiple of 8 elements. `grad_out`: a buffer with
    the same pitch to write the gradient into (re-used across chunks by the streamed form)."""
    rows, V = lc.shape
    assert lc.stride(1) == 1 and lm.stride(1) == 1 and lc.stride(0) == lm.stride(0) and lc.stride(0) % 8 == 0
    kl = torch.empty(rows, device=lc.device, dtype=torch.float32)
    dlm = None
    if want_grad and grad_out is not None:
        assert grad_out.stride(0) == lc.stride(0) and grad_out.shape[0] >= rows and grad_out.dtype == torch.bfloat16
        dlm = grad_out[:rows, :V]
    elif want_grad:
        dlm = torch.empty(rows, lc.stride(0), device=lc.device, dtype=torch.bfloat16)[:, :V]
    lib = _lib()
    lib.pd_vocab_kl.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_longlong,
                                C.c_void_p]
    _check(lib.pd_vocab_kl(lc.data_ptr(), lm.data_ptr(), dlm.data_ptr() if dlm is not None else None, kl.data_ptr(),
                           rows, V, lc.stride(0), _s()), "vocab_kl")
    return kl, dlm


def philox_uniform(seed64: int, stream: int, rows: int, cols: int, row_offset: int, device) -> Tensor:
    """`[rows, cols]` fp32 uniforms, bit-identical to `philox_ref.uniform` and to the GEMM epilogues."""
    out = torch.empty(rows, cols, device=device, dtype=torch.float32)
    lib = _lib()
    lib.pd_philox_uniform.argtypes = [C.c_void_p, C.c_longlong, C.c_int, C.c_ulonglong, C.c_uint, C.c_uint, C.c_void_p,
                                      C.c_void_p]
    _check(lib.pd_philox_uniform(out.data_ptr(), rows, cols, seed64 & (2**64 - 1), stream & 0xFFFFFFFF,
                                 row_offset & 0xFFFFFFFF, nv.step_seed_ptr(seed64) or None, _s()), "philox_uniform")
    return out


def split_bf16(x: Tensor) -> tuple[Tensor, Tensor]:
    assert x.dtype == torch.float32 and x.is_contiguous()
    hi, lo = torch.empty_like(x, dtype=torch.bfloat16), torch.empty_like(x, dtype=torch.bfloat16)
    lib = _lib()
    lib.pd_split_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p]
    _check(lib.pd_split_bf16(x.data_ptr(), hi.data_ptr(), lo.data_ptr(), x.numel(), _s()), "split_bf16")
    return hi, lo


def split3_bf16(x: Tensor, along_cols: bool) -> Tensor:
    """Split-precision copy of `x [g, rows, cols]` fp32 (`x = hi + lo` in bf16) laid out as three K-phases:
    `[g, rows, 3 cols] = [hi | hi | lo]` (`along_cols`) or `[g, 3 rows, cols] = [hi ; lo ; hi]`."""
    assert x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 3 and x.shape[2] % 4 == 0
    g, rows, cols = x.shape
    out = torch.empty((g, rows, 3 * cols) if along_cols else (g, 3 * rows, cols), device=x.device, dtype=torch.bfloat16)
    lib = _lib()
    lib.pd_split3_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_longlong, C.c_int, C.c_void_p]
    _check(lib.pd_split3_bf16(x.data_ptr(), out.data_ptr(), g, rows, cols, int(along_cols), _s()), "split3_bf16")
    return out


def colsum_bf16(x: Tensor) -> Tensor:
    """Column sums of a `[..., rows, C]` bf16 tensor in fp32: `[..., C]` (one read, no fp32 copy)."""
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    lead = x.shape[:-2]
    rows, Cn = x.shape[-2], x.shape[-1]
    flat = x.reshape(-1, rows, Cn)
    out = torch.zeros(flat.shape[0], Cn, device=x.device, dtype=torch.float32)
    lib = _lib()
    lib.pd_colsum_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_int, C.c_void_p]
    for i in range(flat.shape[0]):
        _check(lib.pd_colsum_bf16(flat[i].data_ptr(), out[i].data_ptr(), rows, Cn, _s()), "colsum_bf16")
    return out.reshape(*lead, Cn)
