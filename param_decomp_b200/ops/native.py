"""ctypes binding of the native sm_100a kernel library (`ops/_lib/libpdb200.so`).

The library is plain C ABI: device pointers and a `cudaStream_t` go in, an int comes back
(0 = launched). Nothing here falls back to another implementation: on a machine with a GPU the
library must load, otherwise `lib()` raises.
"""

from __future__ import annotations

import ctypes as C
from functools import lru_cache
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libpdb200.so"

EPI_PLAIN, EPI_MASK_FWD, EPI_MASK_BWD, EPI_FAITH = 0, 1, 2, 3
ACT_NONE, ACT_GELU, ACT_SILU, ACT_RELU = 0, 1, 2, 3
_ACT = {None: ACT_NONE, "none": ACT_NONE, "gelu": ACT_GELU, "silu": ACT_SILU, "relu": ACT_RELU}


class NativeError(RuntimeError):
    pass


class PdGemmCall(C.Structure):
    _fields_ = [
        ("M", C.c_int), ("N", C.c_int), ("batch", C.c_int), ("K0", C.c_int), ("K1", C.c_int),
        ("A0", C.c_void_p), ("lda0", C.c_longlong), ("bsa0", C.c_longlong), ("a_mn0", C.c_int),
        ("B0", C.c_void_p), ("ldb0", C.c_longlong), ("bsb0", C.c_longlong), ("b_mn0", C.c_int),
        ("A1", C.c_void_p), ("lda1", C.c_longlong), ("bsa1", C.c_longlong), ("a_mn1", C.c_int),
        ("B1", C.c_void_p), ("ldb1", C.c_longlong), ("bsb1", C.c_longlong), ("b_mn1", C.c_int),
        ("out0", C.c_void_p), ("ldo0", C.c_longlong), ("bso0", C.c_longlong),
        ("out_fp32", C.c_int), ("accumulate", C.c_int),
        ("out1", C.c_void_p), ("ldo1", C.c_longlong), ("bso1", C.c_longlong),
        ("alpha", C.c_float), ("bias", C.c_void_p), ("bias_bs", C.c_longlong), ("act", C.c_int),
        ("epi", C.c_int),
        ("ci", C.c_void_p), ("ld_ci", C.c_longlong),
        ("H", C.c_void_p), ("ld_h", C.c_longlong),
        ("delta", C.c_void_p), ("rowscale", C.c_void_p),
        ("dci", C.c_void_p), ("ld_dci", C.c_longlong), ("dci_accumulate", C.c_int), ("dci_bf16", C.c_int),
        ("seed", C.c_ulonglong), ("rng_stream", C.c_uint), ("rng_row_offset", C.c_uint), ("mask_mode", C.c_int),
        ("split_k", C.c_int), ("bn", C.c_int), ("max_ctas", C.c_int),
        ("status", C.c_void_p),
        ("bgroup_of_mblock", C.c_void_p), ("kblock_range", C.c_void_p), ("a_bcast", C.c_int), ("b_bcast", C.c_int),
        ("b_groups", C.c_int),
        ("rs_world", C.c_int), ("rs_rows", C.c_int), ("rs_out", C.c_void_p * 8),
        ("ag_world", C.c_int), ("ag_rank", C.c_int), ("ag_rows", C.c_int), ("ag_src", C.c_void_p * 8),
        ("ag_flags", C.c_void_p), ("ag_seq", C.c_uint), ("ag_mode", C.c_int), ("ag_gather_ctas", C.c_int), ("cta_group", C.c_int), ("rowmap", C.c_void_p), ("philox_col0", C.c_uint),
        ("seed_dev", C.c_void_p), ("alpha_dev", C.c_void_p), ("epi_tma", C.c_int),
    ]  # fmt: skip


@lru_cache(maxsize=1)
def lib() -> C.CDLL:
    if not LIB_PATH.exists():
        raise NativeError(
            f"{LIB_PATH} is missing: run `python -m param_decomp_b200.ops.build` (needs nvcc)"
        )
    handle = C.CDLL(str(LIB_PATH))
    handle.pd_gemm.argtypes = [C.POINTER(PdGemmCall), C.c_void_p]
    handle.pd_gemm.restype = C.c_int
    handle.pd_gemm_call_size.restype = C.c_int
    if handle.pd_gemm_call_size() != C.sizeof(PdGemmCall):
        raise NativeError("PdGemmCall layout differs between native.py and gemm_sm100.cu")
    return handle


_LAUNCHES = 0


@lru_cache(maxsize=1)
def _pd_gemm():
    return lib().pd_gemm


def count_launch(n: int = 1) -> None:
    """Every launch of one of this library's kernels is counted (reported by the benchmark)."""
    global _LAUNCHES
    _LAUNCHES += n


def launch_count() -> int:
    return _LAUNCHES


def has_symbol(name: str) -> bool:
    if not LIB_PATH.exists():
        return False
    try:
        getattr(lib(), name)
        return True
    except AttributeError:
        return False


def available() -> bool:
    return torch.cuda.is_available() and LIB_PATH.exists()


def current_stream_ptr() -> int:
    """Raw handle of the current CUDA stream (the C accessor: this runs once per kernel launch)."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


@lru_cache(maxsize=8)
def _status_word(device_index: int) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", device_index))


def status_word() -> torch.Tensor:
    """The per-device int32 the kernels report a timed-out wait in (0 = no error)."""
    return _status_word(torch._C._cuda_getDevice())


@lru_cache(maxsize=8)
def _status_ptr(device_index: int) -> int:
    return _status_word(device_index).data_ptr()


def check_status() -> None:
    """Synchronising check of the status word; raises if a bounded wait ran out."""
    code = int(status_word().item())
    if code != 0:
        status_word().zero_()
        raise NativeError(f"a device-side wait timed out (status code {code})")


_STEP_SEED: tuple[int, int] | None = None  # (seed64 of the running step, device address of the word holding it)


def set_step_seed(seed64: int | None, device_ptr: int = 0) -> None:
    """While set, a kernel asked to draw from `seed64` reads the seed from `device_ptr` at run time instead
    of taking it by value: the train step's seed word lives in the step-scalar table
    (`ops/step_scalars.py`), so a recorded step draws new masks on every replay. Calls with any other
    seed are unaffected."""
    global _STEP_SEED
    _STEP_SEED = None if seed64 is None else (seed64 & (2**64 - 1), device_ptr)


def step_seed_ptr(seed64: int) -> int:
    st = _STEP_SEED
    return st[1] if (st is not None and st[0] == (seed64 & (2**64 - 1))) else 0


def _operand(t: torch.Tensor, mn_major: bool) -> tuple[int, int, int]:
    """(ptr, ld, batch_stride) of a 2-D or 3-D bf16 operand whose last dim is contiguous."""
    assert t.dtype == torch.bfloat16 and t.stride(-1) == 1, (t.dtype, t.stride())
    bs = t.stride(0) if t.dim() == 3 else 0
    return t.data_ptr(), t.stride(-2), bs


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    out: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    a1: torch.Tensor | None = None,
    b1: torch.Tensor | None = None,
    a1_mn: bool = False,
    b1_mn: bool = False,
    accumulate: bool = False,
    alpha: float = 1.0,
    bias: torch.Tensor | None = None,
    act: str | None = None,
    split_k: int = 1,
    bn: int = 256,
    epi: int = EPI_PLAIN,
    out1: torch.Tensor | None = None,
    ci: torch.Tensor | None = None,
    h: torch.Tensor | None = None,
    delta: torch.Tensor | None = None,
    rowscale: torch.Tensor | None = None,
    dci: torch.Tensor | None = None,
    dci_accumulate: bool = False,
    seed: int = 0,
    rng_stream: int = 0,
    row_offset: int = 0,
    mask_mode: int = 0,
    max_ctas: int = 0,
    bgroup_of_mblock: torch.Tensor | None = None,
    kblock_range: torch.Tensor | None = None,
    a_bcast: bool = False,
    b_bcast: bool = False,
    rs: tuple[list[int], int] | None = None,
    ag: tuple[list[int], int, int, torch.Tensor, int] | None = None,
    ag_b: tuple[list[int], int, int, torch.Tensor, int] | None = None,
    ag_gather_ctas: int = 0,
    cta_group: int = 0,
    rowmap: torch.Tensor | None = None,
    philox_col0: int = 0,
    seed_dev: int = 0,
    alpha_dev: torch.Tensor | None = None,
    epi_tma: int = 0,
) -> torch.Tensor:
    """out = epilogue(A @ B [+ A1 @ B1]) on the tcgen05 kernel.

    `a` is `[M, K]` (`a_mn=False`) or `[K, M]` (`a_mn=True`); `b` is `[N, K]` (`b_mn=False`) or
    `[K, N]` (`b_mn=True`); a leading batch dim is allowed on all of a/b/out for the plain epilogue.
    """
    call = PdGemmCall()
    M, N = out.shape[-2], out.shape[-1]
    K0 = a.shape[-2] if a_mn else a.shape[-1]
    assert (b.shape[-2] if b_mn else b.shape[-1]) == K0, (a.shape, b.shape, a_mn, b_mn)
    assert (a.shape[-1] if a_mn else a.shape[-2]) == M and (b.shape[-1] if b_mn else b.shape[-2]) == N
    batch = out.shape[0] if out.dim() == 3 else 1
    call.M, call.N, call.batch, call.K0 = M, N, batch, K0
    call.A0, call.lda0, call.bsa0 = _operand(a, a_mn)
    call.B0, call.ldb0, call.bsb0 = _operand(b, b_mn)
    call.a_mn0, call.b_mn0 = int(a_mn), int(b_mn)
    if a1 is not None:
        assert b1 is not None
        K1 = a1.shape[-2] if a1_mn else a1.shape[-1]
        assert (b1.shape[-2] if b1_mn else b1.shape[-1]) == K1
        call.K1 = K1
        call.A1, call.lda1, call.bsa1 = _operand(a1, a1_mn)
        call.B1, call.ldb1, call.bsb1 = _operand(b1, b1_mn)
        call.a_mn1, call.b_mn1 = int(a1_mn), int(b1_mn)
    assert out.stride(-1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    call.out0, call.ldo0 = out.data_ptr(), out.stride(-2)
    call.bso0 = out.stride(0) if out.dim() == 3 else 0
    call.out_fp32 = int(out.dtype == torch.float32)
    call.accumulate = int(accumulate)
    if out1 is not None:
        assert out1.dtype == torch.bfloat16 and out1.stride(-1) == 1
        call.out1, call.ldo1 = out1.data_ptr(), out1.stride(-2)
    call.alpha = alpha
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.stride(-1) == 1
        call.bias = bias.data_ptr()
        call.bias_bs = bias.stride(0) if bias.dim() == 2 else 0
    call.act = _ACT[act]
    call.epi = epi
    if ci is not None:
        assert ci.dtype == torch.bfloat16 and ci.stride(-1) == 1
        call.ci, call.ld_ci = ci.data_ptr(), ci.stride(-2)
    if h is not None:
        assert h.dtype == torch.bfloat16 and h.stride(-1) == 1
        call.H, call.ld_h = h.data_ptr(), h.stride(-2)
    if delta is not None:
        assert delta.dtype == torch.float32 and delta.is_contiguous() and (delta.numel() == M or rowmap is not None)
        call.delta = delta.data_ptr()
    if rowscale is not None:
        assert rowscale.dtype == torch.float32 and rowscale.is_contiguous() and (rowscale.numel() == M or rowmap is not None)
        call.rowscale = rowscale.data_ptr()
    if dci is not None:
        assert dci.dtype in (torch.float32, torch.bfloat16) and dci.stride(-1) == 1
        call.dci, call.ld_dci = dci.data_ptr(), dci.stride(-2)
        call.dci_bf16 = int(dci.dtype == torch.bfloat16)
    call.dci_accumulate = int(dci_accumulate)
    call.seed, call.rng_stream, call.mask_mode = seed & (2**64 - 1), rng_stream & 0xFFFFFFFF, mask_mode
    call.rng_row_offset = row_offset & 0xFFFFFFFF
    call.philox_col0 = philox_col0
    call.epi_tma = epi_tma  # mask epilogues: 0 automatic, 1 plain loads / stores, 2 TMA-fed operands where allowed
    # device address of the step's Philox seed word (0: the seed is taken by value)
    call.seed_dev = seed_dev or (step_seed_ptr(seed) if epi in (EPI_MASK_FWD, EPI_MASK_BWD) and mask_mode == 0 else 0)
    if alpha_dev is not None:
        assert alpha_dev.dtype == torch.float32 and alpha_dev.is_cuda and epi == EPI_PLAIN
        call.alpha_dev = alpha_dev.data_ptr()
    call.split_k, call.bn, call.max_ctas = split_k, bn, max_ctas
    call.status = _status_ptr(torch._C._cuda_getDevice())
    if bgroup_of_mblock is not None:
        assert bgroup_of_mblock.dtype == torch.int32 and bgroup_of_mblock.numel() == (M + 127) // 128
        call.bgroup_of_mblock = bgroup_of_mblock.data_ptr()
        call.b_groups = b.shape[0]
        call.bsb0 = b.stride(0)
        if b1 is not None:
            call.bsb1 = b1.stride(0)
    if kblock_range is not None:
        assert kblock_range.dtype == torch.int32 and kblock_range.numel() == 2 * batch
        call.kblock_range = kblock_range.data_ptr()
    call.a_bcast, call.b_bcast = int(a_bcast), int(b_bcast)
    if rs is not None:  # (peer pointers of every rank's fp32 [rows_per_rank, N] buffer, rows_per_rank)
        ptrs, rows = rs
        call.rs_world, call.rs_rows = len(ptrs), rows
        for i, ptr in enumerate(ptrs):
            call.rs_out[i] = ptr
    if ag is not None:  # (peer pointers of every rank's A shard, my rank, rows per rank, flags, sequence number)
        ptrs, rank, rows, flags, seq = ag
        assert flags.dtype == torch.int32 and flags.numel() >= (M + 127) // 128
        call.ag_world, call.ag_rank, call.ag_rows = len(ptrs), rank, rows
        for i, ptr in enumerate(ptrs):
            call.ag_src[i] = ptr
        call.ag_flags, call.ag_seq = flags.data_ptr(), seq & 0xFFFFFFFF
    if ag_b is not None:  # the same for K slabs of the MN-major B operand (rows per rank = K rows)
        ptrs, rank, rows, flags, seq = ag_b
        assert ag is None and flags.dtype == torch.int32 and flags.numel() >= (K0 + 63) // 64
        call.ag_world, call.ag_rank, call.ag_rows, call.ag_mode = len(ptrs), rank, rows, 1
        for i, ptr in enumerate(ptrs):
            call.ag_src[i] = ptr
        call.ag_flags, call.ag_seq = flags.data_ptr(), seq & 0xFFFFFFFF
    call.ag_gather_ctas = ag_gather_ctas
    call.cta_group = cta_group
    if rowmap is not None:
        assert rowmap.dtype == torch.int32 and rowmap.shape == (M, 4) and rowmap.is_contiguous()
        call.rowmap = rowmap.data_ptr()
    rc = _pd_gemm()(C.byref(call), current_stream_ptr())
    global _LAUNCHES
    _LAUNCHES += 1
    if rc != 0:
        raise NativeError(f"pd_gemm refused the call (code {rc})")
    return out
