"""ctypes binding of the host-side native library (`ops/_lib/libpdhost.so`, built by `ops/build.py::build_host`).

Optional by design: everything it offers has a pure-torch form that defines the result (`ops/philox_ref.py`), and
`available()` is False until the library has been built, so a source checkout without a compiler still runs.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libpdhost.so"
_lib: C.CDLL | None = None
_tried = False


def lib() -> C.CDLL | None:
    global _lib, _tried
    if not _tried:
        _tried = True
        if LIB_PATH.exists():
            try:
                handle = C.CDLL(str(LIB_PATH))
                handle.pd_host_philox_uniform.argtypes = [C.c_uint64, C.c_uint32, C.c_int64, C.c_int64, C.c_int64,
                                                          C.c_void_p, C.c_int64]
                handle.pd_host_philox_uniform.restype = C.c_int
                _lib = handle
            except OSError:  # built for another machine: fall back to the torch forms
                _lib = None
    return _lib


def available() -> bool:
    return lib() is not None


def philox_uniform(seed64: int, stream: int, rows: int, cols: int, row_offset: int = 0) -> torch.Tensor:
    """`[rows, cols]` fp32 uniforms on the CPU, `cols` a multiple of 8: the stream of `philox_ref.uniform`."""
    handle = lib()
    assert handle is not None, "the host library is not built (python -m param_decomp_b200.ops.build)"
    out = torch.empty(rows, cols, dtype=torch.float32)
    rc = handle.pd_host_philox_uniform(seed64 & 0xFFFFFFFFFFFFFFFF, stream & 0xFFFFFFFF, rows, cols, row_offset,
                                       out.data_ptr(), cols)
    if rc != 0:
        raise ValueError(f"pd_host_philox_uniform refused rows={rows} cols={cols}")
    return out
