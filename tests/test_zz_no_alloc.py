"""The allocation-free clip entry point, called through its exported C symbol.

Some users of this library run where device allocation is forbidden (inside a stream capture, under
a fixed memory budget, inside a host application that owns the allocator). For them
`pd_clip_scale_noalloc` computes the gradient-clipping factor with its scratch in a static array of
the library instead of a freshly allocated accumulator. This test checks it against the regular
path (`pd_sumsq` + `pd_clip_scale`, which needs an allocated, zeroed accumulator) on two calls in a
row: the second call must not be disturbed by what the first left in the shared scratch.
It is collected last so that a failure here cannot hide the result of any other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_noalloc_clip_matches_regular_path_twice():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from param_decomp_b200.ops import native
    from param_decomp_b200.ops import optim as fused_optim

    lib = native.lib()
    fn = lib.pd_clip_scale_noalloc
    fn.argtypes = [C.c_void_p, C.c_longlong, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p]
    fn.restype = C.c_int
    lib.pd_noalloc_strerror.restype = C.c_char_p
    lib.pd_noalloc_strerror.argtypes = [C.c_int]

    torch.manual_seed(0)
    out = torch.empty(2, device="cuda", dtype=torch.float32)  # caller-owned outputs: scale, norm
    stream = torch.cuda.current_stream().cuda_stream
    # two different sizes back to back: the second uses fewer scratch slots than the first left behind
    for n, max_norm in ((3_000_017, 1.0), (70_001, 0.25)):
        g = torch.randn(n, device="cuda") * 0.01
        rc = fn(g.data_ptr(), n, max_norm, out.data_ptr(), out[1:].data_ptr(), stream)
        assert rc == 0, lib.pd_noalloc_strerror(rc).decode()
        norm_ref, scale_ref = fused_optim.grad_norm_and_scale([g], max_norm)
        torch.cuda.synchronize()
        assert float(out[1]) == pytest.approx(float(norm_ref), rel=1e-4)
        assert float(out[0]) == pytest.approx(float(scale_ref), rel=1e-4)
        assert float(out[1]) == pytest.approx(float(g.double().norm()), rel=1e-4)

    # refusals: nothing is launched, the message says why
    too_big = fn(g.data_ptr(), (1 << 31) + 1, 1.0, out.data_ptr(), out[1:].data_ptr(), stream)
    assert too_big == 1 and b"2^31" in lib.pd_noalloc_strerror(too_big)
    assert fn(None, 10, 1.0, out.data_ptr(), out[1:].data_ptr(), stream) == 2
