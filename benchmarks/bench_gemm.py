"""Micro-benchmark of the tcgen05 GEMM engine on the decomposed-site products of the flagship LM.

    python benchmarks/bench_gemm.py                         # table over the three site shapes
    python benchmarks/bench_gemm.py --case mask_fwd --rows 16384 --iters 1   # one small case (profiling)

Cases: `mask_fwd` (`A = (xV) * (m - d)` with the mask drawn in the epilogue, also emits `H = xV`),
`site_out` (`y = A U + (d x) W^T`, two K phases on one accumulator), `mask_bwd` (`dH` and the mask
gradient), `dx` (`dH V^T + dy W`), `dV` / `dU` (weight gradients, split-K fp32 reduce-add).
Device time by CUDA events; an L2-sized buffer is rewritten between timed launches. The roofline
fraction printed is against the `bf16_tflops` burst figure of a cuBLAS GEMM passed with `--peak`.
"""

from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # the repository root (run as a script)

import argparse
import ctypes as C
import json

import torch

from param_decomp_b200.ops import native as nv
from param_decomp_b200.ops.site_linear import _split_k_for

CASES = ("mask_fwd", "site_out", "mask_bwd", "dx", "dV", "dU")


def build(case: str, N: int, C: int, din: int, dout: int, cg: int = 0, epi_tma: int = 0):
    dev, bf = "cuda", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)

    def rn(*s, scale=1.0):
        return (torch.randn(*s, device=dev, generator=g) * scale).to(bf)

    x, V, U, W = rn(N, din), rn(din, C, scale=din**-0.5), rn(C, dout, scale=C**-0.5), rn(dout, din, scale=din**-0.5)
    ci = torch.rand(N, C, device=dev, generator=g).to(bf)
    delta = torch.rand(N, device=dev, generator=g)
    A, H, dy, dH = rn(N, C), rn(N, C), rn(N, dout), rn(N, C)
    if case == "mask_fwd":
        return (lambda: nv.gemm(x, V, A, b_mn=True, epi=nv.EPI_MASK_FWD, out1=H, ci=ci, delta=delta, seed=1,
                                rng_stream=1, cta_group=cg, epi_tma=epi_tma)), 2.0 * N * C * din, (N * din + din * C + 3 * N * C) * 2
    if case == "site_out":
        y = torch.empty(N, dout, device=dev, dtype=bf)
        return (lambda: nv.gemm(A, U, y, b_mn=True, a1=x, b1=W, cta_group=cg)), 2.0 * N * dout * (C + din), \
            (N * C + C * dout + N * din + dout * din + N * dout) * 2
    if case == "mask_bwd":
        dci = torch.empty(N, C, device=dev, dtype=bf)
        return (lambda: nv.gemm(dy, U, dH, epi=nv.EPI_MASK_BWD, ci=ci, h=H, delta=delta, dci=dci, seed=1,
                                rng_stream=1, cta_group=cg, epi_tma=epi_tma)), 2.0 * N * C * dout, (N * dout + C * dout + 4 * N * C) * 2
    if case == "dx":
        dx = torch.empty(N, din, device=dev, dtype=bf)
        return (lambda: nv.gemm(dH, V, dx, a1=dy, b1=W, b1_mn=True, cta_group=cg)), 2.0 * N * din * (C + dout), \
            (N * C + din * C + N * dout + dout * din + N * din) * 2
    if case == "dV":
        gV = torch.zeros(din, C, device=dev)
        sk = _split_k_for(din, C, N)
        return (lambda: nv.gemm(x, dH, gV, a_mn=True, b_mn=True, accumulate=True, split_k=sk, cta_group=cg)), 2.0 * din * C * N, \
            (N * din + N * C) * 2 + din * C * 8
    if case == "dU":
        gU = torch.zeros(C, dout, device=dev)
        sk = _split_k_for(C, dout, N)
        return (lambda: nv.gemm(A, dy, gU, a_mn=True, b_mn=True, accumulate=True, split_k=sk, cta_group=cg)), 2.0 * C * dout * N, \
            (N * C + N * dout) * 2 + C * dout * 8
    raise ValueError(case)


def build_library(case: str, N: int, C: int, din: int, dout: int):
    """The same contraction through `torch.matmul` / `addmm_` (cuBLAS): the comparison arm for the plain cases.
    Two-phase products are two library calls accumulating into one output."""
    dev, bf = "cuda", torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)

    def rn(*s):
        return torch.randn(*s, device=dev, generator=g).to(bf)

    x, V, U, W = rn(N, din), rn(din, C), rn(C, dout), rn(dout, din)
    A, dy, dH = rn(N, C), rn(N, dout), rn(N, C)
    if case == "site_out":
        y = torch.empty(N, dout, device=dev, dtype=bf)
        return lambda: (torch.matmul(A, U, out=y), y.addmm_(x, W.t()))
    if case == "dx":
        dx = torch.empty(N, din, device=dev, dtype=bf)
        return lambda: (torch.matmul(dH, V.t(), out=dx), dx.addmm_(dy, W))
    if case == "dV":
        gV = torch.empty(din, C, device=dev, dtype=bf)
        return lambda: torch.matmul(x.t(), dH, out=gV)
    if case == "dU":
        gU = torch.empty(C, dout, device=dev, dtype=bf)
        return lambda: torch.matmul(A.t(), dy, out=gU)
    if case == "mask_fwd":  # main loop only: H = x V, no mask arithmetic
        H = torch.empty(N, C, device=dev, dtype=bf)
        return lambda: torch.matmul(x, V, out=H)
    if case == "mask_bwd":  # main loop only: dA = dy U^T
        dA = torch.empty(N, C, device=dev, dtype=bf)
        return lambda: torch.matmul(dy, U.t(), out=dA)
    raise ValueError(case)


def time_case(fn, iters: int, warmup: int = 3) -> float:
    flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / max(iters, 1)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", choices=CASES, default=None)
    ap.add_argument("--shape", type=str, default=None, help="d_in,d_out of the site (default with --case: 768,768)")
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--c", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--cta-group", type=int, default=0, help="1 = single-CTA tiles, 2 = CTA pairs, 0 = library default")
    ap.add_argument("--epi-tma", type=int, default=0,
                    help="mask epilogues: 0 = library default, 1 = plain loads / stores, 2 = TMA-fed operand boxes")
    ap.add_argument("--stages", type=int, default=0,
                    help="probe of pipeline depth: use only this many stages of the operand ring (0 = all)")
    ap.add_argument("--probe", type=int, default=0,
                    help="timing probes (results are garbage): 1 = no operand loads, 2 = no MMAs, 3 = neither")
    ap.add_argument("--timeline", action="store_true",
                    help="print CTA 0's cycle stamps of the last launch: set-up, per-tile MMA / epilogue / producer marks")
    ap.add_argument("--library", action="store_true",
                    help="also time the same contraction through torch.matmul (cuBLAS; bf16 output, no mask arithmetic)")
    ap.add_argument("--peak", type=float, default=1647.5, help="cuBLAS bf16 burst TFLOP/s to report fractions of")
    ap.add_argument("--hbm", type=float, default=6566.4, help="copy bandwidth GB/s to report fractions of")
    args = ap.parse_args()
    shapes = [(768, 768), (768, 3072), (3072, 768)]
    nv.lib().pd_gemm_set_stage_limit(args.stages)
    nv.lib().pd_gemm_set_probe(args.probe)
    cases = CASES if args.case is None else (args.case,)
    if args.shape is not None:
        shapes = [tuple(int(v) for v in args.shape.split(","))]
    elif args.case is not None:
        shapes = shapes[:1]
    for din, dout in shapes:
        for case in cases:
            fn, flops, nbytes = build(case, args.rows, args.c, din, dout, args.cta_group, args.epi_tma)
            tl = None
            if args.timeline:
                tl = torch.zeros(256, dtype=torch.int64, device="cuda")
                nv.lib().pd_gemm_set_timeline(C.c_void_p(tl.data_ptr()))
            ms = time_case(fn, args.iters, args.warmup)
            if tl is not None:
                nv.lib().pd_gemm_set_timeline(C.c_void_p(0))
                v = tl.cpu().tolist()
                rel = lambda x: x - v[0] if x else None
                print(json.dumps({"case": case, "timeline_cycles": {
                    "setup_done": rel(v[1]), "teardown_start": rel(v[2]), "exit": rel(v[3]),
                    "mma_granted_committed": [[rel(v[16 + 2 * i]), rel(v[17 + 2 * i])] for i in range(8) if v[16 + 2 * i]],
                    "epi_full_drained": [[rel(v[80 + 2 * i]), rel(v[81 + 2 * i])] for i in range(8) if v[80 + 2 * i]],
                    "producer_tile_issued": [rel(v[144 + i]) for i in range(8) if v[144 + i]],
                    "mask_epilogue_units": [[rel(v[176 + 8 * u + k]) for k in range(7)] for u in range(8) if v[176 + 8 * u]],
                    "mask_epilogue_tile_top": [rel(v[240 + i]) for i in range(8) if v[240 + i]]}}), flush=True)
            del fn
            lib = {}
            if args.library:
                lib_ms = time_case(build_library(case, args.rows, args.c, din, dout), args.iters, args.warmup)
                lib = {"library_us": round(lib_ms * 1e3, 1), "library_tflops": round(flops / lib_ms / 1e9, 1),
                       "ours_over_library_time": round(ms / lib_ms, 3)}
            print(json.dumps({"case": case, "cta_group": args.cta_group, "epi_tma": args.epi_tma, "stages": args.stages, "probe": args.probe, "rows": args.rows, "C": args.c, "d_in": din, "d_out": dout,
                              "us": round(ms * 1e3, 1), "tflops": round(flops / ms / 1e9, 1),
                              "frac_of_measured_gemm_peak": round(flops / ms / 1e9 / args.peak, 3),
                              "algorithmic_gb_per_s": round(nbytes / ms / 1e6, 1),
                              "frac_of_measured_copy_bw": round(nbytes / ms / 1e6 / args.hbm, 3), **lib}), flush=True)
    nv.check_status()


if __name__ == "__main__":
    main()
