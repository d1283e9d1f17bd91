"""The fused compute + collective GEMMs on ONE GPU, every "peer" buffer being local memory.

    python benchmarks/bench_tp_loca.pyl.py [--case rs|ag_rows|ag_weight] [--rows 16384] [--iters 10]

A kernel that waits on another rank never shares a GPU with it as a separate launch, so the multi-rank
paths are measured under `torchrun` (`bench_tp.py`) and profiled here: one process, one kernel, the
rank tables pointing at local buffers. The kernel executes the same code (peer tensor maps, gather
CTAs, flags, rotated rasters); only NVLink is missing, so times are a lower bound for the real thing
and the instruction / memory counters are the kernel's own.
"""

from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # the repository root (run as a script)

import argparse
import json

import torch

from param_decomp_b200.ops import native as nv


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", choices=("rs", "ag_rows", "ag_weight"), default=None)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--c", type=int, default=4096)
    ap.add_argument("--d", type=int, default=3072)
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    dev, bf = "cuda", torch.bfloat16
    M, C, d, W = a.rows, a.c, a.d, a.world
    flags = torch.zeros(max(M // 128, 64), device=dev, dtype=torch.int32)
    seq = [0]
    flush = torch.empty(256 << 20, device=dev, dtype=torch.uint8)

    def timed(fn) -> float:
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        tot = 0.0
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        return tot / a.iters

    cases = {}
    # GEMM -> reduce-scatter: this "rank" contracts its C / W slice; row blocks go to their owners' buffers
    x = torch.randn(M, C // W, device=dev).to(bf)
    u = (torch.randn(C // W, d, device=dev) / C**0.5).to(bf)
    outs = [torch.zeros(M // W, d, device=dev) for _ in range(W)]

    class _Out:
        shape, dtype = (M, d), torch.float32

        def dim(self): return 2
        def stride(self, i): return outs[0].stride(i)
        def data_ptr(self): return outs[0].data_ptr()

    cases["rs"] = (lambda: nv.gemm(x, u, _Out(), b_mn=True, rs=([o.data_ptr() for o in outs], M // W)),
                   2.0 * M * (C // W) * d)
    # all-gather of activation rows -> GEMM (rank 0 of W: its own rows are local, the rest are "remote")
    xs = [torch.randn(M // W, d, device=dev).to(bf) for _ in range(W)]
    full_x = torch.zeros(M, d, device=dev, dtype=bf)
    full_x[: M // W].copy_(xs[0])
    v = (torch.randn(d, C, device=dev) / d**0.5).to(bf)
    y = torch.empty(M, C, device=dev, dtype=bf)

    def ag_rows():
        seq[0] += 1
        nv.gemm(full_x, v, y, b_mn=True, ag=([t.data_ptr() for t in xs], 0, M // W, flags, seq[0]))

    cases["ag_rows"] = (ag_rows, 2.0 * M * d * C)
    # all-gather of a K-sharded weight inside the masked product
    shards = [v[r * d // W:(r + 1) * d // W].contiguous() for r in range(W)]
    full_v = torch.zeros(d, C, device=dev, dtype=bf)
    full_v[: d // W].copy_(shards[0])
    xa = torch.randn(M, d, device=dev).to(bf)
    ci = torch.rand(M, C, device=dev).to(bf)

    def ag_weight():
        seq[0] += 1
        nv.gemm(xa, full_v, y, b_mn=True, epi=nv.EPI_MASK_FWD, ci=ci, seed=1, rng_stream=1,
                ag_b=([t.data_ptr() for t in shards], 0, d // W, flags, seq[0]))

    cases["ag_weight"] = (ag_weight, 2.0 * M * d * C)
    for name, (fn, flops) in cases.items():
        if a.case is not None and name != a.case:
            continue
        ms = timed(fn)
        print(json.dumps({"case": name, "world": W, "rows": M, "C": C, "d": d, "us": round(ms * 1e3, 1),
                          "tflops": round(flops / ms / 1e9, 1)}), flush=True)
    nv.check_status()


if __name__ == "__main__":
    main()
