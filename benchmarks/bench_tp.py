"""Times the fused tensor-parallel GEMMs against their NCCL twins on the ranks of one node.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P benchmarks/bench_tp.py [--rows 32768] [--iters 20]

Shapes are the flagship LM's row-parallel contraction (`A [rows, C/tp] @ U [C/tp, d_out]`, reduce-
scattered over rows) and its sequence-parallel entry (`all_gather(x [rows/tp, d]) @ V [d, C]`).
Device-timed with CUDA events, max over ranks; rank 0 prints one JSON line per case.
"""

from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # the repository root (run as a script)

import argparse
import json
import os

import torch
import torch.distributed as dist

from param_decomp_b200.ops import native
from param_decomp_b200.parallel import tp


def _time(fn, iters: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    total = 0.0
    for _ in range(iters):
        flush.zero_()  # evict L2 between timed iterations
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    t = torch.tensor([total / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--c", type=int, default=4096)
    ap.add_argument("--d", type=int, default=3072)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    dev = torch.device("cuda", torch.cuda.current_device())
    bf = torch.bfloat16
    M, Cc, d = args.rows, args.c, args.d
    ws = tp.TPWorkspace(dist.group.WORLD, max_rows=M, max_cols=max(Cc, d), device=dev)
    flush = torch.empty(256 << 20, device=dev, dtype=torch.uint8)
    a = torch.randn(M, Cc // world, device=dev).to(bf)
    u = (torch.randn(Cc // world, d, device=dev) / Cc**0.5).to(bf)
    x = torch.randn(M // world, d, device=dev).to(bf)
    v = (torch.randn(d, Cc, device=dev) / d**0.5).to(bf)
    out = torch.empty(M, Cc, device=dev, dtype=bf)
    cases = {
        "gemm_reduce_scatter fused": lambda: tp.gemm_reduce_scatter(ws, a, u, b_mn=True),
        "gemm_reduce_scatter nccl": lambda: tp.gemm_reduce_scatter_nccl(dist.group.WORLD, a, u, b_mn=True),
        "allgather_gemm fused": lambda: tp.allgather_gemm(ws, x, v, out, b_mn=True),
        "allgather_gemm nccl": lambda: tp.allgather_gemm_nccl(dist.group.WORLD, x, v, out, b_mn=True),
    }
    xs = torch.randn(M, d, device=dev).to(bf)
    v_loc = (torch.randn(d // world, Cc, device=dev) / d**0.5).to(bf)
    ci = torch.rand(M, Cc, device=dev).to(bf)
    mask_kw = dict(epi=native.EPI_MASK_FWD, ci=ci, seed=1, rng_stream=1)
    cases["allgather_weight_gemm fused (mask epilogue)"] = lambda: tp.allgather_weight_gemm(ws, xs, v_loc, out, **mask_kw)
    cases["allgather_weight_gemm fused, shard already published"] = lambda: tp.allgather_weight_gemm(
        ws, xs, v_loc, out, publish=False, **mask_kw)
    cases["allgather_weight_gemm fused, 16 gather CTAs"] = lambda: tp.allgather_weight_gemm(
        ws, xs, v_loc, out, publish=False, ag_gather_ctas=16, **mask_kw)
    v_all = (torch.randn(d, Cc, device=dev) / d**0.5).to(bf)
    cases["masked x V with a resident weight (no collective)"] = lambda: native.gemm(xs, v_all, out, b_mn=True, **mask_kw)
    cases["allgather_weight_gemm nccl (mask epilogue)"] = lambda: tp.allgather_weight_gemm_nccl(
        dist.group.WORLD, xs, v_loc, out, **mask_kw)
    for name, fn in cases.items():
        ms = _time(fn, args.iters, flush)
        flops = 2.0 * M * (Cc // world) * d if "reduce" in name else 2.0 * M * d * Cc
        if "reduce" in name:
            link_bytes = M * d * 4 * (world - 1) / world
        elif "weight" in name:
            link_bytes = d // world * Cc * 2 * (world - 1)
        else:
            link_bytes = M // world * d * 2 * (world - 1)
        if rank == 0:
            print(json.dumps({"case": name, "world": world, "ms": ms, "tflops_per_gpu": flops / ms / 1e9,
                              "nvlink_gb_per_s_per_gpu": link_bytes / ms / 1e6, "M": M, "C": Cc, "d": d}))
    native.check_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
