"""Times the memory-bound kernels of the routed-expert path at the 42-expert config's sizes.

    python benchmarks/bench_moe_rows.py [--tokens 8192 --k 8 --experts 42 --d 512 --c 512]

Token fan-out to padded job rows, routing-weighted combine, and the narrow CI squash + per-expert
activity (forward and backward); CUDA-event device time with an L2-sized buffer rewritten between
launches; one JSON line per kernel with the algorithmic bytes moved and the fraction of the measured
copy bandwidth (`MEASURED_PEAKS.json` beside the repository root when present, else 6.65 TB/s).
"""

from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # the repository root (run as a script)

import argparse
import json
from pathlib import Path

import torch

from param_decomp_b200.ops import elementwise as ew
from param_decomp_b200.ops import native as nv
from param_decomp_b200.ops.grouped import JobLayout


def _time(fn, iters: int) -> float:
    flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e1)
    return tot / iters


def _peak_gbs() -> tuple[float, str]:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        if "hbm_gbs" in d:
            return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8)
    ap.add_argument("--experts", type=int, default=42)
    ap.add_argument("--d", type=int, default=512)
    ap.add_argument("--c", type=int, default=512)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    nv.lib()
    N, k, E, d, c = a.tokens, a.k, a.experts, a.d, a.c
    g = torch.Generator(device="cuda").manual_seed(0)
    idx = torch.rand(N, E, device="cuda", generator=g).topk(k, dim=-1).indices
    layout = JobLayout.cached(idx, E)
    R = layout.n_rows
    x = torch.randn(N, d, device="cuda", generator=g).to(torch.bfloat16)
    rows = torch.randn(R, d, device="cuda", generator=g).to(torch.bfloat16)
    w = torch.rand(N, k, device="cuda", generator=g)
    pre = (torch.randn(N, k * c, device="cuda", generator=g) * 1.5).to(torch.bfloat16)
    dlow = torch.randn(N, k * c, device="cuda", generator=g).to(torch.bfloat16)
    rm_tok, rm_ci = layout.rowmap(k, 1), layout.rowmap(k, c)
    colsum = torch.zeros(E * c, device="cuda")
    lower, dpre = torch.empty_like(pre), torch.empty_like(pre)
    dcol = torch.rand(E * c, device="cuda", generator=g)
    lib, C = nv.lib(), __import__("ctypes")
    s = nv.current_stream_ptr

    def squash_fwd():
        colsum.zero_()
        lib.pd_ci_squash_activity_jobs(C.c_void_p(pre.data_ptr()), C.c_void_p(lower.data_ptr()),
                                       C.c_void_p(colsum.data_ptr()), C.c_void_p(rm_ci.data_ptr()),
                                       C.c_void_p(layout.bgroup.data_ptr()), C.c_longlong(R), C.c_int(c),
                                       C.c_longlong(k * c), C.c_float(0.3), C.c_int(1), C.c_float(0.01), C.c_void_p(s()))

    def squash_bwd():
        lib.pd_ci_squash_activity_jobs_bwd(C.c_void_p(pre.data_ptr()), C.c_void_p(dlow.data_ptr()),
                                           C.c_void_p(dcol.data_ptr()), C.c_void_p(idx.data_ptr()),
                                           C.c_void_p(dpre.data_ptr()), C.c_longlong(N), C.c_int(k), C.c_int(c),
                                           C.c_float(0.3), C.c_int(1), C.c_float(0.01), C.c_void_p(s()))

    cases = [
        ("rows_expand", lambda: ew.rows_expand(x, rm_tok, None, R, k, rep=1, use_slot=False), (N + R) * d * 2),
        ("rows_combine", lambda: ew.rows_combine(rows, layout.pos, w, N, k), (N * k + N) * d * 2),
        ("ci_squash_activity_jobs", squash_fwd, 2 * N * k * c * 2),
        ("ci_squash_activity_jobs_bwd", squash_bwd, 3 * N * k * c * 2),
    ]
    peak, kind = _peak_gbs()
    for name, fn, nbytes in cases:
        ms = _time(fn, a.iters)
        gbs = nbytes / ms / 1e6
        print(json.dumps({"kernel": name, "us": round(ms * 1e3, 1), "algorithmic_MB": round(nbytes / 1e6, 1),
                          "GB_per_s": round(gbs), f"frac_of_{kind}_copy_bw": round(gbs / peak, 3),
                          "shape": {"tokens": N, "k": k, "experts": E, "d": d, "c": c, "padded_rows": R}}))
    torch.cuda.synchronize()
    nv.check_status()


if __name__ == "__main__":
    main()
