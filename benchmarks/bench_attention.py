"""Times the tcgen05 flash-attention kernels against torch's fused SDPA (library kernels).

    python benchmarks/bench_attention.py [--batch 64 --seq 512 --heads 12 --kv-heads 12 --hd 64]

Causal self-attention, bf16, forward and forward+backward; CUDA-event device time with an L2-sized
buffer rewritten between launches. One JSON line per implementation.
"""

from __future__ import annotations

import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))  # the repository root (run as a script)

import argparse
import json

import torch
import torch.nn.functional as F

from param_decomp_b200.ops import attention as attn
from param_decomp_b200.ops import native as nv


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


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--kv-heads", type=int, default=12)
    ap.add_argument("--hd", type=int, default=64)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    B, T, H, Hkv, hd = a.batch, a.seq, a.heads, a.kv_heads, a.hd
    q = torch.randn(B, T, H, hd, device="cuda").to(torch.bfloat16).requires_grad_(True)
    k = torch.randn(B, T, Hkv, hd, device="cuda").to(torch.bfloat16).requires_grad_(True)
    v = torch.randn(B, T, Hkv, hd, device="cuda").to(torch.bfloat16).requires_grad_(True)
    g = torch.randn(B, T, H, hd, device="cuda").to(torch.bfloat16)
    fwd_flops = 4.0 * B * H * T * T * hd / 2  # causal: half the square

    def ours_fwd():
        with torch.no_grad():
            return attn.flash_attention(q, k, v, True)

    def ours_fb():
        out = attn.flash_attention(q, k, v, True)
        out.backward(g)
        q.grad = k.grad = v.grad = None

    def lib_fwd():
        with torch.no_grad():
            return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                  is_causal=True, enable_gqa=H != Hkv)

    def lib_fb():
        out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                             enable_gqa=H != Hkv)
        out.backward(g.transpose(1, 2))
        q.grad = k.grad = v.grad = None

    for name, fn, flops in (("ours fwd", ours_fwd, fwd_flops), ("library fwd", lib_fwd, fwd_flops),
                            ("ours fwd+bwd", ours_fb, 3.5 * fwd_flops), ("library fwd+bwd", lib_fb, 3.5 * fwd_flops)):
        ms = _time(fn, a.iters)
        print(json.dumps({"case": name, "B": B, "T": T, "H": H, "Hkv": Hkv, "hd": hd, "us": round(ms * 1e3, 1),
                          "tflops": round(flops / ms / 1e9, 1)}), flush=True)
    nv.check_status()


if __name__ == "__main__":
    main()
