"""Context number: the reference's own single-file torch implementation, unmodified, on the flagship target.

    python benchmarks/context_nano_reference.py --batch 16 --steps 5 --warmup 3          # their file
    python bench.py --config benchmarks/configs/lm_llama4l_vpd_nano_objective.yaml --batch 16 --steps 5 --warmup 3   # this library

`nano_param_decomp/run.py::decompose` is the reference repository's readable plain-PyTorch statement of the method
(cuBLAS linears under bf16 autocast, torch SDPA, masks materialised, torch AdamW). It is NOT the reference's
trainer (that is the JAX / XLA program, which cannot be installed here), so this is context for the hand-written
path, never the `--impl reference` arm of `bench.py`. The file is loaded from `baseline/_ref/nano_param_decomp/run.py`
(a copy of the reference's file, not tracked in this repository); when it is absent the script says so and exits 0.

What the harness supplies, none of it a change to their file: a plain torch 4-layer Llama-style target with `nn.Linear`
q/k/v/o/gate/up/down (d_model 768, 12 heads, RoPE, SwiGLU d_ff 3072, RMSNorm, vocabulary 50,277, random init), synthetic
Zipf(1.1) token batches, stand-in `matplotlib` modules (not installed here; no figure is drawn because the slow
evaluation is switched off and the evaluation period is longer than the run), and a loader that stamps the wall
clock after a device synchronise each time the training loop asks for its next batch - the step time is the
distance between two stamps. Step 0 carries their one-off evaluation and is never counted.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import sys
import time
import types
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
NANO = ROOT / "baseline" / "_ref" / "nano_param_decomp" / "run.py"


def load_nano():
    for name in ("matplotlib", "matplotlib.pyplot"):
        if name not in sys.modules:
            try:
                __import__(name)
            except ModuleNotFoundError:
                sys.modules[name] = types.ModuleType(name)
    if "matplotlib" in sys.modules and not hasattr(sys.modules["matplotlib"], "pyplot"):
        sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]  # type: ignore[attr-defined]
    spec = importlib.util.spec_from_file_location("nano_param_decomp_run", NANO)
    assert spec is not None and spec.loader is not None
    mod = importlib.util.module_from_spec(spec)
    sys.modules["nano_param_decomp_run"] = mod
    spec.loader.exec_module(mod)
    return mod


def build_target(vocab: int, d: int, n_layer: int, n_head: int, d_ff: int, seq: int):
    import torch
    import torch.nn as nn
    import torch.nn.functional as F

    class Block(nn.Module):
        def __init__(self) -> None:
            super().__init__()
            self.q_proj, self.k_proj = nn.Linear(d, d, bias=False), nn.Linear(d, d, bias=False)
            self.v_proj, self.o_proj = nn.Linear(d, d, bias=False), nn.Linear(d, d, bias=False)
            self.gate_proj, self.up_proj = nn.Linear(d, d_ff, bias=False), nn.Linear(d, d_ff, bias=False)
            self.down_proj = nn.Linear(d_ff, d, bias=False)
            self.n1, self.n2 = nn.Parameter(torch.ones(d)), nn.Parameter(torch.ones(d))

        def forward(self, x, cos, sin):
            B, S, _ = x.shape
            h = F.rms_norm(x, (d,), self.n1)
            hd = d // n_head

            def heads(t):
                return t.view(B, S, n_head, hd).transpose(1, 2)

            def rope(t):
                t1, t2 = t[..., : hd // 2], t[..., hd // 2:]
                return torch.cat([t1 * cos - t2 * sin, t2 * cos + t1 * sin], -1)

            q, k, v = rope(heads(self.q_proj(h))), rope(heads(self.k_proj(h))), heads(self.v_proj(h))
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, d)
            x = x + self.o_proj(a)
            h = F.rms_norm(x, (d,), self.n2)
            return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))

    class Llama(nn.Module):
        def __init__(self) -> None:
            super().__init__()
            self.embed = nn.Embedding(vocab, d)
            self.layers = nn.ModuleList([Block() for _ in range(n_layer)])
            self.norm = nn.Parameter(torch.ones(d))
            self.head = nn.Linear(d, vocab, bias=False)
            hd = d // n_head
            inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
            ang = torch.arange(seq).float()[:, None] * inv[None]
            self.register_buffer("cos", ang.cos(), persistent=False)
            self.register_buffer("sin", ang.sin(), persistent=False)

        def forward(self, ids):
            x = self.embed(ids)
            S = ids.shape[1]
            cos, sin = self.cos[:S].to(x.dtype), self.sin[:S].to(x.dtype)
            for blk in self.layers:
                x = blk(x, cos, sin)
            return self.head(F.rms_norm(x, (d,), self.norm))

    torch.manual_seed(0)
    return Llama()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=16, help="sequences per step (their default and the flagship's: 64)")
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--c", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--faithfulness-warmup-steps", type=int, default=5,
                    help="their pre-loop component warm-up (400 by default there); not part of the timed steps")
    args = ap.parse_args()
    if not NANO.exists():
        print(json.dumps({"impl": "reference nano torch file (context)", "unavailable":
                          "baseline/_ref/nano_param_decomp/run.py is not present (copy the reference's file there)"}))
        return
    import torch

    nano = load_nano()
    vocab, d, n_layer, n_head, d_ff = 50277, 768, 4, 12, 3072
    target = build_target(vocab, d, n_layer, n_head, d_ff, args.seq)
    sites = {f"layers.{i}.{k}_proj": args.c for i in range(n_layer) for k in ("q", "k", "v", "o", "gate", "up", "down")}
    n_loop = 1 + args.warmup + args.steps  # step 0 carries their evaluation
    cfg = nano.Config(C_per_module=sites, n_steps=n_loop, batch_size=args.batch, seq_len=args.seq,
                      faithfulness_warmup_steps=args.faithfulness_warmup_steps, eval_freq=10**9, slow_eval_freq=10**9,
                      slow_eval_on_first_step=False, eval_batch_size=min(args.batch, 8), log_every=10**9, use_wandb=False)
    g = torch.Generator().manual_seed(0)
    w = 1.0 / torch.arange(1, vocab + 1, dtype=torch.float64) ** 1.1
    stamps: list[float] = []

    def batches(n_rows: int, stamp: bool):
        while True:
            ids = torch.multinomial(w, n_rows * args.seq, replacement=True, generator=g).view(n_rows, args.seq)
            if stamp:
                if torch.cuda.is_available():
                    torch.cuda.synchronize()
                stamps.append(time.perf_counter())
            yield ids

    nano.decompose(target, cfg, batches(args.batch, True), batches(cfg.eval_batch_size, False))
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    stamps.append(time.perf_counter())
    # stamps[i] = start of step i; the timed steps are the last `steps` ones
    per_step = [(b - a) * 1e3 for a, b in zip(stamps[:-1], stamps[1:])]
    timed = per_step[-args.steps:]
    ms = sum(timed) / len(timed)
    print(json.dumps({"impl": "reference nano torch file (context)", "ms_per_step": round(ms, 2),
                      "tokens_per_s": round(args.batch * args.seq / ms * 1e3, 1), "steps": args.steps,
                      "warmup": args.warmup, "per_step_ms": [round(v, 1) for v in per_step],
                      "config": {"batch": args.batch, "seq_len": args.seq, "C": args.c, "target": "4L d768 h12 ff3072 vocab50277",
                                 "objective": "their Config defaults: global CI transformer 2048 x 8, Lp minimality, "
                                              "stochastic subset recon, persistent PGD (2 inner steps), faithfulness"},
                      "peak_memory_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1) if torch.cuda.is_available() else None,
                      "timing": "wall clock between device-synchronised requests for the next batch"}))


if __name__ == "__main__":
    main()
