"""Deviceless fit check: will a run configuration fit a GPU's memory, before any GPU is touched.

    python -m param_decomp_b200.core.debug.fit_check <config.yaml> [--gpus N] [--pool-gib 170]

The reference compiles the real step ahead of time against a device topology and reads XLA's arena
size (param_decomp/core/tools/fit_check.py, experiments/lm/fit_check.py). Without a compiler the
estimate is analytic: persistent state (target weights, fp32 masters + two AdamW moments, bf16
working copies, CI-function parameters) is counted exactly from the shapes the model is built with
on the `meta` device; activations are modelled per pass from the sites' shapes (what the fused
site saves for its backward) and the output edge (logit buffers). The verdict is conservative by a
stated margin rather than exact.
"""

from __future__ import annotations

import argparse
from dataclasses import dataclass
from pathlib import Path
from typing import Any


@dataclass
class FitReport:
    persistent_gib: float
    activations_gib: float
    output_edge_gib: float
    total_gib: float
    pool_gib: float
    fits: bool
    detail: dict[str, float]

    def __str__(self) -> str:
        rows = "\n".join(f"  {k:34s} {v:9.2f} GiB" for k, v in self.detail.items())
        return (f"{rows}\n  {'TOTAL (x1.15 margin)':34s} {self.total_gib:9.2f} GiB of {self.pool_gib:.1f} GiB -> "
                f"{'FITS' if self.fits else 'DOES NOT FIT'}")


def estimate(cfg: Any, n_gpus: int = 1, pool_gib: float = 170.0) -> FitReport:
    from param_decomp_b200.core.objective import build_objective

    arch = cfg.target.spec.arch if hasattr(cfg.target.spec, "arch") else None
    assert arch is not None, "the fit check needs an inline architecture (random_init target) or a resolved one"
    G = 2.0**30
    seq = cfg.data.seq_len
    # the mesh's tp axis holds ranks that see the same rows and split the components (dense sites: along C,
    # expert sites: by expert); the batch is divided over the remaining ranks
    tp = min(getattr(cfg.runtime.mesh, "tp", 1), n_gpus)
    data_shards = max(1, n_gpus // tp)
    rows = cfg.pd.batch_size // data_shards * seq
    wbytes = 2 if cfg.target.weights_dtype == "bfloat16" else 4
    d, L, V = arch.d_model, arch.n_layer, arch.vocab_size
    hd = arch.head_dim or d // arch.n_head
    kv = arch.n_kv_head or arch.n_head
    # sites: (d_in, d_out, C_total, jobs multiplier)
    sites: list[tuple[int, int, int, float]] = []
    cs = cfg.decomposition.sites.cs
    E, k = (arch.n_experts or 1), (arch.experts_per_token or 1)
    dims = {"q": (d, arch.n_head * hd), "k": (d, kv * hd), "v": (d, kv * hd), "o": (arch.n_head * hd, d),
            "gate": (d, arch.d_ff), "up": (d, arch.d_ff), "down": (arch.d_ff, d), "c_fc": (d, arch.d_ff),
            "down_proj": (arch.d_ff, d), "q_proj": (d, arch.n_head * hd), "k_proj": (d, kv * hd),
            "v_proj": (d, kv * hd), "o_proj": (arch.n_head * hd, d), "experts_gate": (d, arch.d_ff),
            "experts_up": (d, arch.d_ff), "experts_down": (arch.d_ff, d)}
    target_params = V * d * (1 if arch.tie_embeddings else 2)
    for kind, C in cs.items():
        if kind not in dims:
            continue
        din, dout = dims[kind]
        blocked = kind.startswith("experts_")
        for _ in range(L):
            sites.append((din, dout, C, float(k) if blocked else 1.0))
    per_layer_target = sum(a * b * (E if n.startswith("experts_") else 1) for n, (a, b) in dims.items()
                           if n in ("q", "k", "v", "o") or n in cs)
    target_params += L * per_layer_target
    comp_params = sum((din + dout) * C for din, dout, C, _ in sites) / tp
    ci_hidden = getattr(cfg.decomposition.ci, "hidden_dims", (0,))[0] if hasattr(cfg.decomposition.ci, "hidden_dims") else 0
    ci_params = sum(din * ci_hidden + ci_hidden * C for din, _, C, _ in sites)
    expert_split = tp > 1 and E > 1  # expert-split stacks keep the replicated optimizer over the batch axes
    shard = data_shards if (isinstance(cfg.runtime.sharding, str) and cfg.runtime.sharding != "ddp"
                            and not expert_split) else 1
    persistent = {
        "target weights": target_params * wbytes / G,
        "component masters + AdamW m, v (fp32)": comp_params * 12 / shard / G,
        "component grads (fp32)": comp_params * 4 / G,
        "bf16 working copies (hi + lo)": comp_params * 4 / G,
        "CI fn params + grads + m, v (fp32)": ci_params * 16 / G,
    }
    n_draws = sum(getattr(t, "n_samples", 1) for t in build_objective(cfg.pd).recon)
    # per draw and site the fused path keeps x, A (and H when the CI needs a gradient), per job row
    # (blocked sites additionally keep the per-job mask rows, the padded job copies and the job outputs)
    act = sum(rows * mult * ((din + 2 * C / tp) * 2 if mult == 1.0 else (2 * din + 5 * (C // E) + 2 * dout) * 2 * 1.25 / tp)
              for din, dout, C, mult in sites)
    ci_act = sum(rows * ((C if mult == 1.0 else C // E * k) * 2 * 3 + ci_hidden * 2) for _, _, C, mult in sites)
    resid = rows * d * 2 * L * 6
    logits = rows * ((V + 63) // 64 * 64) * 2
    detail = dict(persistent)
    detail[f"site activations x {n_draws} draws"] = act * n_draws / G
    detail["CI function activations"] = ci_act / G
    detail["residual stream / block activations"] = resid * (1 + n_draws) / G
    detail["logit buffers (clean, masked, gradient)"] = 3 * logits / G
    total = sum(detail.values()) * 1.15
    return FitReport(sum(persistent.values()), (act * n_draws + ci_act + resid * (1 + n_draws)) / G, 3 * logits / G, total,
                     pool_gib, total <= pool_gib, detail)


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("config", type=Path)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--pool-gib", type=float, default=170.0)
    args = ap.parse_args(argv)
    from param_decomp_b200.config.experiments import LMExperimentConfig

    print(estimate(LMExperimentConfig.from_file(args.config), args.gpus, args.pool_gib))


if __name__ == "__main__":
    main()
