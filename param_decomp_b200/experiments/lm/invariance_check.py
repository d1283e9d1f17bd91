"""`python -m param_decomp_b200.experiments.lm.invariance_check --world 4 --steps 3 [--tp 2] [--sharding zero1] [--objective subset] [--ci global_transformer]
[--muon] [--device cuda]`

Rank-count invariance of the trainer on a tiny Llama target: the SAME global batch, seed and objective run once
in one process and once as `world` data-parallel ranks (gloo on CPU; NCCL with `--device cuda`, one GPU per rank),
and every logged metric of every step must agree up to floating-point reassociation (relative 1e-4 in fp32:
the cross-rank reduction order differs, so bitwise equality is not expected for batch-reduced terms). The
final component matrices are compared too. That is the correctness contract of a layout: how the batch and the
optimizer state are split must not show in the trajectory. Masks and adversary sources are drawn from a
counter-based generator keyed on (seed, step, site, GLOBAL row), so the stochastic terms see the same values.

The objective covers the terms whose reductions cross ranks: importance minimality (global-batch mean inside
the logarithm), stochastic reconstruction, a persistent and a fresh adversary, faithfulness.

Parity: param_decomp/targets/invariance_check.py:1-311 (one layout against all devices of the host).
"""

from __future__ import annotations

import argparse
import json
import os
import socket
import sys
import tempfile
from pathlib import Path
from typing import Any

import torch
import torch.multiprocessing as mp

from param_decomp_b200.config.experiments import LMExperimentConfig

LOSSES = [
    {"type": "ImportanceMinimalityLoss", "coeff": 1e-3, "gamma": 1.0},
    {"type": "StochasticReconLoss", "coeff": 1.0},
    {"type": "PersistentPGDReconLoss", "coeff": 0.5, "source_shape": "bsc", "n_warmup_steps": 1,
     "optimizer": {"type": "sgd", "lr_schedule": 0.05}},
    {"type": "PGDReconLoss", "coeff": 0.5, "init": "random", "source_shape": "bc", "n_steps": 2, "step_size": 0.1},
    {"type": "FaithfulnessLoss", "coeff": 10.0},
]


OBJECTIVES: dict[str, list[dict[str, Any]]] = {
    "default": LOSSES,
    "subset": [{"type": "ImportanceMinimalityLoss", "coeff": 1e-3, "gamma": 2.0},
               {"type": "StochasticReconSubsetLoss", "coeff": 1.0, "routing": {"type": "uniform_k_subset"}},
               {"type": "CIMaskedReconLoss", "coeff": 0.5},
               {"type": "FaithfulnessLoss", "coeff": 10.0}],
    "lp": [{"type": "LpImportanceMinimalityLoss", "coeff": 1e-3, "p_start": 2.0, "p_end": 1.0, "beta": 0.5},
           {"type": "StochasticReconLoss", "coeff": 1.0, "n_samples": 2},
           {"type": "FaithfulnessLoss", "coeff": 10.0}],
    "locality": [{"type": "ImportanceMinimalityLoss", "coeff": 1e-3, "gamma": 1.0, "normalize_at_one": True},
                 {"type": "NonlinearityLocalityLoss", "coeff": 1e-2, "relative_threshold": 8.0,
                  "unit_kind_coefficients": {"neuron": 1.0, "attention_head": 1.0, "deltanet_head": 1.0}},
                 {"type": "StochasticReconLoss", "coeff": 1.0},
                 {"type": "FaithfulnessLoss", "coeff": 10.0}],
    "frequency": [{"type": "ImportanceMinimalityLoss", "coeff": 1e-3, "gamma": 1.0,
                   "frequency": {"coeff": 1e-3, "reference_datapoint_count": 64, "ema_halflife_steps": 2.0}},
                  {"type": "StochasticReconLoss", "coeff": 1.0},
                  {"type": "FaithfulnessLoss", "coeff": 10.0}],
}
CI_FUNCTIONS: dict[str, dict[str, Any]] = {
    "layerwise_mlp": {"type": "layerwise_mlp", "hidden_dims": [32]},
    "global_transformer": {"type": "global_transformer", "d_model": 32, "n_blocks": 2,
                           "attention": {"kind": "mha", "n_heads": 2, "implementation": "xla", "mask": "bidirectional"},
                           "ffn": {"kind": "gelu", "hidden": 64}, "input_tap": "all_block_taps"},
}


def tiny_config(world: int, steps: int, sharding: str, batch: int, cuda: bool, tp: int = 1,
                objective: str = "default", ci: str = "layerwise_mlp", muon: bool = False, family: str = "dense",
                expert_mode: str = "allreduce", with_eval: bool = False, documents: bool = False,
                resident: bool = False) -> LMExperimentConfig:
    """`family: moe` is a top-2-of-5 mixture of experts (five experts on two ranks leave one padding expert); its
    `tp` ranks split the experts, and with `expert_mode: all_to_all` the batch too."""
    raw: dict[str, Any] = {
        "run_name": "invariance",
        "pd": {"seed": 0, "steps": steps, "batch_size": batch,
               "components_optimizer": ({"type": "muon", "lr_schedule": 1e-2} if muon
                                        else {"lr_schedule": 1e-3, "grad_clip_norm": 1.0}),
               "ci_fn_optimizer": {"lr_schedule": 1e-3, "grad_clip_norm": 1.0},
               "loss_metrics": OBJECTIVES[objective]},
        "cadence": {"train_log_every": 1, "checkpointing": {"kind": "none"}},
        "runtime": {"mesh": {"replicate": 1, "fsdp": world // tp, "tp": tp}, "sharding": sharding,
                    "backend": "fused_sm100" if cuda else "eager_torch"},
        "target": {"spec": {"kind": "random_init", "seed": 0,
                            "arch": {"family": "glu_transformer", "n_layer": 2, "d_model": 256 if cuda else 64,
                                     "n_head": 4 if cuda else 2, "d_ff": 512 if cuda else 128,
                                     "vocab_size": 2000 if cuda else 256}},
                   "attention_implementation": "flash" if cuda else "xla",
                   "output_edge": {"kind": "materialized"}, "weights_dtype": "bfloat16" if cuda else "float32"},
        "decomposition": {"sites": {"kind": "glu_transformer", "layers": {"kind": "all"},
                                    "cs": {k: (256 if cuda else 64) for k in ("q", "o", "gate", "down")}},
                          "ci": dict(CI_FUNCTIONS[ci])},
        "data": {"train": {"kind": "synthetic_zipf"}, "eval": {"kind": "synthetic_zipf", "seed": 1},
                 "layout": "unsegmented_tokens", "seq_len": 128 if cuda else 16},
    }
    if resident:  # the `*-replicated-resident` presets are written for a (data, tp) mesh
        raw["runtime"]["mesh"] = {"data": world // tp, "tp": tp}
    if documents:  # packed rows with document boundaries (`write_documents_dataset`): segment-confined attention and losses
        raw["data"].update(train={"kind": "name", "name": DOCUMENTS_DATASET}, eval={"kind": "name", "name": DOCUMENTS_DATASET},
                           layout="documents")
    if with_eval:  # evaluated on the last step: every rank scores its rows of the evaluation batch
        raw["eval"] = {"batch_size": batch, "n_steps": 2, "every": steps - 1 if steps > 1 else 1,
                       "slow_every": steps - 1 if steps > 1 else 1, "slow_on_first_step": False,
                       "metrics": [{"type": "CI_L0", "groups": None}, {"type": "CEandKLLosses", "rounding_threshold": 0.1},
                                   {"type": "PGDReconLoss", "init": "random", "source_shape": "c", "n_steps": 3,
                                    "step_size": 0.1},
                                   {"type": "CIMeanPerComponent"}, {"type": "CIActiveCountsPerPosition"},
                                   {"type": "CIHistograms", "n_batches_accum": 2}, {"type": "ComponentActivationDensity"},
                                   {"type": "CIMaskedAttnPatternsReconLoss"},
                                   {"type": "StochasticAttnPatternsReconLoss"}]}
    if family == "moe":
        raw["target"]["spec"]["arch"] = {"family": "moe", "n_layer": 2, "d_model": 32, "n_head": 2, "d_ff": 16,
                                         "vocab_size": 100, "n_experts": 5, "experts_per_token": 2}
        raw["decomposition"]["sites"] = {"kind": "moe", "layers": {"kind": "all"},
                                         "cs": {"q": 8, "experts_gate": 20, "experts_up": 20, "experts_down": 20}}
        if expert_mode == "all_to_all":
            raw["target"]["expert_implementation"] = "all_to_all"
            raw["runtime"]["mesh"] = {"replicate": 1, "fsdp": world // tp, "tp": tp}
    return LMExperimentConfig.model_validate(raw)


DOCUMENTS_DATASET = "invariance-documents"


def write_documents_dataset(root: Path, vocab_size: int, seq_len: int, rows: int = 96) -> None:
    """A small packed corpus under `<root>/datasets/`: random tokens, a new document every few positions."""
    import numpy as np

    from param_decomp_b200.data.shards import write_token_dataset

    rng = np.random.default_rng(0)
    tok = rng.integers(0, vocab_size, (rows, seq_len)).astype(np.int32)
    starts = rng.random((rows, seq_len)) < 0.2
    starts[:, 0] = False
    doc = np.cumsum(starts, axis=1).astype(np.int32)
    write_token_dataset(root / "datasets" / DOCUMENTS_DATASET, tok, doc, "none", rows_per_group=32, rows_per_shard=48)


def _run(cfg: LMExperimentConfig, root: Path, run_id: str, device: str) -> tuple[Path, list[torch.Tensor]]:
    from param_decomp_b200.experiments.lm.training import train_lm

    states: list = []
    res = train_lm(cfg, root, run_id=run_id, device=device, state_out=states)
    st = states[0]
    return res.run_dir, [p.detach().float().cpu() for p in st.components.parameters()]


def _rank(rank: int, world: int, port: int, root: str, raw: str, cuda: bool, out: Any) -> None:
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.set_num_threads(max(1, (os.cpu_count() or world) // world))
    cfg = LMExperimentConfig.model_validate_json(raw)
    run_dir, params = _run(cfg, Path(root), "p-00000002", f"cuda:{rank}" if cuda else "cpu")
    if rank == 0:
        out["run_dir"] = str(run_dir)
        out["params"] = params


def trajectory(run_dir: Path) -> dict[int, dict[str, float]]:
    steps: dict[int, dict[str, float]] = {}
    for line in (Path(run_dir) / "metrics.jsonl").read_text().splitlines():
        rec = json.loads(line)
        vals = {k: float(v) for k, v in rec.items() if k != "step" and isinstance(v, (int, float))}
        steps.setdefault(int(rec["step"]), {}).update(vals)
    return steps


# wall-clock and memory readings differ between any two runs
# ... and `ce_unrecovered` is a ratio of CE differences already compared one by one; on a random-init target its
# denominator is near zero and multiplies rounding differences a thousandfold
UNCOMPARED = ("perf/", "time/", "mem/", "throughput", "tokens_per_s", "mfu", "step_ms", "elapsed", "lr/",
              "ce_unrecovered")


def relative_gaps(one: dict[int, dict[str, float]], other: dict[int, dict[str, float]]) -> dict[tuple[int, str], float]:
    """`|a - b| / max(|a|, |b|)` of every metric both trajectories logged."""
    out: dict[tuple[int, str], float] = {}
    for step in one.keys() & other.keys():
        for k, a in one[step].items():
            if k in other[step]:
                b = other[step][k]
                out[(step, k)] = abs(a - b) / max(abs(a), abs(b), 1e-30)
    return out


def compare(one: dict[int, dict[str, float]], many: dict[int, dict[str, float]], rtol: float, atol: float,
            floor: dict[tuple[int, str], float] | None = None) -> list[str]:
    """`floor`: how far the one-process run moves when only its summation order changes (`noise_floor`); a metric
    may differ by three times that before it counts. Objectives with discrete inner steps (sign ascent), kinked
    functions or Newton-Schulz updates amplify rounding differences by orders of magnitude within a few steps."""
    bad: list[str] = []
    assert one.keys() == many.keys(), (sorted(one), sorted(many))
    for step in sorted(one):
        keys = [k for k in one[step] if not any(u in k for u in UNCOMPARED)]
        for k in keys:
            if k not in many[step]:
                bad.append(f"step {step} {k}: missing in the multi-rank run")
                continue
            a, b = one[step][k], many[step][k]
            # a gradient norm is a sum of cancelling terms behind kinked functions (hard sigmoid, sign ascent):
            # reassociation noise is amplified there, so it gets ten times the tolerance of a loss
            tol = rtol * (10.0 if "grad_norm" in k else 1.0)
            if floor is not None:
                tol = max(tol, 3.0 * floor.get((step, k), 0.0))
            if abs(a - b) > atol + tol * max(abs(a), abs(b)):
                bad.append(f"step {step} {k}: {a:.8g} (1 rank) vs {b:.8g}")
    return bad


def noise_floor(cfg: LMExperimentConfig, root: Path, reference: dict[int, dict[str, float]], device: str,
                ) -> dict[tuple[int, str], float]:
    """The same one-process run again with another summation order (one thread, the plain GEMM path)."""
    threads, mkldnn = torch.get_num_threads(), torch.backends.mkldnn.enabled
    try:
        torch.set_num_threads(1 if threads > 1 else 2)
        torch.backends.mkldnn.enabled = not mkldnn
        again, _ = _run(cfg, root, "p-00000003", device)
    finally:
        torch.set_num_threads(threads)
        torch.backends.mkldnn.enabled = mkldnn
    return relative_gaps(reference, trajectory(again))


def check(world: int, steps: int, sharding: str, batch: int, device: str, rtol: float | None = None,
          verbose: bool = True, tp: int = 1, with_noise_floor: bool = False, **variant: Any) -> list[str]:
    """`tp` of the `world` ranks see the same tokens and split every site's component axis; the remaining
    `world // tp` split the batch."""
    cuda = device == "cuda"
    if cuda:
        assert torch.cuda.device_count() >= world, f"--device cuda needs {world} GPUs"
    rtol = rtol if rtol is not None else (3e-2 if cuda else 1e-4)  # bf16 operands on the GPU path
    assert world % tp == 0 and batch % (world // tp) == 0, (batch, world, tp)
    with tempfile.TemporaryDirectory() as root:
        if variant.get("documents"):
            first = tiny_config(1, steps, sharding, batch, cuda, **variant)
            write_documents_dataset(Path(root), first.target.spec.arch.vocab_size, first.data.seq_len)
        one_dir, one_params = _run(tiny_config(1, steps, sharding, batch, cuda, **variant), Path(root), "p-00000001",
                                   "cuda:0" if cuda else "cpu")
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        out = mp.Manager().dict()
        mp.spawn(_rank, args=(world, port, root, tiny_config(world, steps, sharding, batch, cuda, tp, **variant).model_dump_json(),
                              cuda, out), nprocs=world, join=True)
        a, b = trajectory(one_dir), trajectory(Path(out["run_dir"]))
        floor = None
        if with_noise_floor and not cuda:
            floor = noise_floor(tiny_config(1, steps, sharding, batch, cuda, **variant), Path(root), a, "cpu")
            if verbose:
                worst = sorted(((sk, v) for sk, v in floor.items() if not any(u in sk[1] for u in UNCOMPARED)),
                               key=lambda kv: -kv[1])[:3]
                print("noise floor (largest):", ", ".join(f"step {s} {k} {v:.2e}" for (s, k), v in worst))
        bad = compare(a, b, rtol, 1e-6, floor)
        for i, (p, q) in enumerate(zip(one_params, out["params"])):
            q = q[: p.shape[0]]  # stacks are padded to a multiple of the rank count
            p = p[tuple(slice(0, n) for n in q.shape)]  # under `tp`, rank 0 holds the leading slice of the component axis
            err = float((p - q).abs().max() / p.abs().max().clamp_min(1e-12))
            # Newton-Schulz runs in bf16 by default: its products round differently on a gathered matrix
            if err > (1e-2 if variant.get("muon") else 10 * rtol):
                bad.append(f"component stack {i}: max relative difference {err:.3g}")
        if verbose:
            last = max(a)
            for k in sorted(a[last]):
                if k in b[last] and not any(u in k for u in UNCOMPARED):
                    print(f"  step {last} {k:55s} {a[last][k]: .8g} {b[last][k]: .8g}")
    return bad


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[1])
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--tp", type=int, default=1, help="ranks that share tokens and split the component axis")
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--sharding", default="ddp")
    ap.add_argument("--device", choices=("cpu", "cuda"), default="cpu")
    ap.add_argument("--rtol", type=float, default=None)
    ap.add_argument("--objective", choices=sorted(OBJECTIVES), default="default")
    ap.add_argument("--ci", choices=sorted(CI_FUNCTIONS), default="layerwise_mlp")
    ap.add_argument("--muon", action="store_true", help="Muon on the component matrices")
    ap.add_argument("--noise-floor", action="store_true",
                    help="also rerun the one-process arm with another summation order and allow three times its drift")
    ap.add_argument("--resident", action="store_true",
                    help="use the (data, tp) mesh of the *-replicated-resident sharding presets")
    ap.add_argument("--documents", action="store_true", help="train on packed rows with document boundaries")
    ap.add_argument("--with-eval", action="store_true", help="also compare the evaluation metrics of the last step")
    ap.add_argument("--family", choices=("dense", "moe"), default="dense")
    ap.add_argument("--expert-mode", choices=("allreduce", "all_to_all"), default="allreduce")
    a = ap.parse_args()
    bad = check(a.world, a.steps, a.sharding, a.batch, a.device, a.rtol, tp=a.tp, objective=a.objective, ci=a.ci,
                muon=a.muon, family=a.family, expert_mode=a.expert_mode, with_noise_floor=a.noise_floor,
                with_eval=a.with_eval, documents=a.documents, resident=a.resident)
    if bad:
        print(f"NOT invariant over {a.world} ranks ({a.sharding}):")
        for line in bad:
            print("  " + line)
        sys.exit(1)
    print(f"invariant: 1 rank == {a.world} ranks ({a.sharding}, {a.steps} steps)")


if __name__ == "__main__":
    main()
