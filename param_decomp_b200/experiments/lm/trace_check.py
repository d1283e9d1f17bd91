"""Deviceless gate for an LM run configuration:

    python -m param_decomp_b200.experiments.lm.trace_check <config.yaml> [--gpus N]

Everything that can be known before a GPU is touched is checked here, so a bad config fails at
validation time and not after accelerator start-up: the schema; the mesh against the world size; the
placement table against the mesh and the sites (every sharded dimension must tile its factor); the
fused kernels' shape rules (16-byte TMA pitches, attention head sizes, sequence tiling) with the
fallback each violation selects; the analytic memory fit; and finally a REPLICA of the run with every
width shrunk (same families, layer pattern, losses, CI function and evaluation list) stepped once on the
CPU, which exercises the real composition root, objective builder, mask samplers and output edge.

The reference lowers its jitted programs on fake CPU devices for the same purpose
(param_decomp/experiments/lm/trace_check.py); with an eager engine the equivalent of "tracing" is
running the same code on tiny shapes.
"""

from __future__ import annotations

import argparse
from pathlib import Path

from param_decomp_b200.config.experiments import LMExperimentConfig


def static_checks(cfg: LMExperimentConfig, n_gpus: int) -> list[str]:
    """Returns human-readable notes; raises AssertionError on anything that cannot run."""
    from param_decomp_b200.config.run import HsdpMeshShape
    from param_decomp_b200.parallel import placement

    notes: list[str] = []
    mesh_cfg = cfg.runtime.mesh
    mesh = ({"replicate": mesh_cfg.replicate, "fsdp": mesh_cfg.fsdp, "tp": mesh_cfg.tp}
            if isinstance(mesh_cfg, HsdpMeshShape) else {"data": mesh_cfg.data, "tp": mesh_cfg.tp})
    world = 1
    for v in mesh.values():
        world *= v
    if n_gpus > 1:
        assert world == n_gpus, f"mesh {mesh} needs {world} ranks, the launch has {n_gpus}"
    else:
        notes.append(f"mesh {mesh} = {world} ranks; a single process runs it as its own 1-rank slice")
    rules = placement.from_config(cfg.runtime.sharding, mesh)
    notes.append(f"placement {rules.name!r}: stack multiple {placement.stack_multiple(rules, mesh)}")
    arch = getattr(cfg.target.spec, "arch", None)
    if arch is not None:
        data_world = world // mesh.get("tp", 1)
        assert cfg.pd.batch_size % max(data_world, 1) == 0, (
            f"global batch {cfg.pd.batch_size} does not split over {data_world} data ranks")
        hd = arch.head_dim or arch.d_model // arch.n_head
        if cfg.runtime.backend == "fused_sm100":
            if hd not in (64, 128) or cfg.data.seq_len % 128 != 0:
                notes.append(f"attention: head_dim {hd}, seq {cfg.data.seq_len}: outside the tcgen05 kernel "
                             "(64/128, multiple of 128) -> library SDPA fallback")
            if arch.d_model % 8 or arch.d_ff % 8:
                notes.append("d_model / d_ff not multiples of 8: affected products fall back to plain ops")
            for kind, C in cfg.decomposition.sites.cs.items():
                per = C // arch.n_experts if (kind.startswith("experts_") and arch.n_experts) else C
                assert per % 8 == 0, f"{kind}: {per} components per matrix is not a multiple of 8 (16-byte rows)"
            if arch.vocab_size % 8:
                notes.append(f"vocab {arch.vocab_size} is padded to {(arch.vocab_size + 63) // 64 * 64} columns for the logits")
        from param_decomp_b200.core.debug import fit_check

        rep = fit_check.estimate(cfg, max(n_gpus, 1))
        notes.append(f"memory estimate {rep.total_gib:.1f} GiB of {rep.pool_gib:.0f} GiB per GPU -> "
                     f"{'fits' if rep.fits else 'DOES NOT FIT'}")
    return notes


def shrunk(cfg: LMExperimentConfig) -> LMExperimentConfig:
    """The same run with every width reduced: a few dozen channels, a handful of components."""
    raw = cfg.model_dump(mode="json")
    arch = raw["target"]["spec"].get("arch")
    assert arch is not None, "the replica needs an inline architecture"
    fam = arch["family"]
    arch.update(d_model=32, n_head=2, n_kv_head=None, head_dim=16 if fam == "qwen35_moe" else None, d_ff=16,
                vocab_size=97, max_seq_len=16, n_layer=min(arch["n_layer"], 4 if fam == "qwen35_moe" else 2))
    E = 1
    if fam in ("moe", "qwen35_moe"):
        E = min(arch["n_experts"], 4)
        arch.update(n_experts=E, experts_per_token=min(arch["experts_per_token"], 2))
    if fam == "qwen35_moe":
        arch.update(full_attention_interval=2, linear_num_key_heads=2, linear_key_head_dim=8,
                    linear_num_value_heads=2, linear_value_head_dim=8, shared_expert_intermediate=16,
                    partial_rotary_factor=0.5, delta_rule_kernel="chunkwise")
    sites = raw["decomposition"]["sites"]
    sites["cs"] = {k: (E * 4 if k.startswith("experts_") else 8) for k in sites["cs"]}
    sites["layers"] = {"kind": "all"}
    ci = raw["decomposition"]["ci"]
    if "hidden_dims" in ci:
        ci["hidden_dims"] = [8]
    raw["target"]["weights_dtype"] = "float32"
    raw["target"]["attention_implementation"] = "xla"
    raw["data"]["seq_len"] = 16
    raw["pd"]["batch_size"] = 2
    raw["pd"]["steps"] = 2
    raw["runtime"]["backend"] = "eager_torch"
    if raw.get("eval"):
        raw["eval"].update(batch_size=2, n_steps=1)
    return LMExperimentConfig.model_validate(raw)


def replica_step(cfg: LMExperimentConfig) -> dict[str, float]:
    import torch

    from param_decomp_b200.core.objective import build_objective
    from param_decomp_b200.core.run import init_train_state
    from param_decomp_b200.core.train import StepContext, train_step
    from param_decomp_b200.experiments.lm.build import build_lm_run

    small = shrunk(cfg)
    run = build_lm_run(small, None, "cpu")
    obj = build_objective(small.pd)
    ctx = StepContext.build(run.model, obj, small.pd, lazy_masks=True)
    state = init_train_state(run.model, run.ci_fn, small.pd, obj, torch.device("cpu"), 2, 16)
    m = train_step(ctx, state, run.sample_train(0))
    out = {k: float(v) for k, v in m.items() if k.startswith("loss/")}
    assert all(v == v for v in out.values()), f"non-finite loss in the replica: {out}"
    if small.eval is not None:
        from param_decomp_b200.evals.lm import LMEvaluation

        LMEvaluation(small.eval, run.sample_eval).run(0, state, ctx)
    return out


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("config", type=Path)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--no-replica", action="store_true")
    args = ap.parse_args(argv)
    cfg = LMExperimentConfig.from_file(args.config)
    for note in static_checks(cfg, args.gpus):
        print("note:", note)
    if not args.no_replica and getattr(cfg.target.spec, "arch", None) is not None:
        print("replica step:", replica_step(cfg))
    print("ok")


if __name__ == "__main__":
    main()
