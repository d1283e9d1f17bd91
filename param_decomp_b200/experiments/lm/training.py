"""LM composition root: topology -> target -> CI function -> data -> evaluation -> engine.

Parity: param_decomp/experiments/lm/training.py:197-301 (`_train`), :315-371 (`main`).
"""

from __future__ import annotations

import os
from pathlib import Path

import torch

from param_decomp_b200.config.experiments import LMExperimentConfig
from param_decomp_b200.core.metrics import MetricsSink, device_peak_flops, get_logger, mint_run_id, pin_launch_config, run_dir_for
from param_decomp_b200.core.run import RunResult, run_decomposition_training
from param_decomp_b200.experiments.lm.build import build_lm_run


def train_lm(cfg: LMExperimentConfig, data_root: Path | None, run_id: str | None = None, device: str | None = None,
             max_steps_this_entry: int | None = None, state_out: list | None = None) -> RunResult:
    from param_decomp_b200.parallel import topology

    topo = topology.initialize(cfg.runtime.mesh, device)
    log = get_logger(topo.rank)
    run = build_lm_run(cfg, data_root, topo.device, topo.data_rank, topo.data_world)
    collectives = topo.collectives()

    run_dir, sink = None, None
    if data_root is not None:
        run_id = topo.broadcast_object(run_id or mint_run_id())
        run_dir = run_dir_for(data_root, run_id)
        if topo.rank == 0:
            pin_launch_config(run_dir, cfg.to_yaml())
        sink = MetricsSink.for_run(run_dir, topo.rank, cfg.wandb, cfg.run_name, cfg.model_dump(mode="json"))
        log.info("run dir %s", run_dir)

    from param_decomp_b200.evals.lm import LMEvaluation
    from param_decomp_b200.utils.flops import decomposition_step_flops

    evaluation = LMEvaluation(cfg.eval, run.sample_eval) if cfg.eval is not None else None
    fused = getattr(run.model, "backend", "") == "fused_sm100"
    flops = decomposition_step_flops(run.model, run.ci_fn, cfg.pd, cfg.data.seq_len)
    try:
        return run_decomposition_training(
            run.model, run.ci_fn, cfg.pd, cfg.cadence, run.sample_train, device=topo.device, run_dir=run_dir,
            sink=sink, evaluation=evaluation, collectives=collectives, resume_provenance=cfg.resume_provenance,
            batch_rows=cfg.pd.batch_size // topo.data_world, positions=cfg.data.seq_len,
            units_per_step=run.tokens_per_step, flops_per_step=flops / topo.world, peak_flops=device_peak_flops(),
            lazy_masks=fused, use_fused_optim=fused, init_components=run.init_components,
            max_steps_this_entry=max_steps_this_entry, state_out=state_out,
            profile_steps=3 if cfg.runtime.profiling.kind == "ad_hoc" else 0)
    finally:
        if sink is not None:
            sink.close()
        topo.shutdown()
