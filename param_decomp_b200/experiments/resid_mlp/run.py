"""`python -m param_decomp_b200.experiments.resid_mlp.run <config.yaml> --data-root <dir>`

YAML -> pretrain the residual-MLP target in-process -> decompose with the generic engine.
Feature values are U(-1, 1); the identity-CI ground truth is checked on `layers.0.mlp_in`.

Parity: param_decomp/experiments/resid_mlp/run.py:1-368.
"""

from __future__ import annotations

import argparse
from pathlib import Path

import torch

from param_decomp_b200.config.experiments import ResidMLPExperimentConfig
from param_decomp_b200.core.metrics import MetricsSink, get_logger, mint_run_id, pin_launch_config, run_dir_for
from param_decomp_b200.core.run import RunResult, run_decomposition_training
from param_decomp_b200.experiments.toy_common import ToyEvaluation, build_toy_ci_fn
from param_decomp_b200.models.resid_mlp import ResidMLPDecomposedModel, pretrain_resid_mlp
from param_decomp_b200.models.tms import sample_sparse_features


def _rows_of_rank(topo, batch: torch.Tensor) -> torch.Tensor:
    n = batch.shape[0] // topo.data_world
    return batch[topo.data_rank * n:(topo.data_rank + 1) * n]


def run_resid_mlp(cfg: ResidMLPExperimentConfig, data_root: Path | None, run_id: str | None = None,
            device: str = "cpu", max_steps_this_entry: int | None = None, state_out: list | None = None) -> RunResult:
    from param_decomp_b200.parallel import topology

    # several processes (torchrun): data parallel, `ddp` placement - replicated state, gradients all-reduced,
    # every rank takes its rows of the one seeded global batch (param_decomp/experiments/tms/run.py:241)
    topo = topology.initialize(None, device)
    device = str(topo.device)
    log = get_logger(topo.rank)
    params = pretrain_resid_mlp(cfg.target, cfg.data.feature_probability, cfg.data.data_generation_type, device)
    site_cs = {s.name: s.C for s in cfg.decomposition.sites.sites}
    model = ResidMLPDecomposedModel(params, site_cs).to(device)
    ci_fn = build_toy_ci_fn(cfg.decomposition.ci, model.sites, cfg.pd.seed)

    run_dir, sink = None, None
    if data_root is not None:
        run_id = topo.broadcast_object(run_id or mint_run_id())
        run_dir = run_dir_for(data_root, run_id)
        if topo.rank == 0:
            pin_launch_config(run_dir, cfg.to_yaml())
        sink = MetricsSink.for_run(run_dir, topo.rank, cfg.wandb, cfg.run_name, cfg.model_dump(mode="json"))
        log.info("run dir %s", run_dir)

    def sample_batch(step: int) -> torch.Tensor:
        g = torch.Generator().manual_seed((cfg.pd.seed * 1_000_003 + 17) * 1_000_003 + step)
        return _rows_of_rank(topo, sample_sparse_features(cfg.pd.batch_size, cfg.target.n_features, cfg.data.feature_probability,
                                      cfg.data.data_generation_type, g, device, low=-1.0))

    def sample_eval(i: int) -> torch.Tensor:
        g = torch.Generator().manual_seed(cfg.pd.seed * 7919 + 104729 + i)
        n = cfg.eval.batch_size if cfg.eval is not None else cfg.pd.batch_size
        return _rows_of_rank(topo, sample_sparse_features(n, cfg.target.n_features, cfg.data.feature_probability,
                                      cfg.data.data_generation_type, g, device, low=-1.0))

    evaluation = ToyEvaluation(cfg.eval, sample_eval, cfg.target.n_features, ("layers.0.mlp_in",), run_dir=run_dir)
    try:
        return run_decomposition_training(model, ci_fn, cfg.pd, cfg.cadence, sample_batch, device=device,
                                          run_dir=run_dir, sink=sink, evaluation=evaluation,
                                          collectives=topo.collectives(),
                                          max_steps_this_entry=max_steps_this_entry, state_out=state_out)
    finally:
        if sink is not None:
            sink.close()
        topo.shutdown()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("config", type=Path)
    ap.add_argument("--data-root", "--data_root", type=Path, required=True)
    ap.add_argument("--run-id", "--run_id", type=str, default=None)
    ap.add_argument("--device", type=str, default="cpu")
    args = ap.parse_args()
    cfg = ResidMLPExperimentConfig.from_file(args.config)
    res = run_resid_mlp(cfg, args.data_root, args.run_id, args.device)
    print(f"finished at step {res.final_step}: {res.run_dir}")


if __name__ == "__main__":
    main()
