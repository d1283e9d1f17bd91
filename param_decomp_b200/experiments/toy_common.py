"""Pieces the two toy composition roots share: CI-fn construction and the toy evaluation.

Parity: param_decomp/experiments/toy_config.py:50-75 (`build_toy_ci_fn_arch`),
experiments/toy_eval.py and core/slow_eval.py:494-551 (identity-CI error via Hungarian matching).
"""

from __future__ import annotations

from typing import Any

import torch
from torch import Tensor, nn

from param_decomp_b200.config.evals import EvalConfig
from param_decomp_b200.config.experiments import LayerwiseMlpCIFnConfig, ToyGlobalMlpCIFnConfig
from param_decomp_b200.core.ci_fn.mlp import GlobalMLPCIFn, LayerwiseMLPCIFn
from param_decomp_b200.core.components import SiteSpec


def build_toy_ci_fn(cfg: LayerwiseMlpCIFnConfig | ToyGlobalMlpCIFnConfig, sites: tuple[SiteSpec, ...],
                    seed: int) -> nn.Module:
    g = torch.Generator().manual_seed(seed + 1)
    if isinstance(cfg, LayerwiseMlpCIFnConfig):
        return LayerwiseMLPCIFn({s.name: (s.d_in, s.C) for s in sites}, {s.name: s.name for s in sites},
                                tuple(cfg.hidden_dims), g)
    return GlobalMLPCIFn(tuple((s.name, s.d_in) for s in sites), {s.name: s.C for s in sites},
                         tuple(cfg.hidden_dims), g)


def identity_ci_error(ci: Tensor, n_features: int, tolerance: float = 0.1) -> float:
    """`ci [n_features, C]`: CI of single-feature probes. After the best one-to-one assignment of
    features to components (Hungarian), count entries off the identity pattern by more than
    `tolerance`: matched entries should be ~1, all others ~0."""
    from scipy.optimize import linear_sum_assignment

    m = ci.detach().float().cpu()
    rows, cols = linear_sum_assignment(-m.numpy())
    target = torch.zeros_like(m)
    target[rows, cols] = 1.0
    return float(((m - target).abs() > tolerance).sum())


def single_feature_probe(n_features: int, value: float = 0.75, device: Any = "cpu") -> Tensor:
    return torch.eye(n_features, device=device) * value


class ToyEvaluation:
    """Runs the configured eval metrics on fresh synthetic batches; also used for the in-loop
    identity-CI ground truth of the toys."""

    def __init__(self, eval_cfg: EvalConfig | None, sample_eval_batch, n_features: int,
                 identity_sites: tuple[str, ...], run_dir: Any = None) -> None:
        self.cfg = eval_cfg
        self.sample = sample_eval_batch
        self.n_features = n_features
        self.identity_sites = identity_sites
        self.run_dir = run_dir  # figures of the slow-tier metrics go to `<run_dir>/figures/`

    def is_due(self, step: int) -> bool:
        if self.cfg is None:
            return False
        return any(self.cfg.is_due(m, step) for m in self.cfg.metrics) or step % self.cfg.every == 0

    def run(self, step: int, state, ctx) -> dict[str, Any]:
        from param_decomp_b200.evals.core import run_eval_metrics

        assert self.cfg is not None
        def probe_ci():
            # one probe per feature (that feature alone, at 0.75): rows = features, columns = components
            dev = next(state.components.parameters()).device
            clean = ctx.model.clean_forward(single_feature_probe(self.n_features, device=dev))
            return run_ci_fn(ctx, state, clean).dense_lower()

        from param_decomp_b200.core.train import run_ci_fn

        out = run_eval_metrics(self.cfg, step, state, ctx, self.sample, run_dir=self.run_dir, probe_ci=probe_ci)
        out.update(identity_metrics(state, ctx, self.n_features, self.identity_sites))
        return out


@torch.no_grad()
def identity_metrics(state, ctx, n_features: int, sites: tuple[str, ...]) -> dict[str, float]:
    from param_decomp_b200.core.train import run_ci_fn

    dev = next(state.components.parameters()).device
    probe = single_feature_probe(n_features, device=dev)
    clean = ctx.model.clean_forward(probe)
    ci = run_ci_fn(ctx, state, clean).dense_lower()
    return {f"identity_ci_error/{s}": identity_ci_error(ci[s], n_features) for s in sites if s in ci}
