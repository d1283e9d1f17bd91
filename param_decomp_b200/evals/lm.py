"""LM evaluation operations: CE / KL under the six mask variants, CI-L0, per-position active
counts, attention-pattern reconstruction, plus the target-agnostic metrics of `evals.core`.

Parity: param_decomp/experiments/lm/eval.py:309-394 (mask variants `ci_masked`, `unmasked`,
`stoch_masked`, `random_masked`, `rounded_masked`, `zero_masked`; CE, KL vs the target, and the
CE-unrecovered fraction against the zero-masked baseline), experiments/lm/eval_operations.py,
attn_patterns_eval.py, ci_position_eval.py.
"""

from __future__ import annotations

from typing import Any, Callable

import torch
from torch import Tensor

from param_decomp_b200.config import evals as E
from param_decomp_b200.core import masking
from param_decomp_b200.core.components import prepare_compute_weights
from param_decomp_b200.core.rng import StepKey
from param_decomp_b200.core.train import StepContext, TrainState, run_ci_fn
from param_decomp_b200.evals.core import run_eval_metrics


@torch.no_grad()
def ce_and_kl(ctx: StepContext, state: TrainState, batch: Any, rounding_threshold: float = 0.0) -> dict[str, float]:
    model = ctx.model
    clean = model.clean_forward(batch)
    weights = prepare_compute_weights(state.components, model.compute_dtype).detached()
    ci = run_ci_fn(ctx, state, clean).mask_inputs()  # masks of expert-blocked sites are narrow (selected blocks only)
    key = StepKey(0xE7A1, 0)
    site_index = ctx.site_index
    off = global_row_offset(ctx, ci)  # draws are keyed on the global row: the same masks however the batch is split
    variants: dict[str, masking.Masks] = {
        "ci_masked": masking.ci_masks(ci),
        "unmasked": masking.unmasked_no_delta(ci),
        "stoch_masked": masking.stochastic_masks(ci, key, 0, 0, site_index=site_index, row_offset=off, lazy=False),
        "random_masked": masking.stochastic_masks({k: torch.zeros_like(v) for k, v in ci.items()}, key, 1, 0,
                                                  site_index=site_index, row_offset=off, with_delta=False, lazy=False),
        "rounded_masked": masking.ci_masks({k: (v > rounding_threshold).to(v.dtype) for k, v in ci.items()}),
        "zero_masked": masking.constant_masks(ci, 0.0, None),
    }
    out: dict[str, float] = {}
    target_ce = float(model.ce_loss(clean, batch.tokens))
    out["ce/target"] = target_ce
    ce: dict[str, float] = {}
    for name, masks in variants.items():
        res = model.masked_forward(weights, batch, masks)
        out[f"kl/{name}"] = float(model.recon_loss(clean, res))
        ce[name] = float(model.ce_loss(res, batch.tokens))
        out[f"ce/{name}"] = ce[name]
    for name in variants:
        if name != "zero_masked":  # linear in the batch, so batch and rank averages commute with it
            out[f"ce_difference/{name}"] = ce[name] - target_ce
    out.update(ce_unrecovered(out))
    return out


def ce_unrecovered(values: dict[str, float], prefix: str = "") -> dict[str, float]:
    """`(ce_v - ce_target) / (ce_zero - ce_target)` per mask variant, from whatever CE values `values` holds under
    `<prefix>ce/...`. A ratio does not commute with averaging: the engine calls this again on the values averaged
    over evaluation batches and ranks (`LMEvaluation.finalize`), so the logged fraction is the ratio of the means."""
    target, zero = values.get(prefix + "ce/target"), values.get(prefix + "ce/zero_masked")
    if target is None or zero is None:
        return {}
    denom = zero - target
    out = {}
    for k, v in values.items():
        if k.startswith(prefix + "ce/") and k != prefix + "ce/target":
            name = k[len(prefix) + 3:]
            out[f"{prefix}ce_unrecovered/{name}"] = (v - target) / denom if abs(denom) > 1e-12 else 0.0
    return out


def global_row_offset(ctx: StepContext, ci: dict[str, Tensor]) -> int:
    first = next(iter(ci.values()))
    rows = 1
    for n in first.shape[:-1]:
        rows *= n
    return ctx.collectives.row_offset(rows)


@torch.no_grad()
def active_counts_per_position(ci: dict[str, Tensor]) -> dict[str, float]:
    out = {}
    for thr in (0.0, 0.01, 0.1):
        per_pos = sum((c > thr).float().sum(-1) for c in ci.values())  # [B, T]
        out[f"l0/per_position/gt_{thr}/mean"] = float(per_pos.mean())
        out[f"l0/per_position/gt_{thr}/last"] = float(per_pos[:, -1].mean())
    return out


@torch.no_grad()
def attention_pattern_recon(ctx: StepContext, state: TrainState, batch: Any, stochastic: bool) -> dict[str, float]:
    from param_decomp_b200.ops.attention_kl import attention_pattern_kl

    model = ctx.model
    n_layer = model.arch.n_layer
    keys = tuple(f"attn_scores.{i}" for i in range(n_layer))
    clean = model.clean_forward(batch, capture=keys)
    weights = prepare_compute_weights(state.components, model.compute_dtype).detached()
    ci = run_ci_fn(ctx, state, clean).mask_inputs()
    masks = (masking.stochastic_masks(ci, StepKey(0xE7A2, 0), 0, 0, site_index=ctx.site_index,
                                      row_offset=global_row_offset(ctx, ci), lazy=False)
             if stochastic else masking.ci_masks(ci))
    res = model.masked_forward(weights, batch, masks, capture=keys)
    vals = [float(attention_pattern_kl(clean.captures[k], res.captures[k])) for k in keys]
    tag = "StochasticAttnPatternsReconLoss" if stochastic else "CIMaskedAttnPatternsReconLoss"
    out = {f"{tag}/layer_{i}": v for i, v in enumerate(vals)}
    out[tag] = sum(vals) / len(vals)
    return out


class LMEvaluation:
    """`encode` (text -> token ids, `experiments/lm/prompt_encoder.py`) builds the operand grid of each
    `ArithmeticCIGrid` metric on first use; `arithmetic_grid` supplies one ready-made grid instead."""

    def __init__(self, cfg: E.EvalConfig, sample_eval: Callable[[int], Any], run_dir: Any = None,
                 arithmetic_grid: Any = None, encode: Callable[[str], list[int]] | None = None) -> None:
        self.cfg = cfg
        self.sample = sample_eval
        self.run_dir = run_dir
        self.arithmetic_grid = arithmetic_grid
        self.encode = encode
        self._grids: dict[tuple, Any] = {}
        if encode is not None and arithmetic_grid is None:  # refuse unequal prompt lengths at startup, not at step N
            for m in cfg.metrics:
                if isinstance(m, E.ArithmeticCIGridConfig):
                    self._grid_for(m)

    def _grid_for(self, metric: E.ArithmeticCIGridConfig) -> Any:
        if self.arithmetic_grid is not None:
            return self.arithmetic_grid
        assert self.encode is not None, "ArithmeticCIGrid needs a prompt encoder (LMEvaluation(encode=...))"
        from param_decomp_b200.evals import lm_ops

        key = (metric.operation, tuple(metric.a_range), tuple(metric.b_range))
        if key not in self._grids:
            self._grids[key] = lm_ops.build_arithmetic_prompt_grid(
                self.encode, lm_ops.inclusive_range(metric.a_range), lm_ops.inclusive_range(metric.b_range),
                metric.operation)
        return self._grids[key]

    def is_due(self, step: int) -> bool:
        return any(self.cfg.is_due(m, step) for m in self.cfg.metrics)

    def _extra(self, metric: Any, step: int, state: TrainState, ctx: StepContext, batch: Any) -> dict[str, float]:
        if isinstance(metric, E.CEandKLLossesConfig):
            return ce_and_kl(ctx, state, batch, metric.rounding_threshold)
        if isinstance(metric, E.CIActiveCountsPerPositionConfig):
            with torch.no_grad():
                clean = ctx.model.clean_forward(batch)
                return active_counts_per_position(run_ci_fn(ctx, state, clean).dense_lower())
        if isinstance(metric, E.CIMaskedAttnPatternsReconLossConfig):
            return attention_pattern_recon(ctx, state, batch, stochastic=False)
        if isinstance(metric, E.StochasticAttnPatternsReconLossConfig):
            return attention_pattern_recon(ctx, state, batch, stochastic=True)
        from param_decomp_b200.evals import lm_ops

        if isinstance(metric, E.RouterDivergenceConfig):
            return lm_ops.router_divergence(ctx, state, batch, tuple(metric.strategies))
        if isinstance(metric, E.WellTemperednessConfig):
            extra = metric.model_extra or {}
            return lm_ops.well_temperedness(ctx, state, batch, metric.n_locations,
                                            int(extra.get("n_components", metric.n_components_per_region)),
                                            run_dir=self.run_dir, groups=metric.groups)
        if isinstance(metric, E.ArithmeticCIGridConfig):
            return lm_ops.arithmetic_ci_grid(ctx, state, self._grid_for(metric), metric.top_k, run_dir=self.run_dir,
                                             thresholds=tuple(metric.thresholds), probe_metrics=metric.probe_metrics)
        return {}

    def run(self, step: int, state: TrainState, ctx: StepContext) -> dict[str, Any]:
        return run_eval_metrics(self.cfg, step, state, ctx, self.sample, extra=self._extra, run_dir=self.run_dir)

    def finalize(self, averaged: dict[str, Any]) -> dict[str, Any]:
        """Called by the engine on the metrics averaged over evaluation batches and ranks: quantities that are not
        linear in the batch are formed here, from the averages."""
        out = dict(averaged)
        out.update(ce_unrecovered(out))
        out.update(ce_unrecovered(out, prefix="ArithmeticCIGrid/probe/"))
        return out
