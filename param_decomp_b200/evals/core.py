"""Target-agnostic evaluation metrics and their scheduler.

Parity: param_decomp/core/ci_l0_eval.py (CI-L0 per site at a threshold, fnmatch groups),
core/recon_eval.py:142-257 (fresh-PGD recon probe, read out after n steps; the slow ladder reads
ONE ascent at several step counts), core/slow_eval.py:93-632 (CI histograms, mean CI per
component, activation density), core/run.py:282-322 (due-evaluation scheduling).
"""

from __future__ import annotations

from fnmatch import fnmatch
from typing import Any, Callable

import torch
from torch import Tensor

from param_decomp_b200.config import evals as E
from param_decomp_b200.core import adversary as adv_mod
from param_decomp_b200.core import masking
from param_decomp_b200.core.components import prepare_compute_weights
from param_decomp_b200.core.objective import ReconTerm
from param_decomp_b200.core.rng import StepKey
from param_decomp_b200.core.train import StepContext, TrainState, masked_recon, reduce_source_grads, run_ci_fn


@torch.no_grad()
def ci_l0(ci_lower: dict[str, Tensor], threshold: float, groups: dict[str, list[str]] | None) -> dict[str, float]:
    """Mean number of components with CI > threshold per position, per site and per group."""
    per_site = {s: float((c > threshold).float().sum(-1).mean()) for s, c in ci_lower.items()}
    out = {f"l0/{s}": v for s, v in per_site.items()}
    for g, pats in (groups or {}).items():
        out[f"l0/{g}"] = sum(v for s, v in per_site.items() if any(fnmatch(s, p) for p in pats))
    return out


@torch.no_grad()
def mean_ci_per_component(ci_lower: dict[str, Tensor]) -> dict[str, Tensor]:
    return {s: c.reshape(-1, c.shape[-1]).float().mean(0) for s, c in ci_lower.items()}


@torch.no_grad()
def activation_density(ci_lower: dict[str, Tensor], threshold: float) -> dict[str, Tensor]:
    return {s: (c.reshape(-1, c.shape[-1]) > threshold).float().mean(0) for s, c in ci_lower.items()}


@torch.no_grad()
def ci_histogram(ci: Tensor, bins: int = 50) -> tuple[Tensor, Tensor]:
    v = ci.float().flatten()
    lo, hi = float(v.min()), float(v.max())
    hi = hi if hi > lo else lo + 1e-6
    return torch.histc(v, bins=bins, min=lo, max=hi), torch.linspace(lo, hi, bins + 1)


def fresh_pgd_recon(ctx: StepContext, state: TrainState, batch: Any, step_size: float,
                    read_out_steps: tuple[int, ...], key: StepKey, auxiliaries=()) -> dict[int, float]:
    """ONE sign-gradient ascent of batch-shared `c` sources, initialised U(0,1), read out (the recon
    loss under the current sources) after each of `read_out_steps`."""
    with torch.no_grad():
        clean = ctx.model.clean_forward(batch)
        weights = prepare_compute_weights(state.components, ctx.model.compute_dtype)
        ci_lower = run_ci_fn(ctx, state, clean).dense_lower()
    lead = tuple(next(iter(ci_lower.values())).shape[:-1])
    positions = lead[1] if ctx.model.has_position_axis and len(lead) > 1 else None
    device = next(iter(ci_lower.values())).device
    leaves = adv_mod.fresh_sources(getattr(ctx.model, "global_sites", ctx.model.sites), "random", "c", lead[0], positions, key, 15, device)
    term = ReconTerm(name="eval_pgd", index=15, strategy="fresh_pgd", cfg=None)  # type: ignore[arg-type]
    out: dict[int, float] = {}
    done = 0
    for target in read_out_steps:
        for _ in range(target - done):
            src, dlt = adv_mod.PersistentAdversary.split(leaves)
            masks = masking.source_masks(ci_lower, src, dlt)
            loss = ctx.model.recon_loss(clean, ctx.model.masked_forward(weights, batch, masks))
            names = list(leaves)
            gs = torch.autograd.grad(loss, [leaves[k] for k in names], allow_unused=True)
            adv_mod.sign_ascent_(leaves, reduce_source_grads(ctx, {
                k: (g if g is not None else torch.zeros_like(leaves[k])) for k, g in zip(names, gs)}, True), step_size)
        done = target
        with torch.no_grad():
            src, dlt = adv_mod.PersistentAdversary.split(leaves)
            masks = masking.source_masks(ci_lower, src, dlt)
            out[target] = float(ctx.model.recon_loss(clean, ctx.model.masked_forward(weights, batch, masks)))
    return out


def run_eval_metrics(cfg: E.EvalConfig, step: int, state: TrainState, ctx: StepContext,
                     sample_eval_batch: Callable[[int], Any],
                     extra: Callable[[Any, int, TrainState, StepContext, Any], dict[str, Any]] | None = None) -> dict[str, Any]:
    """Run every metric due at `step` over `cfg.n_steps` eval batches (identical batches and keys
    at every evaluation, so evaluations carry no sampling variation)."""
    due = [m for m in cfg.metrics if cfg.is_due(m, step)]
    if not due:
        return {}
    out: dict[str, Any] = {}
    acc: dict[str, list[float]] = {}
    for i in range(cfg.n_steps):
        batch = sample_eval_batch(i)
        with torch.no_grad():
            clean = ctx.model.clean_forward(batch)
            ci_lower = run_ci_fn(ctx, state, clean).dense_lower()
        for m in due:
            vals: dict[str, float] = {}
            if isinstance(m, E.CI_L0Config):
                vals = ci_l0(ci_lower, m.ci_alive_threshold, m.groups)
            elif isinstance(m, E.ComponentActivationDensityConfig):
                dens = activation_density(ci_lower, m.ci_alive_threshold)
                vals = {f"activation_density/{s}/alive_frac": float((d > 0).float().mean()) for s, d in dens.items()}
            elif isinstance(m, E.CIMeanPerComponentConfig):
                means = mean_ci_per_component(ci_lower)
                vals = {f"ci_mean/{s}/max": float(v.max()) for s, v in means.items()}
            elif isinstance(m, E.CIHistogramsConfig):
                vals = {f"ci_hist/{s}/frac_above_0.5": float((c > 0.5).float().mean()) for s, c in ci_lower.items()}
            elif isinstance(m, (E.EvalPGDReconLossConfig, E.SlowPGDReconLossConfig)):
                key = StepKey(0xE7A1, i)
                res = fresh_pgd_recon(ctx, state, batch, m.step_size, tuple(m.read_out_steps), key)
                vals = {f"{m.type}_{n}step": v for n, v in res.items()}
            elif extra is not None:
                vals = extra(m, step, state, ctx, batch) or {}
            for k, v in vals.items():
                acc.setdefault(k, []).append(v)
    out.update({k: sum(v) / len(v) for k, v in acc.items()})
    return out
