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
    thr = str(float(threshold))  # keyed `l0/<threshold>_<site>` (param_decomp/core/ci_l0_eval.py:89)
    out = {f"l0/{thr}_{s}": v for s, v in per_site.items()}
    for g, pats in (groups or {}).items():
        out[f"l0/{thr}_{g}"] = sum(v for s, v in per_site.items() if any(fnmatch(s, p) for p in pats))
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
                    read_out_steps: tuple[int, ...], key: StepKey, auxiliaries=(), init: str = "random",
                    source_shape: str = "c") -> dict[int, dict[str, float]]:
    """ONE sign-gradient ascent of fresh sources (`init`, `source_shape` as configured; evaluation probes are
    batch-shared `c` sources initialised U(0,1)), read out after each of `read_out_steps`. The ascent climbs the
    output reconstruction loss plus the configured auxiliaries (their constant coefficients); each read-out
    reports the output loss under `loss` and every auxiliary under its name
    (param_decomp/core/recon_eval.py:142-257). Gradients of batch-shared sources are averaged over the batch
    shards, so every rank ascends the same source."""
    with torch.no_grad():
        keys = tuple(dict.fromkeys(c.capture for a in auxiliaries for c in a.comparisons))
        clean = ctx.model.clean_forward(batch, capture=keys)
        weights = prepare_compute_weights(state.components, ctx.model.compute_dtype)
        ci_lower = run_ci_fn(ctx, state, clean).mask_inputs()  # narrow at expert-blocked sites, with their block selections
    lead = tuple(next(iter(ci_lower.values())).shape[:-1])
    positions = lead[1] if ctx.model.has_position_axis and len(lead) > 1 else None
    device = next(iter(ci_lower.values())).device
    off = ctx.collectives.row_offset(adv_mod.fresh_source_rows(source_shape, lead[0], positions))
    leaves = adv_mod.fresh_sources(getattr(ctx.model, "global_sites", ctx.model.sites), init, source_shape, lead[0],
                                   positions, key, 15, device, row_offset=off)
    from types import SimpleNamespace

    term = ReconTerm(name="eval_pgd", index=15, strategy="fresh_pgd",
                     cfg=SimpleNamespace(auxiliaries=tuple(auxiliaries)))  # type: ignore[arg-type]

    def losses(metrics: dict[str, Tensor] | None):
        src, dlt = adv_mod.PersistentAdversary.split(leaves)
        masks = masking.source_masks(ci_lower, src, dlt)
        return masked_recon(ctx, weights, batch, clean, masks, term, 0, with_aux=bool(auxiliaries), metrics=metrics)

    out: dict[int, dict[str, float]] = {}
    done = 0
    for target in read_out_steps:
        for _ in range(target - done):
            _, full = losses(None)
            names = list(leaves)
            gs = torch.autograd.grad(full, [leaves[k] for k in names], allow_unused=True)
            adv_mod.sign_ascent_(leaves, reduce_source_grads(ctx, {
                k: (g if g is not None else torch.zeros_like(leaves[k])) for k, g in zip(names, gs)},
                source_shape == "c"), step_size)
        done = target
        with torch.no_grad():
            m: dict[str, Tensor] = {}
            e2e, _ = losses(m)
            out[target] = {"loss": float(e2e), **{k.rsplit("/", 1)[-1]: float(v) for k, v in m.items()}}
    return out


def run_eval_metrics(cfg: E.EvalConfig, step: int, state: TrainState, ctx: StepContext,
                     sample_eval_batch: Callable[[int], Any],
                     extra: Callable[[Any, int, TrainState, StepContext, Any], dict[str, Any]] | None = None,
                     run_dir: Any = None, probe_ci: Callable[[], dict[str, Tensor]] | None = None) -> dict[str, Any]:
    """Run every metric due at `step` over `cfg.n_steps` eval batches (identical batches and keys at every
    evaluation, so evaluations carry no sampling variation). CI histograms, mean CI per component and activation
    density share ONE accumulated reduction over the batches (`evals/reductions.py`), summed over the data-parallel
    ranks before it is read; their figures go to `<run_dir>/figures/`. `probe_ci()` (toy targets: one probe
    per feature) feeds the permutation metrics (`evals/permutation.py`)."""
    from param_decomp_b200.evals import permutation as perm
    from param_decomp_b200.evals import reductions as R

    due = [m for m in cfg.metrics if cfg.is_due(m, step)]
    if not due:
        return {}
    out: dict[str, Any] = {}
    acc: dict[str, list[float]] = {}
    by_type = {type(m): m for m in due}
    hist_cfg = by_type.get(E.CIHistogramsConfig)
    dens_cfg = by_type.get(E.ComponentActivationDensityConfig)
    want_reduction = hist_cfg is not None or dens_cfg is not None or E.CIMeanPerComponentConfig in by_type
    red_acc = R.ReductionAccumulation(
        n_comp_bins=hist_cfg.density_heatmap_n_bins if hist_cfg is not None else None,
        alive_threshold=dens_cfg.ci_alive_threshold if dens_cfg is not None else 0.0) if want_reduction else None
    n_accum = hist_cfg.n_batches_accum if (hist_cfg is not None and hist_cfg.n_batches_accum) else cfg.n_steps
    for i in range(max(cfg.n_steps, n_accum if want_reduction else 0)):
        batch = sample_eval_batch(i)
        with torch.no_grad():
            clean = ctx.model.clean_forward(batch)
            ci = run_ci_fn(ctx, state, clean)
            ci_lower = ci.dense_lower()
        if red_acc is not None and i < n_accum:
            R.fold(red_acc, ci.lower)
        if i >= cfg.n_steps:
            continue
        for m in due:
            vals: dict[str, float] = {}
            if isinstance(m, E.CI_L0Config):
                vals = ci_l0(ci_lower, m.ci_alive_threshold, m.groups)
            elif isinstance(m, (E.EvalPGDReconLossConfig, E.SlowPGDReconLossConfig)):
                key = StepKey(0xE7A1, i)
                res = fresh_pgd_recon(ctx, state, batch, m.step_size, tuple(m.read_out_steps), key,
                                      auxiliaries=tuple(getattr(m, "auxiliaries", ()) or ()), init=m.init,
                                      source_shape=m.source_shape)
                for n, d in res.items():
                    vals[f"{m.type}_{n}step"] = d["loss"]
                    vals.update({f"{m.type}_{n}step/{k}": v for k, v in d.items() if k != "loss"})
            elif isinstance(m, (E.CIHistogramsConfig, E.CIMeanPerComponentConfig, E.ComponentActivationDensityConfig,
                                E.IdentityCIErrorConfig, E.PermutedCIPlotsConfig, E.UVPlotsConfig)):
                continue  # read from the accumulated reduction / the probe below
            elif extra is not None:
                vals = extra(m, step, state, ctx, batch) or {}
            for k, v in vals.items():
                acc.setdefault(k, []).append(v)
    out.update({k: sum(v) / len(v) for k, v in acc.items()})
    if red_acc is not None:
        if ctx.collectives.world_size > 1:
            R.merge_over_ranks(red_acc, ctx.collectives.sum_)
        red = R.finalize(red_acc)
        figs: set[str] = set()
        if hist_cfg is not None:
            out.update(R.histogram_scalars(red))
            figs |= {"ci_histograms"} | ({"density_heatmap"} if hist_cfg.density_heatmap_n_bins else set())
        if E.CIMeanPerComponentConfig in by_type:
            out.update(R.mean_ci_scalars(red))
            figs.add("mean_ci")
        if dens_cfg is not None:
            out.update(R.density_scalars(red))
            figs.add("activation_density")
        if ctx.collectives.rank == 0:
            R.render_figures(red, run_dir, step, figs)
    perm_cfgs = [by_type.get(t) for t in (E.IdentityCIErrorConfig, E.PermutedCIPlotsConfig, E.UVPlotsConfig)]
    if any(c is not None for c in perm_cfgs) and probe_ci is not None:
        with torch.no_grad():
            pci = {k: v.detach().float().cpu().numpy() for k, v in probe_ci().items()}
        err_cfg, plot_cfg, uv_cfg = perm_cfgs
        names = list(pci)
        if err_cfg is not None:
            out.update(perm.errors(perm.resolve_spec(names, error_cfg=err_cfg), pci))
        if plot_cfg is not None and ctx.collectives.rank == 0:
            perm.render_permuted_ci(perm.resolve_spec(names, plots_cfg=plot_cfg), pci, run_dir, step)
        if uv_cfg is not None and ctx.collectives.rank == 0:
            V = {s.name: state.components.site(s.name)[0].detach().float().cpu().numpy() for s in ctx.model.sites
                 if not s.blocked}
            U = {s.name: state.components.site(s.name)[1].detach().float().cpu().numpy() for s in ctx.model.sites
                 if not s.blocked}
            perm.render_uv(perm.resolve_spec(names, plots_cfg=uv_cfg), pci, V, U, run_dir, step)
    return out
