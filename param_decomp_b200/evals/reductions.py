"""Accumulated per-site reductions of the causal importances over the evaluation batches, and the figures
drawn from them.

One fold step per evaluation batch adds, for every site: the number of positions, the per-component sum of
CI (-> mean CI per component), the per-component count of positions with CI above the alive threshold
(-> activation density), a histogram of all CI values on `[0, 1]`, and optionally a per-component histogram
(the density heat map). Everything is a sum, so batches - and data-parallel ranks - combine by addition.
Expert-blocked sites contribute their narrow `[.., k * C_block]` values scattered to the components they
belong to; components of experts a token did not select count as CI = 0 for the means and densities, and are
left out of the value histogram (the reference does the same: only materialised entries are binned).

Parity: param_decomp/core/slow_eval.py:93-250 (`ValueHistogram`, `SiteReduction`, binning, alive counts,
per-component sums and histograms), :251-410 (reduction step, fold, finalisation), :635-790 and :948-1045
(figures: value histograms, activation density, grouped mean CI on linear and log scales, dead components,
density heat map).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch
from torch import Tensor

from param_decomp_b200.core.components import SelectedCI
from param_decomp_b200.utils import figures


@dataclass
class SiteAccumulation:
    n_positions: int = 0
    ci_sum: Tensor | None = None  # [C] fp64
    alive: Tensor | None = None  # [C] fp64: positions with CI > threshold
    hist: Tensor | None = None  # [n_bins] fp64: all materialised CI values
    comp_hist: Tensor | None = None  # [C, n_comp_bins] fp64 (density heat map), optional


@dataclass
class ReductionAccumulation:
    n_bins: int = 50
    n_comp_bins: int | None = None
    alive_threshold: float = 0.0
    sites: dict[str, SiteAccumulation] = field(default_factory=dict)
    n_batches: int = 0


def _dense_and_values(v: Tensor | SelectedCI) -> tuple[Tensor, Tensor]:
    """`([positions, C] with zeros where nothing was materialised, flat materialised values)`."""
    if isinstance(v, SelectedCI):
        dense = v.scatter_dense()
        return dense.reshape(-1, dense.shape[-1]).float(), v.values.reshape(-1).float()
    flat = v.reshape(-1, v.shape[-1]).float()
    return flat, flat.reshape(-1)


@torch.no_grad()
def fold(acc: ReductionAccumulation, ci_lower: dict[str, Tensor | SelectedCI]) -> None:
    """Add one evaluation batch."""
    acc.n_batches += 1
    for name, v in ci_lower.items():
        dense, vals = _dense_and_values(v)
        site = acc.sites.setdefault(name, SiteAccumulation())
        C = dense.shape[-1]
        if site.ci_sum is None:
            dev = dense.device
            site.ci_sum = torch.zeros(C, dtype=torch.float64, device=dev)
            site.alive = torch.zeros(C, dtype=torch.float64, device=dev)
            site.hist = torch.zeros(acc.n_bins, dtype=torch.float64, device=dev)
            if acc.n_comp_bins:
                site.comp_hist = torch.zeros(C, acc.n_comp_bins, dtype=torch.float64, device=dev)
        site.n_positions += dense.shape[0]
        site.ci_sum += dense.sum(0).double()
        site.alive += (dense > acc.alive_threshold).sum(0).double()
        site.hist += torch.histc(vals.clamp(0, 1), bins=acc.n_bins, min=0.0, max=1.0).double()
        if site.comp_hist is not None:
            b = (dense.clamp(0, 1) * acc.n_comp_bins).long().clamp_(max=acc.n_comp_bins - 1)  # [positions, C]
            site.comp_hist.scatter_add_(1, b.t().contiguous(), torch.ones_like(b.t(), dtype=torch.float64))


def merge_over_ranks(acc: ReductionAccumulation, sum_fn) -> None:
    """Sum every accumulator over the data-parallel ranks (`sum_fn(t)` all-reduces in place and returns `t`)."""
    for site in acc.sites.values():
        n = sum_fn(torch.tensor([float(site.n_positions)], dtype=torch.float64, device=site.ci_sum.device))
        site.n_positions = int(n.item())
        for t in (site.ci_sum, site.alive, site.hist, site.comp_hist):
            if t is not None:
                sum_fn(t)


@dataclass
class SiteReduction:
    mean_ci: np.ndarray  # [C]
    density: np.ndarray  # [C]: share of positions where the component is alive
    hist: np.ndarray  # [n_bins] counts over [0, 1]
    comp_hist: np.ndarray | None  # [C, n_comp_bins]
    n_positions: int


def finalize(acc: ReductionAccumulation) -> dict[str, SiteReduction]:
    out = {}
    for name, s in acc.sites.items():
        n = max(1, s.n_positions)
        out[name] = SiteReduction((s.ci_sum / n).cpu().numpy(), (s.alive / n).cpu().numpy(), s.hist.cpu().numpy(),
                                  None if s.comp_hist is None else s.comp_hist.cpu().numpy(), s.n_positions)
    return out


def histogram_scalars(red: dict[str, SiteReduction]) -> dict[str, float]:
    """Shares of CI values above 0.1 / 0.5 / 0.9 and the share that is (numerically) zero, per site."""
    out: dict[str, float] = {}
    for name, r in red.items():
        total = max(1.0, float(r.hist.sum()))
        edges = np.linspace(0.0, 1.0, len(r.hist) + 1)
        for thr in (0.1, 0.5, 0.9):
            out[f"ci_hist/{name}/frac_above_{thr}"] = float(r.hist[edges[:-1] >= thr - 1e-9].sum() / total)
        out[f"ci_hist/{name}/frac_in_lowest_bin"] = float(r.hist[0] / total)
    return out


def mean_ci_scalars(red: dict[str, SiteReduction], dead_below: float = 1e-6) -> dict[str, float]:
    out: dict[str, float] = {}
    for name, r in red.items():
        out[f"ci_mean/{name}/max"] = float(r.mean_ci.max())
        out[f"ci_mean/{name}/mean"] = float(r.mean_ci.mean())
        out[f"ci_mean/{name}/n_dead"] = float((r.mean_ci <= dead_below).sum())
    return out


def density_scalars(red: dict[str, SiteReduction]) -> dict[str, float]:
    out: dict[str, float] = {}
    for name, r in red.items():
        out[f"activation_density/{name}/alive_frac"] = float((r.density > 0).mean())
        out[f"activation_density/{name}/mean_density"] = float(r.density.mean())
        out[f"activation_density/{name}/max_density"] = float(r.density.max())
    return out


# ---- figures ----------------------------------------------------------------------------------------


def _resample(v: np.ndarray, n: int = 256) -> np.ndarray:
    """A curve (or the columns of a matrix) sampled at `n` evenly spaced indices, so sites of different widths
    tile into one figure."""
    idx = np.linspace(0, v.shape[-1] - 1, n).round().astype(int)
    return v[..., idx]


def render_figures(red: dict[str, SiteReduction], run_dir, step: int, which: set[str]) -> dict[str, str]:
    """PNG + arrays under `<run_dir>/figures/`: `ci_histograms`, `mean_ci` (sorted, linear and log10 scale),
    `activation_density` (histogram of per-component densities), `density_heatmap`. Returns `{figure: path}`."""
    if run_dir is None or not red:
        return {}
    names = list(red)
    out: dict[str, str] = {}
    if "ci_histograms" in which:
        png = figures.grid_of_heatmaps([np.log1p(red[n].hist)[None, :].repeat(12, 0) for n in names], cols=4, cell=3)
        p = figures.save_figure(run_dir, f"ci_histograms_step{step}", png, {n: red[n].hist for n in names})
        out["ci_histograms"] = str(p)
    if "mean_ci" in which:
        mats = []
        for n in names:
            srt = np.sort(red[n].mean_ci)[::-1]
            lin = srt / max(srt.max(), 1e-12)
            log = (np.log10(np.maximum(srt, 1e-8)) + 8.0) / 8.0
            mats.append(np.stack([_resample(lin)] * 6 + [_resample(log)] * 6))
        png = figures.grid_of_heatmaps(mats, cols=2, cell=2)
        p = figures.save_figure(run_dir, f"mean_ci_step{step}", png, {n: red[n].mean_ci for n in names})
        out["mean_ci"] = str(p)
    if "activation_density" in which:
        hists = [np.histogram(red[n].density, bins=100, range=(0.0, 1.0))[0].astype(np.float64) for n in names]
        png = figures.grid_of_heatmaps([np.log1p(h)[None, :].repeat(12, 0) for h in hists], cols=4, cell=3)
        p = figures.save_figure(run_dir, f"activation_density_step{step}", png, {n: red[n].density for n in names})
        out["activation_density"] = str(p)
    if "density_heatmap" in which and all(red[n].comp_hist is not None for n in names):
        mats = []
        for n in names:
            order = np.argsort(-red[n].mean_ci)
            mats.append(_resample(np.log1p(red[n].comp_hist[order]).T))  # bins x (components by mean CI)
        png = figures.grid_of_heatmaps(mats, cols=2, cell=2)
        p = figures.save_figure(run_dir, f"ci_density_heatmap_step{step}", png,
                                {n: red[n].comp_hist for n in names})
        out["density_heatmap"] = str(p)
    return out
