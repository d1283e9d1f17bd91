"""Slow-tier LM evaluation operations: router divergence, well-temperedness, the arithmetic CI grid,
CI histograms / permutation figures.

Every operation is `op(ctx, state, batch, cfg, run_dir) -> {key: float}`; figures go to
`<run_dir>/figures/` as PNG + the arrays behind them (`utils/figures.py`).

Parity: param_decomp/experiments/lm/router_divergence_eval.py (per-layer router drift under pinned
routing), well_temperedness.py (ordering of CI pre-activations vs single-component ablation damage,
by region), arithmetic_probe.py + arithmetic_eval.py (operand grid, per-component CI / activation
heat maps), diagnostic_eval_operations.py (site figures, permutation), core/slow_eval.py:494-551.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

import numpy as np
import torch
from torch import Tensor

from param_decomp_b200.core import masking
from param_decomp_b200.core.components import prepare_compute_weights
from param_decomp_b200.core.rng import StepKey
from param_decomp_b200.core.train import StepContext, TrainState, run_ci_fn
from param_decomp_b200.utils import figures


# ---- router divergence ------------------------------------------------------------------------------

def _router_keys(model: Any) -> tuple[str, ...]:
    return tuple(f"router_probs.{i}" for i in range(model.arch.n_layer))


@torch.no_grad()
def _strategy_masks(ctx: StepContext, state: TrainState, batch: Any, clean, ci, weights, strat) -> dict | None:
    """Masks of one evaluation masking strategy (`config/evals.py`: `ci_masked`, `stochastic`, `fresh_pgd`,
    `persistent`); `strat` may also be the bare kind of the two that need no parameters."""
    from param_decomp_b200.core import adversary as adv_mod
    from param_decomp_b200.core.objective import ReconTerm
    from param_decomp_b200.core.train import masked_recon, reduce_source_grads

    kind = strat if isinstance(strat, str) else strat.kind
    if kind == "ci_masked":
        return masking.ci_masks(ci.mask_inputs())
    if kind == "stochastic":
        from param_decomp_b200.evals.lm import global_row_offset

        inputs = ci.mask_inputs()
        return masking.stochastic_masks(inputs, StepKey(0xE7A3, 0), 0, 0, site_index=ctx.site_index,
                                        row_offset=global_row_offset(ctx, inputs), lazy=False)
    ci_lower = ci.mask_inputs()
    lead = tuple(next(iter(ci_lower.values())).shape[:-1])
    positions = lead[1] if ctx.model.has_position_axis and len(lead) > 1 else None
    device = next(iter(ci_lower.values())).device
    sites = getattr(ctx.model, "global_sites", ctx.model.sites)
    if kind == "fresh_pgd":
        # batch-shared sources, random init, sign ascent against the output loss (param_decomp/core/recon_eval.py:142-257)
        from types import SimpleNamespace

        leaves = adv_mod.fresh_sources(sites, "random", "c", lead[0], positions, StepKey(0xE7A4, 0), 14, device)
        term = ReconTerm(name="eval_router_pgd", index=14, strategy="fresh_pgd", cfg=SimpleNamespace(auxiliaries=()))  # type: ignore[arg-type]
        w_d = weights
        with torch.enable_grad():
            for _ in range(strat.n_steps):
                src, dlt = adv_mod.PersistentAdversary.split(leaves)
                e2e, _ = masked_recon(ctx, w_d, batch, clean, masking.source_masks(ci_lower, src, dlt), term, 0, with_aux=False)
                names = list(leaves)
                gs = torch.autograd.grad(e2e, [leaves[k] for k in names], allow_unused=True)
                adv_mod.sign_ascent_(leaves, reduce_source_grads(ctx, {
                    k: (g if g is not None else torch.zeros_like(leaves[k])) for k, g in zip(names, gs)}, True),
                    strat.step_size)
        src, dlt = adv_mod.PersistentAdversary.split({k: v.detach() for k, v in leaves.items()})
        return masking.source_masks(ci_lower, src, dlt)
    if kind == "persistent":
        adv = state.adversaries.get(strat.state_key)
        assert adv is not None, (f"RouterDivergence persistent strategy names state_key {strat.state_key!r}, but the "
                                 f"run's persistent terms are {sorted(state.adversaries)}")
        leaves = {k: v.detach() for k, v in adv.leaves().items()}
        if adv.pool_size > 1:  # one particle per row, as training samples them
            pick = torch.zeros(next(iter(leaves.values())).shape[0], dtype=torch.long, device=device)
            leaves = adv.select_particles(leaves, pick)
        rows = next(iter(leaves.values())).shape[0]
        if not adv.batch_shared and rows != lead[0]:
            # per-row sources index TRAINING rows: every evaluation sequence draws one of them, fixed across evaluations
            g = torch.Generator().manual_seed(0xE7A5)
            idx = torch.randint(0, rows, (lead[0],), generator=g).to(device)
            leaves = {k: v.index_select(0, idx) for k, v in leaves.items()}
        src, dlt = adv_mod.PersistentAdversary.split(leaves)
        return masking.source_masks(ci_lower, src, dlt)
    raise ValueError(kind)


def router_divergence(ctx: StepContext, state: TrainState, batch: Any, strategies: tuple = ("ci_masked",),
                      ) -> dict[str, float]:
    """Per MoE layer and masking strategy: KL(target router || masked router) per token, the share of
    the target's top-k the masked router would still select (a counterfactual read-out: the forward
    itself stays pinned to the target's experts), and the L1 distance of the applied mixing weights.
    `strategies`: `config/evals.py` strategy objects (or bare kinds for the parameter-free two)."""
    model = ctx.model
    assert hasattr(model, "expert_site_names"), "router divergence needs a target with an expert router"
    keys = _router_keys(model)
    clean = model.clean_forward(batch, capture=keys)
    if not all(k in clean.captures for k in keys):
        return {}
    weights = prepare_compute_weights(state.components, model.compute_dtype).detached()
    ci = run_ci_fn(ctx, state, clean)
    out: dict[str, float] = {}
    k = model.arch.experts_per_token
    for strategy in strategies:
        strat = strategy if isinstance(strategy, str) else strategy.kind
        masks = _strategy_masks(ctx, state, batch, clean, ci, weights, strategy)
        res = model.masked_forward(weights, batch, masks, capture=keys, clean=clean)
        per_layer = []
        for i, key in enumerate(keys):
            p, q = clean.captures[key].float(), res.captures[key].float()
            kl = (p * (torch.log(p.clamp_min(1e-30)) - torch.log(q.clamp_min(1e-30)))).sum(-1)
            top_p, top_q = p.topk(k, dim=-1).indices, q.topk(k, dim=-1).indices
            kept = (top_p.unsqueeze(-1) == top_q.unsqueeze(-2)).any(-1).float().mean(-1)
            wp = p.gather(-1, top_p)
            wq = q.gather(-1, top_p)  # masked weights at the PINNED experts
            l1 = (wp / wp.sum(-1, keepdim=True) - wq / wq.sum(-1, keepdim=True)).abs().sum(-1)
            out[f"RouterDivergence/{strat}/kl/layer_{i}"] = float(kl.mean())
            out[f"RouterDivergence/{strat}/topk_kept/layer_{i}"] = float(kept.mean())
            out[f"RouterDivergence/{strat}/weight_l1/layer_{i}"] = float(l1.mean())
            per_layer.append(float(kl.mean()))
        out[f"RouterDivergence/{strat}/kl"] = sum(per_layer) / max(len(per_layer), 1)
    return out


# ---- well-temperedness -----------------------------------------------------------------------------

def in_region(pre: Tensor, region: str) -> Tensor:
    if region == "below_zero":
        return pre < 0
    if region == "zero_to_one":
        return (pre >= 0) & (pre <= 1)
    return pre > 1


def fraction_well_ordered_pairs(pre: Tensor, damage: Tensor) -> float:
    """Over all pairs with different pre-activations: how often the larger pre-activation also has
    the larger ablation damage (ties in damage count half). 0.5 = random, 1 = perfectly ordered."""
    n = pre.numel()
    if n < 2:
        return float("nan")
    dp = pre[:, None] - pre[None, :]
    dd = damage[:, None] - damage[None, :]
    valid = dp > 0
    if not valid.any():
        return float("nan")
    good = ((dd > 0) & valid).float().sum() + 0.5 * ((dd == 0) & valid).float().sum()
    return float(good / valid.float().sum())


@torch.no_grad()
def well_temperedness(ctx: StepContext, state: TrainState, batch: Any, n_locations: int = 4,
                      n_components: int = 16, seed: int = 0, run_dir: Any = None,
                      groups: dict[str, list[str]] | None = None) -> dict[str, float]:
    """Whether higher CI pre-activations mean greater ablation effects. At `n_locations` sampled (sequence,
    position) locations components are ablated one at a time (mask 1 everywhere, 0 for that component at that
    position) and the output change AT that position is scored. Sampling is stratified by the pre-activation's
    region at the location (`below_zero`, `zero_to_one`, `above_one`): every region schedules `n_components`
    ablations per location and pads a sparse region with out-of-region components whose damage is computed and
    discarded, so the number of forwards does not depend on the data. `groups` maps names to fnmatch patterns of
    site names; each group gets its own scores (param_decomp/experiments/lm/well_temperedness.py,
    eval_config.py:141-156)."""
    import fnmatch

    model = ctx.model
    B, T = batch.tokens.shape
    g = torch.Generator().manual_seed(seed + ctx.collectives.row_offset(B))  # every batch shard samples its own rows
    clean = model.clean_forward(batch)
    ci = run_ci_fn(ctx, state, clean)
    dense_sites = [s for s in model.sites if not s.blocked]
    if not dense_sites:
        return {}
    weights = prepare_compute_weights(state.components, model.compute_dtype).detached()
    lower = ci.mask_inputs()
    ones = {k: torch.ones_like(v) for k, v in lower.items()}
    base = model.masked_forward(weights, batch, masking.ci_masks(ones), clean=clean).output
    regions = ("below_zero", "zero_to_one", "above_one")
    pres, dmg, site_of = [], [], []
    for _ in range(n_locations):
        b, t = int(torch.randint(B, (1,), generator=g)), int(torch.randint(T, (1,), generator=g))
        pre_here = torch.cat([ci.preactivations[s.name][b, t].float().reshape(-1) for s in dense_sites])
        owner = torch.cat([torch.full((s.C,), i) for i, s in enumerate(dense_sites)])
        first = torch.tensor([0] + [s.C for s in dense_sites]).cumsum(0)
        for region in regions:
            inside = in_region(pre_here, region).nonzero()[:, 0]
            take = inside[torch.randperm(inside.numel(), generator=g)[:n_components]]
            pad = n_components - take.numel()  # a sparse region: its quota is filled with components that do not count
            padded = torch.cat([take, torch.randint(pre_here.numel(), (pad,), generator=g)]) if pad else take
            for j, flat in enumerate(padded.tolist()):
                si = int(owner[flat])
                site, c = dense_sites[si], flat - int(first[si])
                m = {k: v.clone() if k == site.name else v for k, v in ones.items()}
                m[site.name][b, t, c] = 0.0
                out = model.masked_forward(weights, batch, masking.ci_masks(m), clean=clean).output
                if j >= take.numel():
                    continue  # padding: computed, discarded
                a_, r_ = out[b, t].float(), base[b, t].float()
                dmg.append(float((a_ - r_).pow(2).sum() / r_.pow(2).sum().clamp_min(1e-30)))
                pres.append(float(pre_here[flat]))
                site_of.append(site.name)
    # The score is a statistic of PAIRS, so it is formed once from every batch shard's ablations together (a mean
    # over ranks of per-rank pair fractions would weight ranks equally whatever they sampled, and one rank with
    # fewer than two ablations would turn it into NaN). Shards contribute a fixed-size, NaN-padded table.
    site_names = [s.name for s in dense_sites]
    quota = n_locations * len(regions) * n_components
    table = torch.full((quota, 3), float("nan"), dtype=torch.float64)
    if pres:
        table[:len(pres)] = torch.tensor([[p, d, float(site_names.index(sn))] for p, d, sn in zip(pres, dmg, site_of)],
                                         dtype=torch.float64)
    dev = next(state.components.parameters()).device
    table = ctx.collectives.gather_rows(table.to(dev)).cpu()
    table = table[~table[:, 0].isnan()]
    pre_t, dmg_t = table[:, 0].float(), table[:, 1].float()
    site_of = [site_names[int(i)] for i in table[:, 2].tolist()]
    res = {"WellTemperedness/all": fraction_well_ordered_pairs(pre_t, dmg_t)}
    for region in regions:
        sel = in_region(pre_t, region)
        res[f"WellTemperedness/{region}"] = fraction_well_ordered_pairs(pre_t[sel], dmg_t[sel])
        res[f"WellTemperedness/{region}/n"] = float(sel.sum())
    for name, patterns in (groups or {}).items():
        sel = torch.tensor([any(fnmatch.fnmatch(sn, p) for p in patterns) for sn in site_of], dtype=torch.bool)
        res[f"WellTemperedness/group/{name}"] = fraction_well_ordered_pairs(pre_t[sel], dmg_t[sel])
        res[f"WellTemperedness/group/{name}/n"] = float(sel.sum())
    figures.save_figure(run_dir, "well_temperedness_pre_vs_damage",
                        figures.scatter(pre_t.numpy(), np.log10(dmg_t.numpy() + 1e-30)),
                        {"preactivation": pre_t.numpy(), "damage": dmg_t.numpy()})
    return res


# ---- arithmetic grid --------------------------------------------------------------------------------

@dataclass
class ArithmeticPromptGrid:
    tokens: Tensor        # [A * B, L] row-major (a, b)
    a_values: list[int]
    b_values: list[int]
    answers: list[int]


def inclusive_range(bounds: tuple[int, int]) -> list[int]:
    """`(lo, hi)` of a config's `a_range` / `b_range` as the operand list `lo..hi`, both ends included."""
    vals = list(range(int(bounds[0]), int(bounds[1]) + 1))
    assert vals, f"empty operand range {bounds}"
    return vals


def build_arithmetic_prompt_grid(encode: Callable[[str], list[int]], a_values: list[int], b_values: list[int],
                                 operation: str = "add", modulus: int | None = None) -> ArithmeticPromptGrid:
    """`"<a><symbol><b>="` prompts, one per row, all rows one shared token length (refused otherwise:
    padding would shift the answer position)."""
    sym = {"add": "+", "sub": "-", "mul": "*"}[operation]
    fn = {"add": lambda a, b: a + b, "sub": lambda a, b: a - b, "mul": lambda a, b: a * b}[operation]
    rows, answers = [], []
    for a in a_values:
        for b in b_values:
            rows.append(encode(f"{a}{sym}{b}="))
            ans = fn(a, b)
            answers.append(ans % modulus if modulus else ans)
    lengths = {len(r) for r in rows}
    assert len(lengths) == 1, f"arithmetic prompts tokenise to different lengths {sorted(lengths)}"
    return ArithmeticPromptGrid(torch.tensor(rows, dtype=torch.int64), list(a_values), list(b_values), answers)


@torch.no_grad()
def arithmetic_ci_grid(ctx: StepContext, state: TrainState, grid: ArithmeticPromptGrid, top_k: int = 24,
                       run_dir: Any = None, thresholds: tuple[float, ...] = (0.1,), probe_metrics: Any = None,
                       ) -> dict[str, float]:
    """Per site: CI of every component at the `=` position as an `a x b` heat map; the `top_k`
    components by mean CI are drawn. Returns alive counts (mean CI above 0.01, and above each of `thresholds`)
    and, with `probe_metrics` (`config/evals.py::ArithmeticProbeMetrics`), the scalar operations evaluated on
    the grid's prompts instead of corpus batches: the six-mask CE / KL table, CI-L0 per site or group, and
    optionally a fresh-PGD reconstruction (param_decomp/experiments/lm/arithmetic_eval_operation.py)."""
    from param_decomp_b200.models.transformer import LMBatch

    model = ctx.model
    dev = next(iter(state.components.parameters())).device
    batch = LMBatch(grid.tokens.to(dev))
    clean = model.clean_forward(batch)
    ci = run_ci_fn(ctx, state, clean).dense_lower()
    A, Bn = len(grid.a_values), len(grid.b_values)
    out: dict[str, float] = {}
    if probe_metrics is not None:
        from param_decomp_b200.evals.core import ci_l0, fresh_pgd_recon
        from param_decomp_b200.evals.lm import ce_and_kl

        for k, v in ce_and_kl(ctx, state, batch, probe_metrics.ce_kl.rounding_threshold).items():
            out[f"ArithmeticCIGrid/probe/{k}"] = v
        for k, v in ci_l0(ci, probe_metrics.ci_l0.ci_alive_threshold, probe_metrics.ci_l0.groups).items():
            out[f"ArithmeticCIGrid/probe/{k}"] = v
        if probe_metrics.fresh_pgd is not None:
            with torch.enable_grad():
                res = fresh_pgd_recon(ctx, state, batch, probe_metrics.fresh_pgd.step_size,
                                      (probe_metrics.fresh_pgd.n_steps,), StepKey(0xE7A6, 0))
            out[f"ArithmeticCIGrid/probe/PGDReconLoss_{probe_metrics.fresh_pgd.n_steps}step"] = \
                res[probe_metrics.fresh_pgd.n_steps]["loss"]
    for site, v in ci.items():
        last = v[:, -1].float().reshape(A, Bn, -1)  # [A, B, C]
        mean = last.mean((0, 1))
        out[f"ArithmeticCIGrid/{site}/n_alive"] = float((mean > 0.01).sum())
        for thr in thresholds:
            out[f"ArithmeticCIGrid/{site}/n_above_{thr:g}"] = float((last > thr).any(0).any(0).sum())
        top = mean.topk(min(top_k, mean.numel())).indices
        mats = [last[:, :, int(c)].cpu().numpy() for c in top]
        figures.save_figure(run_dir, f"arithmetic_ci_{site}", figures.grid_of_heatmaps(mats),
                            {"ci": torch.stack([last[:, :, int(c)] for c in top]).cpu().numpy(),
                             "components": top.cpu().numpy()})
    return out


# ---- CI figures ------------------------------------------------------------------------------------

@torch.no_grad()
def ci_histogram_figures(ci_lower: dict[str, Tensor], run_dir: Any, bins: int = 50) -> dict[str, float]:
    out: dict[str, float] = {}
    for site, v in ci_lower.items():
        counts = torch.histc(v.float().clamp(0, 1), bins=bins, min=0.0, max=1.0).cpu().numpy()
        figures.save_figure(run_dir, f"ci_hist_{site}", figures.histogram(counts), {"counts": counts})
        out[f"ci_hist/{site}/frac_above_0.5"] = float((v > 0.5).float().mean())
    return out


def permute_to_identity(ci: Tensor) -> tuple[Tensor, Tensor]:
    """Reorder components so the `[features, C]` CI matrix is as diagonal as possible
    (Hungarian assignment on `-CI`); returns the permuted matrix and the permutation."""
    from scipy.optimize import linear_sum_assignment

    m = ci.float().cpu().numpy()
    rows, cols = linear_sum_assignment(-m)
    rest = [c for c in range(m.shape[1]) if c not in set(cols.tolist())]
    perm = np.concatenate([cols[np.argsort(rows)], np.array(rest, dtype=int)])
    return torch.from_numpy(m[:, perm]), torch.from_numpy(perm)


def permuted_ci_figure(ci_by_site: dict[str, Tensor], run_dir: Any) -> None:
    """`ci_by_site[s]`: CI of single-feature probes `[features, C]` (toys)."""
    for site, m in ci_by_site.items():
        pm, perm = permute_to_identity(m)
        figures.save_figure(run_dir, f"permuted_ci_{site}", figures.heatmap(pm.numpy(), cell=6, vmin=0.0, vmax=1.0),
                            {"ci": pm.numpy(), "permutation": perm.numpy()})


def uv_figures(components: Any, sites: tuple[str, ...], run_dir: Any) -> None:
    """`V` and `U^T` of each site as heat maps (the toys' UV plots)."""
    for s in sites:
        V, U = components.site(s)
        if V.dim() != 2:
            continue
        figures.save_figure(run_dir, f"uv_{s}_V", figures.heatmap(V.detach().float().cpu().numpy(), cell=4))
        figures.save_figure(run_dir, f"uv_{s}_U", figures.heatmap(U.detach().float().cpu().numpy().T, cell=4))
