"""Loss functions of the decomposition objective (pure functions on tensors).

Parity map:
  relative squared error, categorical KL from logits      param_decomp/core/losses.py:59-92
  smooth-L0 importance minimality + frequency penalty      core/losses.py:375-485, configs.py:155-201
  EMA frequency estimator with first-order surrogate grad  core/losses.py:487-577
  L_p importance minimality with p-anneal                  nano_param_decomp/run.py:408-429
  faithfulness  mean_s ||W_s - (V_s U_s)^T||^2 / ||W_s||^2  core/faithfulness.py:16-104
  nonlinearity-locality soft unit count                    core/losses.py:180-313
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F
from torch import Tensor

from param_decomp_b200.core.components import ComponentStacks, SelectedCI
from param_decomp_b200.formats.nonlinearity import Neurons

# ---- output comparisons ------------------------------------------------------------------------


def relative_squared_error(pred: Tensor, target: Tensor, eps: float = 1e-8) -> Tensor:
    """Mean over positions of `||pred - target||^2 / max(||target||^2, eps)` (last axis = features)."""
    num = (pred.float() - target.float()).pow(2).sum(-1)
    den = target.float().pow(2).sum(-1).clamp_min(eps)
    return (num / den).mean()


def kl_from_logits(target_logits: Tensor, pred_logits: Tensor) -> Tensor:
    """`KL(softmax(target) || softmax(pred))`, mean over positions, fp32 accumulators."""
    t = F.log_softmax(target_logits.float(), dim=-1)
    p = F.log_softmax(pred_logits.float(), dim=-1)
    return (t.exp() * (t - p)).sum(-1).mean()


def mse(pred: Tensor, target: Tensor) -> Tensor:
    return (pred.float() - target.float()).pow(2).mean()


# ---- importance minimality ---------------------------------------------------------------------


def smooth_l0(c: Tensor, gamma: float | Tensor, normalize_at_one: bool) -> Tensor:
    """Geman-McClure `c^2 / (c^2 + gamma^2)`; times `1 + gamma^2` when normalised so psi(1) = 1."""
    c2 = c * c
    psi = c2 / (c2 + gamma * gamma)
    return psi * (1 + gamma * gamma) if normalize_at_one else psi


def component_activity(ci_upper: Tensor | SelectedCI, gamma: float | Tensor, normalize_at_one: bool,
                       n_positions: int | None = None) -> Tensor:
    """`f_c = mean over batch/positions of psi(ci_upper)`, shape `[C]` (local-batch mean)."""
    if isinstance(ci_upper, SelectedCI):
        psi = SelectedCI(smooth_l0(ci_upper.values.float(), gamma, normalize_at_one),
                         ci_upper.selection, ci_upper.n_blocks)
        n = n_positions or max(1, ci_upper.values.numel() // ci_upper.values.shape[-1])
        return psi.sum_per_component() / n
    psi = smooth_l0(ci_upper.float(), gamma, normalize_at_one)
    return psi.reshape(-1, psi.shape[-1]).mean(0)


def frequency_penalty(f: Tensor, reference_count: int) -> Tensor:
    """`sum_c f_c * log2(1 + a' f_c)`; zero at f = 0 by construction."""
    return (f * torch.log2(1 + reference_count * f)).sum()


@dataclass
class FrequencyEMA:
    """Debiased EMA of per-component firing frequency. The penalty is evaluated at the smoothed
    estimate while its gradient flows through the current batch's `f` at single-batch scale:
    `penalty(ema_detached) + <grad_penalty(ema_detached), f - f.detach()>`."""

    halflife_steps: float
    value: Tensor  # [C] running (biased) average
    weight: float = 0.0  # sum of decay weights, for debiasing

    @property
    def decay(self) -> float:
        return 0.5 ** (1.0 / self.halflife_steps)

    def update(self, f_batch: Tensor) -> Tensor:
        d = self.decay
        self.value = d * self.value + (1 - d) * f_batch.detach()
        self.weight = d * self.weight + (1 - d)
        return self.value / max(self.weight, 1e-12)

    def surrogate(self, f_batch: Tensor, reference_count: int) -> Tensor:
        smoothed = self.update(f_batch).detach().requires_grad_(True)
        with torch.enable_grad():
            pen = frequency_penalty(smoothed, reference_count)
            (g,) = torch.autograd.grad(pen, smoothed)
        return pen.detach() + (g.detach() * (f_batch - f_batch.detach())).sum()


def lp_importance_minimality(ci_upper: dict[str, Tensor], p: float, eps: float, beta: float,
                             world_size: int = 1, mean_over_ranks=None) -> Tensor:
    """Per site: `sum_c [mean_c + beta * mean_c * log2(1 + sum_c)]` of `(ci+eps)^p`, with `mean_c` / `sum_c`
    taken over the GLOBAL batch: `mean_over_ranks` is the differentiable mean over the batch shards (each
    holds the same number of rows), applied before the logarithm - a per-shard estimate inside the log is
    biased (Jensen) and would make a data-parallel run differ from the single-process one."""
    total = None
    for c in ci_upper.values():
        vals = (c.float() + eps).pow(p).reshape(-1, c.shape[-1])
        mean_c = vals.mean(0)
        if mean_over_ranks is not None and world_size > 1:
            mean_c = mean_over_ranks(mean_c)
        sum_c = mean_c * (vals.shape[0] * world_size)
        site = (mean_c + beta * mean_c * torch.log2(1 + sum_c)).sum()
        total = site if total is None else total + site
    assert total is not None
    return total


# ---- faithfulness ------------------------------------------------------------------------------


def weight_delta(W: Tensor, V: Tensor, U: Tensor) -> Tensor:
    """`W - (V U)^T` in fp32; blocked operands broadcast over the leading block axis."""
    return W.float() - (V.float() @ U.float()).transpose(-1, -2)


def faithfulness_loss(stacks: ComponentStacks, target_weights: dict[str, Tensor],
                      weight_sq_norms: dict[str, Tensor] | None = None, relative: bool = True) -> Tensor:
    """Reference form: mean over sites of `||Delta_s||_F^2 / ||W_s||_F^2`. `relative=False` is the
    paper form `sum ||Delta||^2 / sum numel`."""
    if not relative:
        num = sum(weight_delta(target_weights[s.name], *stacks.site(s.name)).pow(2).sum() for s in stacks.sites)
        den = sum(target_weights[s.name].numel() for s in stacks.sites)
        return num / den
    terms = []
    for s in stacks.sites:
        W = target_weights[s.name]
        wn = weight_sq_norms[s.name] if weight_sq_norms is not None else W.float().pow(2).sum()
        terms.append(weight_delta(W, *stacks.site(s.name)).pow(2).sum() / wn)
    return torch.stack(terms).mean()


def faithfulness_terms(stacks: ComponentStacks, target_weights: dict[str, Tensor],
                       weight_sq_norms: dict[str, Tensor], component_group=None) -> Tensor:
    """`[n_sites]`: `||Delta_s||_F^2 / ||W_s||_F^2` per site, in `stacks.sites` order. With
    `component_group` every rank holds a slice of each site's components: the products `V_r U_r` are
    summed over the group (each rank then sees the whole residual and the exact gradient of its slice)."""
    terms = []
    for s in stacks.sites:
        V, U = stacks.site(s.name)
        W = target_weights[s.name]
        if component_group is not None:
            from param_decomp_b200.parallel.group_ops import ReduceFromGroup

            delta = W.float() - ReduceFromGroup.apply(V.float() @ U.float(), component_group).transpose(-1, -2)
        else:
            delta = weight_delta(W, V, U)
        terms.append(delta.pow(2).sum() / weight_sq_norms[s.name])
    return torch.stack(terms)


# ---- nonlinearity locality -----------------------------------------------------------------------


def nonlinearity_locality(stacks: ComponentStacks, relative_threshold: float,
                          unit_kind_coefficients: dict[str, float | None], normalize_at_one: bool,
                          expert_shard=None, split_grad_scale: float = 1.0) -> Tensor:
    """Soft count of nonlinearity units each component touches, averaged per unit kind.

    For a site whose `alignment.side` faces a nonlinearity, take the component vectors on that side
    (`U` rows for "output", `V` columns for "input"), split them into units (neurons, or contiguous
    head blocks), form each unit's energy share `e_u = ||v_u||^2 / ||v||^2`, and count units softly
    with `e^2 / (e^2 + tau^2)`, `tau = relative_threshold / n_units` (relative to the uniform share).

    `expert_shard` (`parallel/expert_shard.py::StackSharding`, expert mode): this rank holds only its experts'
    blocks of the blocked sites (padding experts excluded here) and every component of the other sites. A kind's
    mean is then taken over ALL of the job's components: split sums and counts are added over the group. The
    returned value is that job-wide mean; its gradient is the local part's, with the split sites' share scaled by
    `split_grad_scale` (see `DistCollectives.split_grad_scale`).
    """
    by_expert = expert_shard is not None and not expert_shard.by_component
    per_kind: dict[str, list[Tensor]] = {}
    per_kind_split: dict[str, list[Tensor]] = {}
    for s in stacks.sites:
        al = s.alignment
        if al is None:
            continue
        kind = al.partition.unit_kind
        coeff = unit_kind_coefficients.get(kind)
        assert kind in unit_kind_coefficients, f"unit_kind_coefficients must name {kind!r}"
        if coeff is None:
            continue
        V, U = stacks.site(s.name)
        vecs = U if al.side == "output" else V.transpose(-1, -2)  # [C, width]
        vecs = vecs.reshape(-1, vecs.shape[-1]).float()
        width = vecs.shape[-1]
        n_units = width if isinstance(al.partition, Neurons) else al.partition.head_count
        energy = vecs.pow(2).reshape(vecs.shape[0], n_units, width // n_units).sum(-1)
        share = energy / energy.sum(-1, keepdim=True).clamp_min(1e-20)
        tau = relative_threshold / n_units
        count = (share.pow(2) / (share.pow(2) + tau * tau)).sum(-1)
        if normalize_at_one:
            count = count * (1 + tau * tau)
        mult = getattr(al.partition, "use_multiplicity", 1)
        if by_expert and s.blocked:
            real = expert_shard.n_real * s.C_block  # blocks of padding experts sit at the end and are not components
            per_kind_split.setdefault(kind, []).append(count[:real] * mult)
        else:
            per_kind.setdefault(kind, []).append(count * mult)
    total = None
    if by_expert:
        kinds = sorted(set(per_kind) | set(per_kind_split))
        if kinds:
            dev = next(stacks.parameters()).device
            zero = torch.zeros((), device=dev)
            rep = torch.stack([torch.cat(per_kind[k]).sum() if k in per_kind else zero for k in kinds])
            spl = torch.stack([torch.cat(per_kind_split[k]).sum() if k in per_kind_split else zero for k in kinds])
            n_rep = torch.tensor([sum(c.numel() for c in per_kind.get(k, [])) for k in kinds], device=dev, dtype=rep.dtype)
            n_spl = torch.tensor([sum(c.numel() for c in per_kind_split.get(k, [])) for k in kinds], device=dev, dtype=rep.dtype)
            group_wide = expert_shard.sum_over_group(torch.stack([spl.detach(), n_spl]))
            n_all = (n_rep + group_wide[1]).clamp_min(1.0)
            coeffs = torch.tensor([float(unit_kind_coefficients[k]) for k in kinds], device=dev, dtype=rep.dtype)  # type: ignore[arg-type]
            value = (((rep.detach() + group_wide[0]) / n_all) * coeffs).sum()
            local = (((rep + split_grad_scale * spl) / n_all) * coeffs).sum()
            return value + (local - local.detach())
    for kind, counts in per_kind.items():
        val = torch.cat(counts).mean() * float(unit_kind_coefficients[kind])  # type: ignore[arg-type]
        total = val if total is None else total + val
    if total is None:
        p = next(stacks.parameters())
        return p.new_zeros(())
    return total


def anneal_linear(start: float, end: float, frac: float) -> float:
    return start + (end - start) * frac


def geman_mcclure_max_slope(gamma: float) -> float:
    """Largest derivative of `c^2/(c^2+gamma^2)` (at c = gamma/sqrt(3)): `3*sqrt(3)/(8*gamma)`."""
    return 3 * math.sqrt(3) / (8 * gamma)
