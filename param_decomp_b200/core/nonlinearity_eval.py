"""Standing nonlinearity evaluation: how many nonlinearity units (neurons, heads) each component's
aligned vector touches.

Two statistics per component, both scaled by the partition's use multiplicity (under GQA a kv block
feeds `n_head / n_kv_head` query heads): the fixed-threshold soft use count the locality loss
penalises, and the L1 effective count `(sum_u r_u)^2 / sum_u r_u^2` of unit-block norms `r_u`.
Parity: param_decomp/core/nonlinearity_eval.py.
"""

from __future__ import annotations

import torch
from torch import Tensor

from param_decomp_b200.core.components import ComponentStacks
from param_decomp_b200.formats.nonlinearity import Neurons


@torch.no_grad()
def component_nonlinearity_stats(stacks: ComponentStacks, relative_threshold: float = 1.0) -> dict[str, dict[str, Tensor]]:
    """`{site: {"soft_count": [C], "effective_count": [C], "unit_kind": str}}` for aligned sites."""
    out: dict[str, dict[str, Tensor]] = {}
    for s in stacks.sites:
        al = s.alignment
        if al is None:
            continue
        V, U = stacks.site(s.name)
        vecs = (U if al.side == "output" else V.transpose(-1, -2)).reshape(-1, (U if al.side == "output" else V.transpose(-1, -2)).shape[-1]).float()
        width = vecs.shape[-1]
        n_units = width if isinstance(al.partition, Neurons) else al.partition.head_count
        if width % n_units:
            continue
        block = vecs.reshape(vecs.shape[0], n_units, width // n_units)
        r = torch.linalg.vector_norm(block, dim=-1)  # [C, units]
        energy = r.pow(2)
        share = energy / energy.sum(-1, keepdim=True).clamp_min(1e-20)
        tau = relative_threshold / n_units
        mult = getattr(al.partition, "use_multiplicity", 1)
        out[s.name] = {
            "soft_count": (share.pow(2) / (share.pow(2) + tau * tau)).sum(-1) * mult,
            "effective_count": r.sum(-1).pow(2) / energy.sum(-1).clamp_min(1e-20) * mult,
            "unit_kind": al.partition.unit_kind,  # type: ignore[dict-item]
        }
    return out


def nonlinearity_log_entries(stats: dict[str, dict[str, Tensor]], mean_ci: dict[str, Tensor] | None = None) -> dict[str, float]:
    """Site and unit-kind means, over all components and over those with positive mean CI."""
    out: dict[str, float] = {}
    by_kind: dict[str, list[Tensor]] = {}
    for site, st in stats.items():
        for key in ("soft_count", "effective_count"):
            v = st[key]
            out[f"nonlinearity/{key}/{site}"] = float(v.mean())
            if mean_ci is not None and site in mean_ci:
                alive = mean_ci[site].reshape(-1) > 0
                if alive.any():
                    out[f"nonlinearity/{key}/{site}/alive"] = float(v[alive].mean())
        by_kind.setdefault(str(st["unit_kind"]), []).append(st["effective_count"])
    for kind, vals in by_kind.items():
        out[f"nonlinearity/effective_count/{kind}"] = float(torch.cat(vals).mean())
    return out
