"""A component's two activations, and the scale symmetry between its factors.

Component `c` adds `(x V[:, c]) U[c, :]` to its site's output; `U[c] -> a U[c]`, `V[:, c] -> V[:, c] / a`
changes nothing the network computes. So `x V[:, c]` (gauge-VARIANT) depends on how the pair happens
to be scaled, while `(x V[:, c]) ||U[c]||` (gauge-INVARIANT) is the size of the contribution itself.
Parity: param_decomp/core/gauge.py (activations), core/train.py:234-261 (norm-ratio metrics).
"""

from __future__ import annotations

from typing import Any

import torch
from torch import Tensor

from param_decomp_b200.core.components import ComponentStacks


def u_norms_of(U: Tensor) -> Tensor:
    """`||U[c]||` per component (row norms, fp32 accumulation): `[..., C, d_out] -> [..., C]`."""
    return torch.linalg.vector_norm(U, dim=-1, dtype=torch.float32)


def gauge_invariant_activation(activation: Tensor, u_norm: Tensor) -> Tensor:
    return activation.float() * u_norm


def gauge_variant_activation(invariant: Tensor, u_norm: Tensor) -> Tensor:
    assert bool((u_norm > 0).all()), "a component with U[c] = 0 has no gauge-variant activation"
    return invariant.float() / u_norm


@torch.no_grad()
def uv_norm_ratio_metrics(components: ComponentStacks, shard: Any = None) -> dict[str, float]:
    """Per site `||U||_F / ||V||_F`, plus mean and max: drift of the pair's scale during training.
    `shard` (`parallel/expert_shard.py::StackSharding`): stacks it marks as split hold only this rank's experts or
    component slice, so their sums of squares are added over its group before the ratio is taken."""
    if not components.sites:
        return {}
    sq = torch.stack([torch.stack([U.float().pow(2).sum(), V.float().pow(2).sum()])
                      for V, U in (components.site(s.name) for s in components.sites)])  # [sites, (U, V)]
    if shard is not None:
        import torch.distributed as dist

        split = torch.tensor([ComponentStacks.param_key(s.group) in shard.blocked_keys for s in components.sites],
                             device=sq.device)
        total = sq.clone()
        dist.all_reduce(total, group=shard.group)
        sq = torch.where(split[:, None], total, sq)
    ratios = torch.sqrt(sq[:, 0] / sq[:, 1].clamp_min(1e-30)).tolist()
    out = {f"uv_norm_ratio['{s.name}']": r for s, r in zip(components.sites, ratios)}
    out["uv_norm_ratio_mean"] = sum(ratios) / len(ratios)
    out["uv_norm_ratio_max"] = max(ratios)
    return out


@torch.no_grad()
def balance(components: ComponentStacks) -> None:
    """Move every component to the balanced gauge `||V[:, c]|| = ||U[c]||` (function unchanged)."""
    for s in components.sites:
        V, U = components.site(s.name)
        vn = torch.linalg.vector_norm(V, dim=-2, dtype=torch.float32).clamp_min(1e-20)  # [..., C]
        un = u_norms_of(U).clamp_min(1e-20)
        a = torch.sqrt(vn / un)  # U *= a, V /= a
        U.mul_(a.unsqueeze(-1).to(U.dtype))
        V.div_(a.unsqueeze(-2).to(V.dtype))
