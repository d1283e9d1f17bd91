"""A component's two activations, and the scale symmetry between its factors.

Component `c` adds `(x V[:, c]) U[c, :]` to its site's output; `U[c] -> a U[c]`, `V[:, c] -> V[:, c] / a`
changes nothing the network computes. So `x V[:, c]` (gauge-VARIANT) depends on how the pair happens
to be scaled, while `(x V[:, c]) ||U[c]||` (gauge-INVARIANT) is the size of the contribution itself.
Parity: param_decomp/core/gauge.py (activations), core/train.py:234-261 (norm-ratio metrics).
"""

from __future__ import annotations

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
def uv_norm_ratio_metrics(components: ComponentStacks) -> dict[str, float]:
    """Per site `||U||_F / ||V||_F`, plus mean and max: drift of the pair's scale during training."""
    out: dict[str, float] = {}
    ratios = []
    for s in components.sites:
        V, U = components.site(s.name)
        r = float(torch.sqrt(U.float().pow(2).sum() / V.float().pow(2).sum().clamp_min(1e-30)))
        out[f"uv_norm_ratio['{s.name}']"] = r
        ratios.append(r)
    if ratios:
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
