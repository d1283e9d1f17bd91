"""The decomposed-linear primitive (eager reference implementation).

    out = ((x V) * (m - d)) U + d * (x W^T);   out = where(route, out, x W^T)

The residual `W - (VU)^T` is never formed: its contribution `d * x (W - (VU)^T)^T` is folded into
the coefficient `m - d` on the component path plus `d * (x W^T)`.

Parity: param_decomp/core/decomposed_linear.py:65-85,142-175 (dense), :209-271 (blocked).
The fused sm_100a implementation of the same contract is `ops/site_linear.py`.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import Tensor

from param_decomp_b200.core.masking import SiteMask


def site_forward_split(x: Tensor, V: Tensor, U: Tensor, W: Tensor | None, sm: SiteMask, group,
                       bias: Tensor | None = None) -> Tensor:
    """The same contract with the component axis split over `group`: `V [d_in, C / W]`, `U [C / W, d_out]`
    are this rank's columns / rows, `sm` is the whole site's mask (replicated). Each rank contracts over
    its own components; the partial outputs are summed over the group and the target term, which does not
    depend on the components, is added once (param_decomp/core/decomposed_linear.py:142-175)."""
    from param_decomp_b200.parallel.group_ops import ReduceFromGroup, copy_to_group

    sm = sm.column_shard(group).materialize()
    h = copy_to_group(x, group) @ V.to(x.dtype)
    coef = sm.mask
    if sm.delta is not None:
        d = copy_to_group(sm.delta, group)  # its gradient through the component path is partial per rank
        coef = (coef - d) if coef is not None else (1.0 - d)
    if coef is not None:
        h = h * coef.to(h.dtype)
    out = ReduceFromGroup.apply(h @ U.to(x.dtype), group)
    return _target_term(out, x, W, sm, bias)


def _target_term(out: Tensor, x: Tensor, W: Tensor | None, sm: SiteMask, bias: Tensor | None) -> Tensor:
    if sm.delta is not None or sm.route is not None:
        assert W is not None, "delta masks and partial routing need the frozen weight"
        xw = F.linear(x, W.to(x.dtype))
        if sm.delta is not None:
            out = out + sm.delta.to(out.dtype) * xw
        if sm.route is not None:
            out = torch.where(sm.route.unsqueeze(-1), out, xw)
    if bias is not None:
        out = out + bias.to(out.dtype)
    return out


def site_forward(x: Tensor, V: Tensor, U: Tensor, W: Tensor | None, sm: SiteMask,
                 bias: Tensor | None = None) -> Tensor:
    """`x [..., d_in]`, `V [d_in, C]`, `U [C, d_out]`, `W [d_out, d_in]` (needed iff delta/route)."""
    sm = sm.materialize()
    h = x @ V.to(x.dtype)
    coef = sm.mask if sm.mask is not None else None
    if sm.delta is not None:
        coef = (coef - sm.delta) if coef is not None else (1.0 - sm.delta)
    if coef is not None:
        h = h * coef.to(h.dtype)
    out = h @ U.to(x.dtype)
    need_w = sm.delta is not None or sm.route is not None
    if need_w:
        assert W is not None, "delta masks and partial routing need the frozen weight"
        xw = F.linear(x, W.to(x.dtype))
        if sm.delta is not None:
            out = out + sm.delta.to(out.dtype) * xw
        if sm.route is not None:
            out = torch.where(sm.route.unsqueeze(-1), out, xw)
    if bias is not None:
        out = out + bias.to(out.dtype)
    return out


def blocked_site_forward(x_jobs: Tensor, block_of_job: Tensor, V: Tensor, U: Tensor, W: Tensor | None,
                         mask_jobs: Tensor | None, delta_jobs: Tensor | None,
                         route_jobs: Tensor | None = None) -> Tensor:
    """Blocked (per-expert) site on a flat list of jobs (token-expert pairs).

    `x_jobs [J, d_in]`, `block_of_job [J]`, `V [E, d_in, c]`, `U [E, c, d_out]`, `W [E, d_out, d_in]`,
    `mask_jobs [J, c]` (the job's block slice of the site mask), `delta_jobs [J, 1]`.
    Dense-gather oracle: O(J * d * c) memory; the grouped kernels avoid the gathers.
    """
    Vj = V[block_of_job].to(x_jobs.dtype)  # [J, d_in, c]
    Uj = U[block_of_job].to(x_jobs.dtype)
    h = torch.einsum("jd,jdc->jc", x_jobs, Vj)
    coef = mask_jobs
    if delta_jobs is not None:
        coef = (coef - delta_jobs) if coef is not None else (1.0 - delta_jobs)
    if coef is not None:
        h = h * coef.to(h.dtype)
    out = torch.einsum("jc,jco->jo", h, Uj)
    if delta_jobs is not None or route_jobs is not None:
        assert W is not None
        xw = torch.einsum("jd,jod->jo", x_jobs, W[block_of_job].to(x_jobs.dtype))
        if delta_jobs is not None:
            out = out + delta_jobs.to(out.dtype) * xw
        if route_jobs is not None:
            out = torch.where(route_jobs.unsqueeze(-1), out, xw)
    return out
