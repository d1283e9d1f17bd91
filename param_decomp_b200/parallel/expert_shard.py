"""Engine-side bookkeeping for component stacks that are split over the mesh's tp axis: by expert
(mixture-of-experts targets) or along the component axis `C` (dense targets, `V[:, C/W]`, `U[C/W, :]`).

The MoE targets under expert parallelism (`parallel/ep.py`) keep, per rank, the component blocks of
that rank's experts only: a blocked group's stacks are `V [sites, E_loc, d_in, c]`,
`U [sites, E_loc, c, d_out]` with `E_loc = ceil(E / W)` (the tail of the last rank holds never-routed
dummies that stay zero). Everything else in the run - dense sites, the CI function, the batch - is
replicated over that group. This module is the one place that knows which leaves are split:

  * seeded initialisation that matches the single-process run (draw the global stacks, keep a slice),
  * gradient norms (the split leaves' squares are summed over the group before the clip),
  * gradient reduction (replicated leaves average over the whole job, which also re-synchronises
    them; split leaves average over the batch axes only),
  * checkpoints in the global layout (gather on save, slice on load), so a run can resume on a
    different group size and analysis tools see ordinary stacks.

Parity: param_decomp/core/placement.py:1040-1048,1087-1100 (`expert -> tp` for blocked sites),
param_decomp/routed/experts.py:28-40 (tokens replicated over the shard axis).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor

from param_decomp_b200.core.components import ComponentStacks, SiteSpec


@dataclass
class StackSharding:
    """Which component stacks are split over the tp group, and how (by expert, or along `C`)."""

    group: Any  # the process group of the mesh's tp axis
    n_experts: int  # true expert count E (before padding to a multiple of the group); 0 in component mode
    blocked_keys: frozenset[str]  # parameter keys (`ComponentStacks.param_key`) of the split groups
    by_component: bool = False  # True: dense stacks split along C (`V[..., C/W]`, `U[..., C/W, :]`)

    def __post_init__(self) -> None:
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.e_loc = (self.n_experts + self.world - 1) // self.world
        self.lo = self.rank * self.e_loc
        self.n_real = max(0, min(self.n_experts, self.lo + self.e_loc) - self.lo)  # non-dummy local experts

    @classmethod
    def for_model(cls, model: Any) -> "StackSharding | None":
        ep = getattr(model, "ep", None)
        if ep is not None:
            keys = frozenset(ComponentStacks.param_key(s.group) for s in model.sites if s.blocked)
            return cls(ep.group, ep.n_experts, keys)
        group = getattr(model, "component_group", None)
        if group is not None:
            keys = frozenset(ComponentStacks.param_key(s.group) for s in model.sites)
            return cls(group, 0, keys, by_component=True)
        return None

    def _axis(self, leaf_name: str) -> int:
        """Which axis of a split leaf is divided: the expert axis, or (component mode) `C` - the last axis of
        a `V`-shaped leaf, the one before last of a `U`-shaped leaf."""
        if not self.by_component:
            return 1
        parts = leaf_name.replace(".", "/").split("/")
        return -1 if "V" in parts else -2

    # ---- which leaves are split ----------------------------------------------------------------
    def is_split(self, leaf_name: str) -> bool:
        """`leaf_name`: a `ComponentStacks` parameter name (`V.<key>` / `U.<key>`), an optimizer-state
        name derived from it (`V/<key>/mu`) or a checkpoint name (`components/<group>/V`)."""
        parts = leaf_name.replace(".", "/").split("/")
        return any(ComponentStacks.param_key(p) in self.blocked_keys for p in parts)

    # ---- global <-> local ------------------------------------------------------------------------
    def local_slice(self, t_global: Tensor, leaf_name: str = "") -> Tensor:
        """`[sites, E, ...] -> [sites, E_loc, ...]`: this rank's experts, zero dummies at the tail (component
        mode: this rank's equal slice of the `C` axis)."""
        if self.by_component:
            ax = self._axis(leaf_name)
            width = t_global.shape[ax] // self.world
            return t_global.narrow(ax, self.rank * width, width).contiguous()
        out = t_global.new_zeros(t_global.shape[0], self.e_loc, *t_global.shape[2:])
        if self.n_real:
            out[:, :self.n_real] = t_global[:, self.lo:self.lo + self.n_real]
        return out

    def gather(self, t_local: Tensor, leaf_name: str = "") -> Tensor:
        """`[sites, E_loc, ...]` on every rank of the group `-> [sites, E, ...]` (collective); component
        mode: the slices of the `C` axis side by side."""
        parts = [torch.empty_like(t_local) for _ in range(self.world)]
        dist.all_gather(parts, t_local.contiguous(), group=self.group)
        if self.by_component:
            return torch.cat(parts, dim=self._axis(leaf_name)).contiguous()
        return torch.cat(parts, dim=1)[:, :self.n_experts].contiguous()

    def global_sites(self, sites: tuple[SiteSpec, ...]) -> tuple[SiteSpec, ...]:
        if self.by_component:
            return tuple(SiteSpec(s.name, s.d_in, s.d_out, s.C * self.world, group=s.group, alignment=s.alignment)
                         for s in sites)
        return tuple(s if not s.blocked else SiteSpec(s.name, s.d_in, s.d_out, s.C_block * self.n_experts, group=s.group,
                                                      n_blocks=self.n_experts, alignment=s.alignment, routed=s.routed) for s in sites)

    @torch.no_grad()
    def init_components(self, local: ComponentStacks, generator: torch.Generator) -> None:
        """Draw the global stacks from `generator` exactly as a single process would and keep this
        rank's blocks."""
        full = ComponentStacks(self.global_sites(local.sites))
        full.init_random(generator)
        for gname in local.groups:
            key = local.param_key(gname)
            for leaf, mine, theirs in (("V", local.V[key], full.V[key]), ("U", local.U[key], full.U[key])):
                n = theirs.shape[0]
                if key in self.blocked_keys:
                    mine[:n].copy_(self.local_slice(theirs, leaf))
                else:
                    mine[:n].copy_(theirs)

    # ---- reductions ----------------------------------------------------------------------------------
    def sum_over_group(self, t: Tensor) -> Tensor:
        dist.all_reduce(t, group=self.group)
        return t

    def grad_norm(self, names: list[str], grads: list[Tensor]) -> Tensor:
        """Global L2 norm of a leaf list in which the split leaves contribute their group-wide sum."""
        dev = grads[0].device
        rep = torch.zeros((), device=dev, dtype=torch.float32)
        split = torch.zeros((), device=dev, dtype=torch.float32)
        for n, g in zip(names, grads):
            sq = g.float().pow(2).sum()
            if self.is_split(n):
                split = split + sq
            else:
                rep = rep + sq
        return (rep + self.sum_over_group(split)).sqrt()
