"""Decomposition sites and the trainable rank-one component stacks.

A site's frozen weight `W [d_out, d_in]` is approximated by `(V U)^T` with `V [d_in, C]` and
`U [C, d_out]`; component `c` is the rank-one matrix `V[:, c] (x) U[c, :]`. Sites that share a shape
(e.g. every layer's `q_proj`) form one *group* and are stored stacked: `V [g, d_in, C]`,
`U [g, C, d_out]`, fp32 masters. Expert banks use a blocked factorization: `n_blocks` independent
`(V_e [d_in, c], U_e [c, d_out])` pairs whose components are laid out block-major on a flat
`C = n_blocks * c` axis, so masks and CI see one flat component axis per site.

Parity: param_decomp/core/components.py:55-63 (`SiteC`), :243-384 (site spec + factorizations),
:531-598 (`ComponentStacks`), :600-636 (stack padding), :650-713 (init `V ~ N(0, 1/d_in)`,
`U ~ N(0, 1/C)`), :65-214 (selected/narrow CI for expert sites).
"""

from __future__ import annotations

import math
from collections import OrderedDict
from dataclasses import dataclass, field

import torch
from torch import Tensor, nn

from param_decomp_b200.formats.nonlinearity import NonlinearityAlignment


@dataclass(frozen=True)
class SiteC:
    name: str
    C: int


@dataclass(frozen=True)
class SiteSpec:
    """One decomposed matrix. `n_blocks > 1` (or `routed`) marks a blocked (per-expert) factorization where
    `d_in`/`d_out` are the dimensions of ONE block and `C` is the flat count `n_blocks * C_block`."""

    name: str
    d_in: int
    d_out: int
    C: int
    group: str = ""
    n_blocks: int = 1
    alignment: NonlinearityAlignment | None = None
    routed: bool = False  # an expert bank's matrix: blocked even when this rank holds a single expert of it

    def __post_init__(self) -> None:
        assert self.C % self.n_blocks == 0, f"{self.name}: C={self.C} must tile n_blocks={self.n_blocks}"
        if not self.group:
            object.__setattr__(self, "group", f"{self.d_in}x{self.d_out}x{self.C}x{self.n_blocks}")

    @property
    def C_block(self) -> int:
        return self.C // self.n_blocks

    @property
    def blocked(self) -> bool:
        return self.n_blocks > 1 or self.routed


@dataclass(frozen=True)
class BlockSelection:
    """Per-position top-k block (expert) choice: `indices [..., k]` into the site's blocks and the
    routing `weights [..., k]` the target applied."""

    indices: Tensor
    weights: Tensor


@dataclass(frozen=True)
class SelectedCI:
    """Narrow CI of a blocked site: values only for the `k` selected blocks of each position.
    `values [..., k * C_block]`, ordered like `selection.indices`."""

    values: Tensor
    selection: BlockSelection
    n_blocks: int

    @property
    def C_block(self) -> int:
        return self.values.shape[-1] // self.selection.indices.shape[-1]

    def scatter_dense(self) -> Tensor:
        """Full-width `[..., n_blocks * C_block]` with zeros at unselected blocks."""
        k, c = self.selection.indices.shape[-1], self.C_block
        lead = self.values.shape[:-1]
        dense = self.values.new_zeros(*lead, self.n_blocks, c)
        idx = self.selection.indices.unsqueeze(-1).expand(*lead, k, c)
        dense.scatter_add_(-2, idx, self.values.reshape(*lead, k, c))
        return dense.reshape(*lead, self.n_blocks * c)

    def sum_per_component(self) -> Tensor:
        """Sum over all leading positions of the dense view, without materialising it: `[C]`."""
        k, c = self.selection.indices.shape[-1], self.C_block
        flat_idx = self.selection.indices.reshape(-1, k)
        vals = self.values.reshape(-1, k, c)
        out = vals.new_zeros(self.n_blocks, c)
        out.index_add_(0, flat_idx.reshape(-1), vals.reshape(-1, c))
        return out.reshape(-1)

    def max_per_component(self) -> Tensor:
        k, c = self.selection.indices.shape[-1], self.C_block
        flat_idx = self.selection.indices.reshape(-1)
        vals = self.values.reshape(-1, c)
        out = vals.new_zeros(self.n_blocks, c)
        out.scatter_reduce_(0, flat_idx[:, None].expand(-1, c), vals, reduce="amax", include_self=True)
        return out.reshape(-1)


def group_sites(sites: tuple[SiteSpec, ...]) -> "OrderedDict[str, list[SiteSpec]]":
    groups: OrderedDict[str, list[SiteSpec]] = OrderedDict()
    for s in sites:
        groups.setdefault(s.group, []).append(s)
    for name, members in groups.items():
        shapes = {(m.d_in, m.d_out, m.C, m.n_blocks) for m in members}
        assert len(shapes) == 1, f"group {name!r} mixes shapes {shapes}"
    return groups


def pad_to_multiple(n: int, multiple: int) -> int:
    return ((n + multiple - 1) // multiple) * multiple


class ComponentStacks(nn.Module):
    """fp32 masters for every site, one `(V, U)` stack per group.

    `stack_multiple` pads each stack's leading axis with inert all-zero matrices so it tiles the mesh
    axes it is sharded over; pads never appear in `site()` views and are stripped from checkpoints.
    """

    def __init__(self, sites: tuple[SiteSpec, ...], stack_multiple: int = 1) -> None:
        super().__init__()
        names = [s.name for s in sites]
        assert len(set(names)) == len(names), f"duplicate site names: {names}"
        self.sites = tuple(sites)
        self.site_by_name = {s.name: s for s in sites}
        self.groups = group_sites(self.sites)
        self.site_stack_indices: dict[str, tuple[str, int]] = {}
        self.stack_pads: dict[str, int] = {}
        self.V = nn.ParameterDict()
        self.U = nn.ParameterDict()
        for gname, members in self.groups.items():
            ref = members[0]
            g = pad_to_multiple(len(members), stack_multiple)
            self.stack_pads[gname] = g - len(members)
            key = self.param_key(gname)
            if ref.blocked:
                v_shape = (g, ref.n_blocks, ref.d_in, ref.C_block)
                u_shape = (g, ref.n_blocks, ref.C_block, ref.d_out)
            else:
                v_shape = (g, ref.d_in, ref.C)
                u_shape = (g, ref.C, ref.d_out)
            self.V[key] = nn.Parameter(torch.zeros(v_shape, dtype=torch.float32))
            self.U[key] = nn.Parameter(torch.zeros(u_shape, dtype=torch.float32))
            for i, s in enumerate(members):
                self.site_stack_indices[s.name] = (gname, i)

    @staticmethod
    def param_key(group: str) -> str:
        return group.replace(".", "_")

    @torch.no_grad()
    def init_random(self, generator: torch.Generator | None = None) -> None:
        """`V ~ N(0, 1/d_in)`, `U ~ N(0, 1/C_block)`; pads stay zero."""
        for gname, members in self.groups.items():
            ref, key = members[0], self.param_key(gname)
            n = len(members)
            V, U = self.V[key], self.U[key]
            v = torch.randn(V[:n].shape, generator=generator, dtype=torch.float32) / math.sqrt(ref.d_in)
            u = torch.randn(U[:n].shape, generator=generator, dtype=torch.float32) / math.sqrt(ref.C_block)
            V[:n].copy_(v.to(V.device))
            U[:n].copy_(u.to(U.device))

    def site(self, name: str) -> tuple[Tensor, Tensor]:
        """Views `(V_s, U_s)`: `[d_in, C]`, `[C, d_out]` (dense) or `[E, d_in, c]`, `[E, c, d_out]`."""
        gname, i = self.site_stack_indices[name]
        key = self.param_key(gname)
        return self.V[key][i], self.U[key][i]

    def set_site(self, name: str, V: Tensor, U: Tensor) -> None:
        v, u = self.site(name)
        with torch.no_grad():
            v.copy_(V)
            u.copy_(U)

    def component_activations(self, name: str, x: Tensor) -> Tensor:
        V, _ = self.site(name)
        assert V.dim() == 2, "component_activations is defined for dense sites"
        return x.to(V.dtype) @ V

    def weight(self, name: str) -> Tensor:
        """`(V U)^T` in the target's `[d_out, d_in]` layout (dense) or `[E, d_out, d_in]` (blocked)."""
        V, U = self.site(name)
        return (V @ U).transpose(-1, -2)

    def n_components(self) -> int:
        return sum(s.C for s in self.sites)


@dataclass
class ComputeWeights:
    """Per-step working copies in the compute dtype (bf16 for LMs): cast once, used by every masked
    forward of the step.

    Eager backend: `V`/`U` are autograd views of the cast masters, gradients flow back through the
    cast. Fused backend (`direct_grads=True`): `V`/`U` carry no autograd history; the site kernels
    accumulate fp32 weight gradients straight into `grad_V`/`grad_U`, which are views of the stacked
    masters' `.grad` buffers."""

    V: dict[str, Tensor] = field(default_factory=dict)
    U: dict[str, Tensor] = field(default_factory=dict)
    grad_V: dict[str, Tensor] = field(default_factory=dict)
    grad_U: dict[str, Tensor] = field(default_factory=dict)
    direct_grads: bool = False

    def site(self, name: str) -> tuple[Tensor, Tensor]:
        return self.V[name], self.U[name]

    def detached(self) -> "ComputeWeights":
        """Same operands, no gradient of any kind (adversary ascents, evaluation)."""
        return ComputeWeights({k: v.detach() for k, v in self.V.items()},
                              {k: v.detach() for k, v in self.U.items()})


def prepare_compute_weights(stacks: ComponentStacks, dtype: torch.dtype, direct_grads: bool = False,
                            working: dict[str, Tensor] | None = None) -> ComputeWeights:
    """`working`: already-cast copies keyed `"V/<group>"` / `"U/<group>"` (the sharded optimizer's
    all-gathered bf16 buffer); when given, no cast happens here."""
    out = ComputeWeights(direct_grads=direct_grads)
    for gname, members in stacks.groups.items():
        key = stacks.param_key(gname)
        pV, pU = stacks.V[key], stacks.U[key]
        if working is not None:
            assert direct_grads, "a pre-cast working copy carries no autograd link to the masters"
            Vc, Uc = working["V/" + key], working["U/" + key]
            assert pV.grad is not None and pU.grad is not None
        elif direct_grads:
            with torch.no_grad():
                Vc, Uc = pV.to(dtype), pU.to(dtype)
            if pV.grad is None:
                pV.grad = torch.zeros_like(pV)
            if pU.grad is None:
                pU.grad = torch.zeros_like(pU)
        else:
            Vc, Uc = pV.to(dtype), pU.to(dtype)  # one cast per stack; site views slice it
        for i, s in enumerate(members):
            out.V[s.name], out.U[s.name] = Vc[i], Uc[i]
            if direct_grads:
                out.grad_V[s.name], out.grad_U[s.name] = pV.grad[i], pU.grad[i]
    return out
