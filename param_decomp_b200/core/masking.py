"""Per-site masks for masked forwards, and the samplers that build them.

A masked forward evaluates, at each decomposed site,
    out = ((x V) * (m - d)) U + d * (x W^T),      then   where(route, out, x W^T)
with `m [..., C]` the component mask, `d [..., 1]` the delta mask (weight on the residual
`W - (VU)^T`), `route [...]` which positions use the decomposition at all.

Mask sources (parity: param_decomp/core/masking.py:135-396, core/source_mask.py:13-70,
core/recon.py:46-264):
  stochastic        m = ci + (1 - ci) u,  d = u'          u, u' ~ U(0,1)
  ci-masked         m = ci,               d = 0
  unmasked          m = 1,                d = 1           (reproduces the target exactly)
  unmasked-no-delta m = 1,                d = 0           (the full component sum)
  source            m = ci + (1 - ci) s,  d = s_delta     s from a persistent or fresh adversary
  merged            per batch row: source masks with prob adv_fraction, else stochastic + routing
Routing: uniform-k-subset (k ~ U{1..S} per position, the k sites with smallest noise are routed),
static probability, or all.

Stochastic masks can stay *lazy* (`StochasticSpec`): the fused sm_100a site kernel then draws `u`
in its epilogue from the same Philox counters `materialize()` uses, so `m` never exists in memory.
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import torch
from torch import Tensor

from param_decomp_b200.core import rng
from param_decomp_b200.core.rng import StepKey


@dataclass(frozen=True)
class StochasticSpec:
    """Lazy `m = ci + (1 - ci) * u`, `u = philox(seed64, stream)[row_offset + row, col]`."""

    seed64: int
    stream: int
    row_offset: int = 0
    col_offset: int = 0  # global index of `ci`'s first column when `ci` is a column slice of the site (multiple of 8)


@dataclass(frozen=True)
class SiteMask:
    ci: Tensor | None = None  # [..., C] lower-leaky CI when `stochastic` is set
    mask: Tensor | None = None  # [..., C] materialised m; None with stochastic=None means all ones
    delta: Tensor | None = None  # [..., 1]; None = no delta path (d = 0)
    route: Tensor | None = None  # bool [...]; None = every position routed
    stochastic: StochasticSpec | None = None

    def materialize(self) -> "SiteMask":
        """Replace a lazy stochastic spec by the explicit mask tensor (eager backend, tests)."""
        if self.stochastic is None:
            return self
        assert self.ci is not None
        lead, C = self.ci.shape[:-1], self.ci.shape[-1]
        key = StepKey(self.stochastic.seed64 >> 32, self.stochastic.seed64 & 0xFFFFFFFF)
        c0 = self.stochastic.col_offset
        u = rng.uniform_like_rows(key, self.stochastic.stream, tuple(lead), c0 + C,
                                  self.stochastic.row_offset, self.ci.device)[..., c0:].to(self.ci.dtype)
        return replace(self, mask=self.ci + (1 - self.ci) * u, stochastic=None)

    def column_shard(self, group) -> "SiteMask":
        """This rank's equal column slice of a mask that is replicated over `group` (components split
        over tensor-parallel ranks): `ci` / `mask` are sliced with a gradient that re-assembles the full
        tensor on every rank, a lazy draw keeps its place in the counter space, `delta` / `route` are
        per-position and stay whole."""
        import torch.distributed as dist

        from param_decomp_b200.parallel.group_ops import slice_columns

        cut = lambda t: None if t is None else slice_columns(t, group)  # noqa: E731
        st = self.stochastic
        if st is not None:
            assert self.ci is not None
            width = self.ci.shape[-1] // dist.get_world_size(group)
            st = replace(st, col_offset=st.col_offset + dist.get_rank(group) * width)
        return replace(self, ci=cut(self.ci), mask=cut(self.mask), stochastic=st)


Masks = dict[str, SiteMask]


def _lead(ci: Tensor) -> tuple[int, ...]:
    return tuple(ci.shape[:-1])


def ci_masks(ci: dict[str, Tensor]) -> Masks:
    return {name: SiteMask(mask=c) for name, c in ci.items()}


def unmasked(ci: dict[str, Tensor]) -> Masks:
    return {name: SiteMask(mask=None, delta=torch.ones(*_lead(c), 1, device=c.device, dtype=c.dtype))
            for name, c in ci.items()}


def unmasked_no_delta(ci: dict[str, Tensor]) -> Masks:
    return {name: SiteMask() for name in ci}


def constant_masks(ci: dict[str, Tensor], value: float, delta: float | None) -> Masks:
    out = {}
    for name, c in ci.items():
        d = None if delta is None else torch.full((*_lead(c), 1), delta, device=c.device, dtype=c.dtype)
        out[name] = SiteMask(mask=torch.full_like(c, value), delta=d)
    return out


def sample_routing(kind: str, p: float | None, site_names: list[str], lead: tuple[int, ...],
                   key: StepKey, term: int, draw: int, row_offset: int,
                   device: torch.device | str) -> dict[str, Tensor | None]:
    """Per-site boolean route tensors of shape `lead` (None = all routed)."""
    if kind == "all":
        return {n: None for n in site_names}
    S = len(site_names)
    noise = torch.stack([
        rng.uniform_like_rows(key, StepKey.stream(rng.PURPOSE_ROUTE_NOISE, term, draw, i), lead, 1,
                              row_offset, device)[..., 0]
        for i in range(S)
    ])  # [S, *lead]
    if kind == "static_probability":
        assert p is not None
        return {n: noise[i] < p for i, n in enumerate(site_names)}
    assert kind == "uniform_k_subset", kind
    uk = rng.uniform_like_rows(key, StepKey.stream(rng.PURPOSE_ROUTE_K, term, draw), lead, 1,
                               row_offset, device)[..., 0]
    k = torch.clamp((uk * S).floor().long() + 1, max=S)  # uniform on {1..S}
    ranks = noise.argsort(dim=0).argsort(dim=0)  # rank of each site's noise at every position
    return {n: ranks[i] < k for i, n in enumerate(site_names)}


def stochastic_masks(ci: dict[str, Tensor], key: StepKey, term: int, draw: int, *,
                     site_index: dict[str, int], row_offset: int = 0, with_delta: bool = True,
                     delta_pinned: float | None = None, routing: dict[str, Tensor | None] | None = None,
                     lazy: bool = True) -> Masks:
    """One stochastic draw for every site. `delta_pinned=1.0` is the non-target pass's spelling."""
    out: Masks = {}
    for name, c in ci.items():
        lead = _lead(c)
        si = site_index[name]
        spec = StochasticSpec(key.seed64, StepKey.stream(rng.PURPOSE_MASK, term, draw, si), row_offset)
        if delta_pinned is not None:
            d = torch.full((*lead, 1), delta_pinned, device=c.device, dtype=c.dtype)
        elif with_delta:
            d = rng.uniform_like_rows(key, StepKey.stream(rng.PURPOSE_DELTA, term, draw, si), lead, 1,
                                      row_offset, c.device).to(c.dtype)
        else:
            d = None
        sm = SiteMask(ci=c, delta=d, route=None if routing is None else routing[name], stochastic=spec)
        out[name] = sm if lazy else sm.materialize()
    return out


def select_source_blocks(source: Tensor, indices: Tensor, n_blocks: int) -> Tensor:
    """A full-width source `[*src_lead, n_blocks * c]` (leading axes of size 1 are shared) read at each position's
    selected blocks: `[*lead, k * c]`, slot-major like the narrow importances. Indexing, not expansion: nothing of
    size `positions x n_blocks x c` is formed, and the gradient accumulates into the selected blocks only
    (param_decomp/core/masking.py:43-120, selected source values)."""
    lead, k = tuple(indices.shape[:-1]), indices.shape[-1]
    c = source.shape[-1] // n_blocks
    assert c * n_blocks == source.shape[-1], (source.shape, n_blocks)
    src_lead = (1,) * (len(lead) - (source.dim() - 1)) + tuple(source.shape[:-1])
    assert len(src_lead) == len(lead), f"source {tuple(source.shape)} has more leading axes than the importances {lead}"
    table = source.reshape(*src_lead, n_blocks, c)
    index: list[Tensor] = []
    for axis, (have, want) in enumerate(zip(src_lead, lead)):
        assert have in (1, want), f"source axis {axis} is {have}, the importances have {want}"
        ix = torch.arange(want, device=source.device) if have == want and want > 1 else torch.zeros(1, dtype=torch.long, device=source.device)
        shape = [1] * (len(lead) + 1)
        shape[axis] = ix.numel()
        index.append(ix.view(shape))
    picked = table[(*index, indices.long())]  # [*lead, k, c]
    return picked.reshape(*lead, k * c)


def source_masks(ci: dict[str, Tensor], sources: dict[str, Tensor], delta_sources: dict[str, Tensor] | None,
                 routing: dict[str, Tensor | None] | None = None) -> Masks:
    """`m = ci + (1 - ci) s` with broadcastable sources (`[1,C]`, `[B,C]`, `[B,1,C]`, `[B,T,C]`). Where `ci` carries
    block selections (`MaskInputs.selections`: narrow importances of expert-blocked sites) the full-width source
    is read at the selected blocks."""
    out: Masks = {}
    selections = getattr(ci, "selections", {})
    for name, c in ci.items():
        s = sources[name].to(c.dtype)
        if name in selections:
            s = select_source_blocks(s, *selections[name])
        d = None
        if delta_sources is not None:
            d = delta_sources[name].to(c.dtype).expand(*_lead(c), 1)
        out[name] = SiteMask(mask=c + (1 - c) * s, delta=d, route=None if routing is None else routing[name])
    return out


def merged_masks(ci: dict[str, Tensor], sources: dict[str, Tensor], delta_sources: dict[str, Tensor],
                 adv_fraction: float, key: StepKey, term: int, draw: int, *, site_index: dict[str, int],
                 routing_kind: str, routing_p: float | None, row_offset: int = 0) -> Masks:
    """Per batch row: persistent sources at every site with prob `adv_fraction`, else a fresh
    stochastic draw with subset routing. The choice is shared along the row's sequence."""
    names = list(ci)
    first = ci[names[0]]
    lead = _lead(first)
    B = lead[0]
    pick = rng.uniform(key, StepKey.stream(rng.PURPOSE_ADV_CHOICE, term, draw), B, 1, row_offset_rows(row_offset, lead),
                       first.device)[:, 0] < adv_fraction
    pick_lead = pick.reshape(B, *([1] * (len(lead) - 1))).expand(*lead)
    routes = sample_routing(routing_kind, routing_p, names, lead, key, term, draw, row_offset, first.device)
    stoch = stochastic_masks(ci, key, term, draw, site_index=site_index, row_offset=row_offset, lazy=False)
    adv = source_masks(ci, sources, delta_sources)
    out: Masks = {}
    for name in names:
        sel = pick_lead.unsqueeze(-1)
        m = torch.where(sel, adv[name].mask, stoch[name].mask)
        d = torch.where(sel, adv[name].delta, stoch[name].delta)
        r = routes[name]
        route = None if r is None else (r | pick_lead)  # adversarial rows route every site
        out[name] = SiteMask(mask=m, delta=d, route=route)
    return out


def row_offset_rows(row_offset: int, lead: tuple[int, ...]) -> int:
    """Convert a flattened-position offset into a batch-row offset."""
    per_row = 1
    for n in lead[1:]:
        per_row *= n
    return row_offset // per_row
