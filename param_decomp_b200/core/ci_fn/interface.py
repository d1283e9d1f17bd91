"""The CI-function contract.

A CI function reads *taps* (clean activations of the target, keyed by name) and emits one
pre-activation tensor `[..., C_site]` per decomposed site. `squash` turns pre-activations into the
two importances the objective uses: `lower` (masks) and `upper` (minimality penalty).

Parity: param_decomp/core/ci_fn/interface.py:24-110 (CI triple, CIFn protocol, TapSpec),
architecture.py:14-43 (parameter census / useful FLOPs hooks), runtime.py:10-27.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Protocol

from torch import Tensor, nn

from param_decomp_b200.core.components import SelectedCI
from param_decomp_b200.core.squashing import lower_leaky_hard_sigmoid, upper_leaky_hard_sigmoid


@dataclass(frozen=True)
class TapSpec:
    key: str
    width: int


class MaskInputs(dict):
    """`{site: importances}` as the mask samplers consume them, plus - for expert-blocked sites, whose values are
    NARROW - which blocks each position's slots are: `selections[site] = (indices [..., k], n_blocks)`. Samplers
    that combine the importances with full-width quantities (adversary sources) gather those at the same blocks."""

    selections: dict[str, tuple[Tensor, int]]

    def __init__(self, values: dict[str, Tensor], selections: dict[str, tuple[Tensor, int]] | None = None) -> None:
        super().__init__(values)
        self.selections = dict(selections or {})

    def map(self, fn) -> "MaskInputs":
        return MaskInputs({k: fn(v) for k, v in self.items()}, self.selections)


@dataclass
class CI:
    preactivations: dict[str, Tensor | SelectedCI]
    lower: dict[str, Tensor | SelectedCI]
    upper: dict[str, Tensor | SelectedCI]
    activity: dict[str, Tensor] | None = None
    """Fused backend only: per-component mean smooth-L0 activity `[C]`, produced in the same pass
    as `lower` (then `upper` is not materialised)."""

    def mask_inputs(self) -> MaskInputs:
        """What the mask samplers consume: dense `[..., C]` for dense sites, the NARROW
        `[..., k * C_block]` values (slot-major, in routing order) for expert-blocked sites."""
        return MaskInputs({k: (v.values if isinstance(v, SelectedCI) else v) for k, v in self.lower.items()},
                          {k: (v.selection.indices, v.n_blocks) for k, v in self.lower.items()
                           if isinstance(v, SelectedCI)})

    def dense_lower(self) -> dict[str, Tensor]:
        return {k: (v.scatter_dense() if isinstance(v, SelectedCI) else v) for k, v in self.lower.items()}

    def dense_upper(self) -> dict[str, Tensor]:
        return {k: (v.scatter_dense() if isinstance(v, SelectedCI) else v) for k, v in self.upper.items()}


def _map(fn, v):
    if isinstance(v, SelectedCI):
        return SelectedCI(fn(v.values), v.selection, v.n_blocks)
    return fn(v)


def squash_fused(pre: dict[str, Tensor | SelectedCI], gamma: float, normalize_at_one: bool) -> CI:
    """One kernel pass per site: lower importances and the minimality activity together."""
    from param_decomp_b200.ops.elementwise import squash_activity, squash_activity_selected

    lower, act = {}, {}
    for k, v in pre.items():
        if isinstance(v, SelectedCI):
            low, act[k] = squash_activity_selected(v.values, v.selection.indices, v.n_blocks, gamma, normalize_at_one)
            lower[k] = SelectedCI(low, v.selection, v.n_blocks)
        else:
            lower[k], act[k] = squash_activity(v, gamma, normalize_at_one)
    return CI(preactivations=pre, lower=lower, upper={}, activity=act)


def squash(pre: dict[str, Tensor | SelectedCI]) -> CI:
    return CI(
        preactivations=pre,
        lower={k: _map(lower_leaky_hard_sigmoid, v) for k, v in pre.items()},
        upper={k: _map(upper_leaky_hard_sigmoid, v) for k, v in pre.items()},
    )


class CIFn(Protocol):
    """`nn.Module`s implementing `forward(taps, **context) -> {site: preactivations}`."""

    input_taps: tuple[str, ...]

    def forward(self, taps: dict[str, Tensor], **context: Any) -> dict[str, Tensor | SelectedCI]: ...

    def parameter_census(self) -> dict[str, int]: ...

    def useful_flops_per_position(self) -> int: ...


def census(module: nn.Module) -> dict[str, int]:
    out: dict[str, int] = {"total": 0, "matrix": 0, "other": 0}
    for p in module.parameters():
        out["total"] += p.numel()
        out["matrix" if p.dim() >= 2 else "other"] += p.numel()
    return out
