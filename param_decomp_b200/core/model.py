"""`DecomposedModel`: everything the engine knows about a target.

Parity: param_decomp/core/model.py:185-212 (`ForwardResult`/captures), :306-448 (protocol).
The engine calls: `clean_forward` (no grad; yields the clean output, the site-input taps the CI
function reads, and named captures), `masked_forward` (the decomposed forward under per-site
masks), `recon_loss` (output comparison), `target_weight` (frozen `W` per site, for faithfulness
and the delta path).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Protocol, runtime_checkable

import torch
from torch import Tensor

from param_decomp_b200.core.components import ComputeWeights, SiteSpec
from param_decomp_b200.core.masking import Masks


@dataclass
class ForwardResult:
    output: Any  # logits / toy output, or a factored (hidden, head) pair for streamed edges
    taps: dict[str, Tensor] = field(default_factory=dict)  # CI-fn inputs, keyed by tap name
    captures: dict[str, Tensor] = field(default_factory=dict)  # named internal activations
    aux: dict[str, Any] = field(default_factory=dict)  # target-specific extras (e.g. routing)


@runtime_checkable
class DecomposedModel(Protocol):
    sites: tuple[SiteSpec, ...]
    has_position_axis: bool
    compute_dtype: torch.dtype

    def clean_forward(self, batch: Any, capture: tuple[str, ...] = ()) -> ForwardResult: ...

    def masked_forward(self, weights: ComputeWeights, batch: Any, masks: Masks,
                       capture: tuple[str, ...] = ()) -> ForwardResult: ...

    def recon_loss(self, clean: ForwardResult, masked: ForwardResult) -> Tensor: ...

    def target_weight(self, site: str) -> Tensor: ...

    def tap_for_site(self, site: str) -> str: ...

    def batch_size(self, batch: Any) -> int: ...


def target_weights(model: DecomposedModel) -> dict[str, Tensor]:
    return {s.name: model.target_weight(s.name) for s in model.sites}


def target_weight_sq_norms(model: DecomposedModel) -> dict[str, Tensor]:
    return {s.name: model.target_weight(s.name).float().pow(2).sum() for s in model.sites}


def lead_shape(model: DecomposedModel, clean: ForwardResult, site: str) -> tuple[int, ...]:
    return tuple(clean.taps[model.tap_for_site(site)].shape[:-1])
