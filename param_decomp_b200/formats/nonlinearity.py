"""Vocabulary for which side of a matrix faces a nonlinearity and how that side splits into units.

Parity: param_decomp_formats/nonlinearity.py:6-87. Consumed by nonlinearity-aligned init and by
the nonlinearity-locality loss.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar, Literal

NonlinearityUnitKind = Literal["neuron", "attention_head", "deltanet_head"]
ComponentSide = Literal["input", "output"]


@dataclass(frozen=True)
class Neurons:
    unit_kind: ClassVar[NonlinearityUnitKind] = "neuron"
    use_multiplicity: ClassVar[int] = 1


def _positive(**named: int) -> None:
    for key, val in named.items():
        if val < 1:
            raise AssertionError(f"{key} must be positive: {val}")


@dataclass(frozen=True)
class QueryHeads:
    head_count: int
    unit_kind: ClassVar[NonlinearityUnitKind] = "attention_head"
    use_multiplicity: ClassVar[int] = 1

    def __post_init__(self) -> None:
        _positive(head_count=self.head_count)


@dataclass(frozen=True)
class KVHeads:
    """K/V blocks are written once but read by `n_head / n_kv_head` query heads."""

    head_count: int
    use_multiplicity: int
    unit_kind: ClassVar[NonlinearityUnitKind] = "attention_head"

    def __post_init__(self) -> None:
        _positive(head_count=self.head_count, use_multiplicity=self.use_multiplicity)


@dataclass(frozen=True)
class DeltaNetHeads:
    head_count: int
    use_multiplicity: int
    unit_kind: ClassVar[NonlinearityUnitKind] = "deltanet_head"

    def __post_init__(self) -> None:
        _positive(head_count=self.head_count, use_multiplicity=self.use_multiplicity)


NonlinearityPartition = Neurons | QueryHeads | KVHeads | DeltaNetHeads


@dataclass(frozen=True)
class NonlinearityAlignment:
    side: ComponentSide
    partition: NonlinearityPartition

    def unit_count(self, aligned_width: int) -> int:
        if isinstance(self.partition, Neurons):
            return aligned_width
        return self.partition.head_count
