"""Packed token rows as plain numpy arrays (no Arrow import needed to pass rows along).

Parity: param_decomp_formats/packed_rows.py:10-44.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class PackedRows:
    token_ids: np.ndarray  # int32 [rows, seq]
    document_ids: np.ndarray  # int32 [rows, seq], nondecreasing by steps of 0/1 within a row

    def __post_init__(self) -> None:
        t, d = self.token_ids, self.document_ids
        assert t.dtype == np.int32 and d.dtype == np.int32, "token_ids/document_ids must be int32"
        assert t.ndim == 2 and t.shape[1] > 0, "token_ids must be [batch, sequence], nonempty"
        assert d.shape == t.shape, "token_ids and document_ids must have identical shapes"
        assert (t >= 0).all() and (d >= 0).all(), "ids must be nonnegative"
        step = np.diff(d, axis=1)
        assert ((step == 0) | (step == 1)).all(), "document IDs must be contiguous within a row"

    def validate_vocabulary(self, vocab_size: int) -> None:
        assert vocab_size > 0
        assert (self.token_ids < vocab_size).all(), (
            f"token IDs outside [0, {vocab_size}): dataset and target vocabularies differ"
        )

    @classmethod
    def from_unsegmented_sequences(cls, token_ids: np.ndarray) -> "PackedRows":
        return cls(token_ids, np.zeros_like(token_ids))
