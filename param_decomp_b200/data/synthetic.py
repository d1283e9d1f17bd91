"""Seeded synthetic token batches: ids drawn from a Zipf(exponent) law over the vocabulary.

A batch is a pure function of `(seed, step)`, and each rank cuts its own rows out of the global
batch, so data order does not depend on the device count and a resumed run replays the same
stream (the property the reference gets from its `(seed, epoch, step)` batch schedule,
param_decomp/lm/batch_schedule.py:76-118).
"""

from __future__ import annotations

import numpy as np
import torch

from param_decomp_b200.models.transformer import LMBatch


class ZipfTokenSource:
    def __init__(self, vocab_size: int, seq_len: int, exponent: float = 1.1, seed: int = 0) -> None:
        ranks = np.arange(1, vocab_size + 1, dtype=np.float64)
        p = ranks ** (-exponent)
        self.cdf = np.cumsum(p / p.sum())
        self.cdf[-1] = 1.0
        self.vocab_size, self.seq_len, self.seed = vocab_size, seq_len, seed
        # a fixed permutation so frequent ids are not the smallest ids
        self.perm = np.random.default_rng(seed ^ 0xA5A5).permutation(vocab_size).astype(np.int32)

    def rows(self, step: int, first_row: int, n_rows: int, global_rows: int) -> np.ndarray:
        """Rows `[first_row, first_row + n_rows)` of the global batch of `step`: `[n_rows, seq_len]` int32."""
        rng = np.random.default_rng([self.seed, step])
        u = rng.random((global_rows, self.seq_len))[first_row:first_row + n_rows]
        idx = np.searchsorted(self.cdf, u, side="left").astype(np.int32)
        return self.perm[np.minimum(idx, self.vocab_size - 1)]

    def batch(self, step: int, global_rows: int, rank: int = 0, world: int = 1, pin: bool = False) -> LMBatch:
        per = global_rows // world
        t = torch.from_numpy(self.rows(step, rank * per, per, global_rows))
        if pin and torch.cuda.is_available():
            t = t.pin_memory()
        return LMBatch(tokens=t)
