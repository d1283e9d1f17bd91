"""Counter-based randomness for masks, routing and sources.

Every random number the train step draws is a pure function of `(run seed, step, purpose, term,
draw, site, global row, column)`, through the Philox stream shared by the CUDA kernels
(`ops/csrc/common.cuh`) and its torch restatement (`ops/philox_ref.py`). Consequences: the eager and
fused backends see identical masks; a rank draws exactly the rows it owns, so results do not
depend on the device count; the backward pass regenerates masks instead of storing them; and a
resumed run replays the same stream because nothing but `step` advances.

The reference derives per-step keys with `fold_in(run_key, step)` and per-term keys with
`fold_in(key, offset + term_idx)` (param_decomp/core/run.py:1141, core/train.py:438); this module
is the counter-based equivalent (bitwise parity with threefry is not a goal).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import Tensor

from param_decomp_b200.ops import philox_ref

PURPOSE_MASK, PURPOSE_DELTA, PURPOSE_ROUTE_K, PURPOSE_ROUTE_NOISE, PURPOSE_ADV_CHOICE, PURPOSE_SOURCE_INIT, PURPOSE_ROUND, PURPOSE_POOL = range(8)


@dataclass(frozen=True)
class StepKey:
    """`seed64 = run_seed << 32 | step` keys Philox; `stream` separates uses within the step."""

    run_seed: int
    step: int

    @property
    def seed64(self) -> int:
        return ((self.run_seed & 0xFFFFFFFF) << 32) | (self.step & 0xFFFFFFFF)

    @staticmethod
    def stream(purpose: int, term: int = 0, draw: int = 0, site: int = 0) -> int:
        assert 0 <= purpose < 16 and 0 <= term < 16 and 0 <= draw < 16 and 0 <= site < (1 << 20)
        return (purpose << 28) | (term << 24) | (draw << 20) | site


def uniform(key: StepKey, stream: int, rows: int, cols: int, row_offset: int = 0,
            device: torch.device | str = "cpu") -> Tensor:
    """`[rows, cols]` uniforms in (0,1); `cols` is padded up to a multiple of 8 internally."""
    if torch.device(device).type == "cuda":
        from param_decomp_b200.ops import native

        if native.LIB_PATH.exists():  # same stream, one kernel instead of ~150 tiny integer ops
            from param_decomp_b200.ops.elementwise import philox_uniform

            return philox_uniform(key.seed64, stream, rows, cols, row_offset, device)
    padded = ((cols + 7) // 8) * 8
    if torch.device(device).type == "cpu":
        from param_decomp_b200.ops import host_native

        if host_native.available():  # the same stream from one native loop instead of a dozen tensor ops per round
            return host_native.philox_uniform(key.seed64, stream, rows, padded, row_offset)[:, :cols]
    u = philox_ref.uniform(key.seed64, stream, rows, padded, row_offset, device)
    return u[:, :cols]


def uniform_like_rows(key: StepKey, stream: int, lead_shape: tuple[int, ...], cols: int,
                      row_offset: int = 0, device: torch.device | str = "cpu") -> Tensor:
    """Uniforms for a tensor with leading shape `lead_shape` flattened to rows: `[*lead, cols]`."""
    rows = 1
    for n in lead_shape:
        rows *= n
    return uniform(key, stream, rows, cols, row_offset, device).reshape(*lead_shape, cols)
