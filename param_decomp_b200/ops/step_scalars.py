"""Per-step scalars kept in device memory.

A decomposition step depends on a handful of host-computed numbers that change every step: the
Philox seed word, scheduled coefficients (`gamma`, loss coefficients, learning rates), Adam's bias
corrections, the sequence numbers of the peer barriers. Passed by value they are baked into each
kernel launch, which rules out recording the step once and replaying it (CUDA graphs). Here every
such number has a slot in one small device table; kernels and torch ops read the slot, and the host
refreshes the whole table with ONE pinned-memory copy per step before the step's launches (or its
recorded graph) are issued.

Each entry is registered once, with the function that computes it from the step index; later steps
only re-evaluate the functions. The pinned staging buffers form a ring guarded by events, so the
host can run a few steps ahead of the device without overwriting a buffer whose copy has not
executed yet.

The reference obtains the same effect by passing schedule values as array leaves of its jitted
step (param_decomp/core/runtime_schedule.py:12-90).
"""

from __future__ import annotations

import struct
from dataclasses import dataclass
from typing import Callable

import torch
from torch import Tensor

_RING = 4


@dataclass
class _Entry:
    name: str
    slot: int
    kind: str  # "f32" | "u32" | "u64"
    width: int  # number of 32-bit words
    fn: Callable[[int], object]


class StepScalars:
    def __init__(self, device: torch.device | str, capacity: int = 512) -> None:
        self.device = torch.device(device)
        self.capacity = capacity
        self.words = torch.zeros(capacity, dtype=torch.int32, device=self.device)
        cuda = self.device.type == "cuda"
        self._host = [torch.zeros(capacity, dtype=torch.int32, pin_memory=cuda) for _ in range(_RING if cuda else 1)]
        self._events = [torch.cuda.Event() if cuda else None for _ in self._host]
        self._busy = [False] * len(self._host)
        self._turn = 0
        self._entries: dict[str, _Entry] = {}
        self._used = 0
        self.step: int | None = None
        self.frozen = False  # set once a recording refers to the table: no new entries after that

    # -- registration --------------------------------------------------------------------------
    def _register(self, name: str, kind: str, width: int, fn: Callable[[int], object], align: int = 1) -> _Entry:
        e = self._entries.get(name)
        if e is not None:
            assert e.kind == kind and e.width == width, f"scalar {name!r} re-registered with another shape"
            e.fn = fn  # closures may capture fresh objects; the slot stays
            return e
        assert not self.frozen, f"scalar {name!r} first requested after the step was recorded"
        slot = (self._used + align - 1) // align * align
        assert slot + width <= self.capacity, "step-scalar table is full"
        self._used = slot + width
        e = _Entry(name, slot, kind, width, fn)
        self._entries[name] = e
        if self.step is not None:  # registered in the middle of a step: make this step's value visible now
            buf = torch.zeros(width, dtype=torch.int32)
            self._encode(e, self.step, buf, 0)
            self.words[slot:slot + width].copy_(buf)
        return e

    def f32(self, name: str, fn: Callable[[int], float]) -> Tensor:
        """0-d fp32 device tensor holding `fn(step)`."""
        e = self._register(name, "f32", 1, fn)
        return self.words[e.slot:e.slot + 1].view(torch.float32).reshape(())

    def f32_block(self, name: str, n: int, fn: Callable[[int], tuple]) -> Tensor:
        """`[n]` fp32 device tensor holding the tuple `fn(step)` (16-byte aligned)."""
        e = self._register(name, "f32", n, fn, align=4)
        return self.words[e.slot:e.slot + n].view(torch.float32)

    def u32(self, name: str, fn: Callable[[int], int]) -> Tensor:
        e = self._register(name, "u32", 1, fn)
        return self.words[e.slot:e.slot + 1]

    def u64(self, name: str, fn: Callable[[int], int]) -> Tensor:
        """1-element int64 device tensor holding the 64-bit pattern `fn(step)`."""
        e = self._register(name, "u64", 2, fn, align=2)
        return self.words[e.slot:e.slot + 2].view(torch.int64)

    def host_value(self, name: str, step: int):
        return self._entries[name].fn(step)

    # -- per step --------------------------------------------------------------------------------
    @staticmethod
    def _encode(e: _Entry, step: int, buf: Tensor, at: int) -> None:
        v = e.fn(step)
        if e.kind == "f32":
            vals = v if isinstance(v, (tuple, list)) else (v,)
            assert len(vals) == e.width
            raw = struct.unpack(f"<{e.width}i", struct.pack(f"<{e.width}f", *[float(x) for x in vals]))
        elif e.kind == "u32":
            raw = struct.unpack("<i", struct.pack("<I", int(v) & 0xFFFFFFFF))
        else:
            raw = struct.unpack("<2i", struct.pack("<Q", int(v) & 0xFFFFFFFFFFFFFFFF))
        for i, w in enumerate(raw):
            buf[at + i] = w

    def begin(self, step: int) -> None:
        """Evaluate every entry at `step` and queue the table's refresh on the current stream."""
        self.step = step
        if not self._entries:
            return
        i = self._turn
        self._turn = (self._turn + 1) % len(self._host)
        if self._busy[i] and self._events[i] is not None:
            self._events[i].synchronize()  # the copy that last read this staging buffer has run
        host = self._host[i]
        for e in self._entries.values():
            self._encode(e, step, host, e.slot)
        self.words[:self._used].copy_(host[:self._used], non_blocking=True)
        if self._events[i] is not None:
            self._events[i].record()
            self._busy[i] = True


def ptr_or_zero(t: Tensor | None) -> int:
    return 0 if t is None else t.data_ptr()
