"""Fork / join of independent pieces of a step onto CUDA side streams.

With a small per-rank batch many products of the step have fewer tiles than the GPU has SMs (a
`[4096, 768]` output is 48 two-CTA tiles on 74 CTA-pair slots), so a kernel that runs alone leaves
a third of the machine idle. The q / k / v sites of a block read the same input and do not depend
on each other, nor do gate / up, nor the mask draws of a reconstruction term: run side by side they
fill the idle SMs. `Lanes.run([f0, f1, ...])` runs `f0` on the current stream and every other
function on a side stream that first waits for everything queued on the current stream so far; the
current stream then waits for all of them. Autograd replays each backward node on the stream its
forward ran on, so the backward pass forks the same way. Inside a recorded step (CUDA graph) the
forks become parallel branches of the graph and cost no host time.

Memory: a tensor produced on a side stream is consumed on the current stream only after the join,
and every new use of a side stream begins by waiting for the current stream, so a block the caching
allocator hands back to a side stream is never re-used before its last reader has been ordered
ahead of the new writer.
"""

from __future__ import annotations

from typing import Any, Callable

import torch


class Lanes:
    def __init__(self) -> None:
        self._streams: dict[tuple[int, int], torch.cuda.Stream] = {}
        self._dirty: dict[int, torch.cuda.Stream] = {}  # side streams used since the last `join_all`

    def _side(self, parent: torch.cuda.Stream, index: int) -> torch.cuda.Stream:
        key = (parent.cuda_stream, index)
        s = self._streams.get(key)
        if s is None:
            s = torch.cuda.Stream(device=parent.device)
            self._streams[key] = s
        self._dirty[s.cuda_stream] = s
        return s

    def run(self, fns: list[Callable[[], Any]]) -> list[Any]:
        """Results of `fns`, evaluated concurrently on the device (sequentially on the host)."""
        if len(fns) == 1:
            return [fns[0]()]
        cur = torch.cuda.current_stream()
        fork = cur.record_event()
        outs: list[Any] = [None] * len(fns)
        used = []
        for i in range(1, len(fns)):
            s = self._side(cur, i)
            s.wait_event(fork)
            with torch.cuda.stream(s):
                outs[i] = fns[i]()
            used.append(s)
        outs[0] = fns[0]()
        for s in used:
            cur.wait_event(s.record_event())
        return outs

    def join_all(self) -> None:
        """The current stream waits for every side stream used since the last call (kernels that write without going
        through autograd - direct weight-gradient accumulation - are ordered before the optimizer)."""
        cur = torch.cuda.current_stream()
        for s in self._dirty.values():
            if s.cuda_stream != cur.cuda_stream:
                cur.wait_event(s.record_event())
        self._dirty = {}
