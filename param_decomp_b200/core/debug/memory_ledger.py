"""Memory ledger: what is alive on the device at named points of a step, and which tensors.

The reference reads XLA's buffer assignment (every buffer with size, offset, live range and source
line: param_decomp/core/tools/memory_ledger.py, ledger_diff.py, memreport.py). With an eager engine
the same questions are answered at run time: `Ledger.mark(name)` records allocator counters and
the largest live tensors (with the Python frame that allocated them when the allocator history is
on), `diff` compares two ledgers mark by mark, `report` prints the peak.
"""

from __future__ import annotations

import gc
import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

import torch


@dataclass
class Mark:
    name: str
    allocated: int
    reserved: int
    peak_allocated: int
    top_tensors: list[tuple[str, int]]  # (shape/dtype description, bytes)


@dataclass
class Ledger:
    device: Any = None
    top_n: int = 12
    marks: list[Mark] = field(default_factory=list)

    def _stats(self) -> tuple[int, int, int]:
        if torch.cuda.is_available():
            return (torch.cuda.memory_allocated(self.device), torch.cuda.memory_reserved(self.device),
                    torch.cuda.max_memory_allocated(self.device))
        return 0, 0, 0

    def _live_tensors(self, with_total: bool = False):
        seen: dict[int, tuple[str, int]] = {}
        for obj in gc.get_objects():
            try:
                if isinstance(obj, torch.Tensor) and (obj.is_cuda or not torch.cuda.is_available()):
                    st = obj.untyped_storage()
                    key = st.data_ptr()
                    if key and key not in seen:
                        seen[key] = (f"{tuple(obj.shape)} {str(obj.dtype).replace('torch.', '')}", st.nbytes())
            except Exception:  # noqa: BLE001  (objects mid-destruction)
                continue
        top = sorted(seen.values(), key=lambda kv: -kv[1])[: self.top_n]
        return (top, sum(b for _, b in seen.values())) if with_total else top

    def mark(self, name: str) -> Mark:
        a, r, p = self._stats()
        top, total = self._live_tensors(with_total=True)
        if not torch.cuda.is_available():  # no allocator counters on the host: the live tensors' storages stand in
            a = r = total
            p = max([total] + [m.peak_allocated for m in self.marks])
        m = Mark(name, a, r, p, top)
        self.marks.append(m)
        return m

    def reset_peak(self) -> None:
        if torch.cuda.is_available():
            torch.cuda.reset_peak_memory_stats(self.device)

    def save(self, path: Path | str) -> None:
        Path(path).write_text(json.dumps([asdict(m) for m in self.marks], indent=1))

    @classmethod
    def load(cls, path: Path | str) -> "Ledger":
        led = cls()
        led.marks = [Mark(**{**m, "top_tensors": [tuple(t) for t in m["top_tensors"]]})
                     for m in json.loads(Path(path).read_text())]
        return led

    def report(self) -> str:
        if not self.marks:
            return "empty ledger"
        peak = max(self.marks, key=lambda m: m.peak_allocated)
        lines = [f"peak {peak.peak_allocated / 2**30:.2f} GiB by mark '{peak.name}'"]
        for m in self.marks:
            lines.append(f"  {m.name:32s} allocated {m.allocated / 2**30:8.2f} GiB  reserved {m.reserved / 2**30:8.2f} GiB")
        lines.append("largest live tensors at the peak mark:")
        lines += [f"  {b / 2**20:10.1f} MiB  {d}" for d, b in peak.top_tensors]
        return "\n".join(lines)


def main() -> None:
    """`python -m param_decomp_b200.core.debug.memory_ledger <run_dir | ledger.json> [--top N]`: the peak, every mark,
    and the largest live tensors at the peak mark. A run started with `runtime.profiling: {kind: ad_hoc, ...}` leaves
    its ledger at `<run_dir>/profile/memory_ledger.json` (one mark per phase of the first profiled step)."""
    import argparse

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("path", type=Path)
    ap.add_argument("--top", type=int, default=12)
    a = ap.parse_args()
    path = a.path / "profile" / "memory_ledger.json" if a.path.is_dir() else a.path
    assert path.exists(), f"no ledger at {path}"
    led = Ledger.load(path)
    for m in led.marks:
        m.top_tensors = m.top_tensors[: a.top]
    print(led.report())


def diff(a: Ledger, b: Ledger) -> list[tuple[str, int]]:
    """Per shared mark: bytes allocated in `b` minus `a` (what a change cost, where)."""
    bm = {m.name: m for m in b.marks}
    return [(m.name, bm[m.name].allocated - m.allocated) for m in a.marks if m.name in bm]


if __name__ == "__main__":
    main()
