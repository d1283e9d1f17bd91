"""Diff two saved memory ledgers: "what did my change do to memory".

    python -m param_decomp_b200.core.debug.ledger_diff <a.json> <b.json> [--mark NAME] [--top N] [--peak-only]

Per mark both runs share: the change in allocated / reserved / peak bytes, and the live-tensor groups (one group
per shape and dtype among the mark's recorded largest tensors) that were created, destroyed or resized between A
and B. `--peak-only` looks only at each side's own peak mark (what moved the high-water mark); the default walks
every shared mark. Tensor identities do not survive a run, so groups - not tensors - are compared.
Parity: param_decomp/core/tools/ledger_diff.py (the same question asked of XLA's buffer assignment).
"""

from __future__ import annotations

import argparse
from dataclasses import dataclass
from pathlib import Path

from param_decomp_b200.core.debug.memory_ledger import Ledger, Mark

GIB = float(2**30)


@dataclass(frozen=True)
class GroupStat:
    n_tensors: int
    total_bytes: int


@dataclass(frozen=True)
class GroupDelta:
    key: str
    a: GroupStat | None
    b: GroupStat | None

    @property
    def delta_bytes(self) -> int:
        return (self.b.total_bytes if self.b else 0) - (self.a.total_bytes if self.a else 0)


@dataclass(frozen=True)
class MarkDiff:
    mark: str
    allocated: tuple[int, int]
    reserved: tuple[int, int]
    peak: tuple[int, int]
    created: tuple[GroupDelta, ...]
    destroyed: tuple[GroupDelta, ...]
    resized: tuple[GroupDelta, ...]


def tensor_groups(mark: Mark) -> dict[str, GroupStat]:
    groups: dict[str, GroupStat] = {}
    for desc, nbytes in mark.top_tensors:
        g = groups.get(desc, GroupStat(0, 0))
        groups[desc] = GroupStat(g.n_tensors + 1, g.total_bytes + int(nbytes))
    return groups


def diff_marks(a: Mark, b: Mark, name: str | None = None) -> MarkDiff:
    ga, gb = tensor_groups(a), tensor_groups(b)
    created = tuple(GroupDelta(k, None, gb[k]) for k in gb if k not in ga)
    destroyed = tuple(GroupDelta(k, ga[k], None) for k in ga if k not in gb)
    resized = tuple(GroupDelta(k, ga[k], gb[k]) for k in ga if k in gb and ga[k] != gb[k])
    by_size = lambda ds: tuple(sorted(ds, key=lambda d: -abs(d.delta_bytes)))  # noqa: E731
    return MarkDiff(name or a.name, (a.allocated, b.allocated), (a.reserved, b.reserved),
                    (a.peak_allocated, b.peak_allocated), by_size(created), by_size(destroyed), by_size(resized))


def diff_ledgers(a: Ledger, b: Ledger, mark: str | None = None, peak_only: bool = False) -> list[MarkDiff]:
    if peak_only:
        pa, pb = (max(led.marks, key=lambda m: m.peak_allocated) for led in (a, b))
        return [diff_marks(pa, pb, f"peak ({pa.name} -> {pb.name})")]
    bm = {m.name: m for m in b.marks}
    shared = [m for m in a.marks if m.name in bm and (mark is None or m.name == mark)]
    assert shared, f"the ledgers share no mark{'' if mark is None else ' named ' + repr(mark)}"
    return [diff_marks(m, bm[m.name]) for m in shared]


def render(diffs: list[MarkDiff], top: int = 10) -> str:
    lines: list[str] = []
    for d in diffs:
        lines.append(f"{d.mark}: allocated {d.allocated[0] / GIB:.3f} -> {d.allocated[1] / GIB:.3f} GiB "
                     f"({(d.allocated[1] - d.allocated[0]) / GIB:+.3f}), reserved {(d.reserved[1] - d.reserved[0]) / GIB:+.3f}, "
                     f"peak {(d.peak[1] - d.peak[0]) / GIB:+.3f}")
        for title, rows in (("created", d.created), ("destroyed", d.destroyed), ("resized", d.resized)):
            for g in rows[:top]:
                na, nb = (g.a.n_tensors if g.a else 0), (g.b.n_tensors if g.b else 0)
                lines.append(f"    {title:9s} {g.delta_bytes / 2**20:+10.1f} MiB  {na} -> {nb} x {g.key}")
    return "\n".join(lines)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("a", type=Path)
    ap.add_argument("b", type=Path)
    ap.add_argument("--mark", type=str, default=None)
    ap.add_argument("--top", type=int, default=10)
    ap.add_argument("--peak-only", action="store_true")
    args = ap.parse_args()
    print(render(diff_ledgers(Ledger.load(args.a), Ledger.load(args.b), args.mark, args.peak_only), args.top))


if __name__ == "__main__":
    main()
