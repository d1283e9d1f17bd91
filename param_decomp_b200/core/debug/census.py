"""Census of what one training step launches: kernels of this library by entry point, torch kernels,
and collectives by kind. The analogue of the reference's HLO collective census
(param_decomp/core/tools/hlo_census.py:190-...): there the compiler inserts the collectives and the
census reads them back out of the compiled program; here they are explicit calls, so the census
counts them where they are issued and checks them against what a placement is expected to issue.
"""

from __future__ import annotations

import contextlib
import ctypes
from collections import Counter
from dataclasses import dataclass, field
from typing import Any, Iterator

import torch
import torch.distributed as dist

_COLLECTIVES = ("all_reduce", "all_gather_into_tensor", "reduce_scatter_tensor", "all_to_all_single", "broadcast",
                "all_gather", "barrier")


@dataclass
class Census:
    native: Counter = field(default_factory=Counter)       # pd_* entry point -> launches
    collectives: Counter = field(default_factory=Counter)  # torch.distributed function -> calls
    collective_bytes: Counter = field(default_factory=Counter)

    def summary(self) -> dict[str, Any]:
        return {"native_launches": sum(self.native.values()), "native": dict(self.native.most_common()),
                "collectives": dict(self.collectives), "collective_bytes": dict(self.collective_bytes)}

    def assert_collectives(self, allowed: set[str]) -> None:
        """A placement names the collective kinds a step may issue; anything else is a bug."""
        extra = set(self.collectives) - allowed
        assert not extra, f"unexpected collectives in the step: {sorted(extra)} (allowed {sorted(allowed)})"


@contextlib.contextmanager
def census() -> Iterator[Census]:
    """Count native entry points (by wrapping the C functions of the loaded library) and
    `torch.distributed` collectives issued inside the block."""
    from param_decomp_b200.ops import native as nv

    c = Census()
    patched: list[tuple[Any, str, Any]] = []
    if nv.LIB_PATH.exists():
        lib = nv.lib()
        import subprocess

        names = [ln.split()[-1] for ln in subprocess.run(["nm", "-D", "--defined-only", str(nv.LIB_PATH)],
                                                         capture_output=True, text=True).stdout.splitlines()
                 if ln.split() and ln.split()[-1].startswith("pd_")]
        for name in names:
            fn = getattr(lib, name)
            if not isinstance(fn, ctypes._CFuncPtr):  # type: ignore[attr-defined]
                continue

            class _Counting:
                def __init__(self, inner: Any, key: str) -> None:
                    self.inner, self.key = inner, key

                def __call__(self, *a: Any) -> Any:
                    c.native[self.key] += 1
                    return self.inner(*a)

                def __getattr__(self, item: str) -> Any:
                    return getattr(self.inner, item)

                def __setattr__(self, k: str, v: Any) -> None:
                    if k in ("inner", "key"):
                        object.__setattr__(self, k, v)
                    else:
                        setattr(self.inner, k, v)

            patched.append((lib, name, fn))
            lib.__dict__[name] = _Counting(fn, name)  # CDLL caches resolved symbols in its __dict__
        nv._pd_gemm.cache_clear()
    originals = {}
    for name in _COLLECTIVES:
        if not hasattr(dist, name):
            continue
        orig = getattr(dist, name)
        originals[name] = orig

        def wrap(orig=orig, name=name):
            def inner(*a: Any, **k: Any) -> Any:
                c.collectives[name] += 1
                for t in a:
                    if isinstance(t, torch.Tensor):
                        c.collective_bytes[name] += t.numel() * t.element_size()
                        break
                return orig(*a, **k)

            return inner

        setattr(dist, name, wrap())
    try:
        yield c
    finally:
        for name, orig in originals.items():
            setattr(dist, name, orig)
        for lib, name, fn in patched:
            lib.__dict__[name] = fn
        if patched:
            nv._pd_gemm.cache_clear()
