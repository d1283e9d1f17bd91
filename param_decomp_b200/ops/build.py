"""Build the native sm_100a kernel library in-tree.

`python -m param_decomp_b200.ops.build` compiles every `csrc/*.cu` for `sm_100a` with nvcc
(cross-compiling needs no GPU) into `ops/_lib/libpdb200.so`. The library has a plain C ABI and is
loaded with `ctypes` (`native.py`), so it carries no dependency on the torch C++ headers and builds
in seconds. Object files are cached by source hash so only changed sources recompile.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

OPS_DIR = Path(__file__).resolve().parent
CSRC = OPS_DIR / "csrc"
LIB_DIR = OPS_DIR / "_lib"
LIB_PATH = LIB_DIR / "libpdb200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-lineinfo",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: the sm_100a kernels cannot be built")
    return cand


def _digest(path: Path, headers: list[Path]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for p in [path, *headers]:
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile changed sources and link the shared library. Returns its path."""
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    nvcc = _nvcc()

    jobs: list[tuple[Path, Path]] = []
    objects: list[Path] = []
    for src in sources:
        obj = obj_dir / f"{src.stem}.{_digest(src, headers)}.o"
        objects.append(obj)
        if force or not obj.exists():
            for stale in obj_dir.glob(f"{src.stem}.*.o"):
                stale.unlink()
            jobs.append((src, obj))

    def compile_one(job: tuple[Path, Path]) -> None:
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            list(pool.map(compile_one, jobs))

    if jobs or not LIB_PATH.exists():
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objects), "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB_PATH


HOST_SRC = OPS_DIR / "csrc_host"
HOST_LIB_PATH = LIB_DIR / "libpdhost.so"
HOST_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-shared", "-fno-math-errno"]


def build_host(force: bool = False) -> Path:
    """The host-side native pieces (`csrc_host/*.cpp`: the CPU twin of the device mask stream) into
    `ops/_lib/libpdhost.so` with the system C++ compiler. Plain C ABI, loaded with `ctypes` (`host_native.py`);
    callers fall back to the pure-torch forms when it has not been built."""
    LIB_DIR.mkdir(exist_ok=True)
    sources = sorted(HOST_SRC.glob("*.cpp"))
    h = hashlib.sha256(" ".join(HOST_FLAGS).encode())
    for src in sources:
        h.update(src.read_bytes())
    stamp = LIB_DIR / "libpdhost.digest"
    digest = h.hexdigest()
    if not force and HOST_LIB_PATH.exists() and stamp.exists() and stamp.read_text() == digest:
        return HOST_LIB_PATH
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("no C++ compiler found: the host library cannot be built")
    res = subprocess.run([cxx, *HOST_FLAGS, *map(str, sources), "-o", str(HOST_LIB_PATH)], capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("host library build failed")
    stamp.write_text(digest)
    return HOST_LIB_PATH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="--force" in sys.argv))
    print(build_host(force="--force" in sys.argv))
