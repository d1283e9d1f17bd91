"""Out-of-core uniform row shuffle of a packed dataset, with a verified multiset fingerprint.

The batch schedule cuts every batch from consecutive rows of one or two parquet row groups, so a corpus stored
in packing order would serve batches of neighbouring rows from one source file. This tool permutes whole rows
across the corpus without ever holding the corpus in memory:

  scatter   every source shard (one worker process each) gives each of its rows a seeded random bucket and
            writes ONE staging file whose row groups are its non-empty buckets, in bucket order; a sidecar
            lists which row group is which bucket. Memory: one source shard.
  gather    every bucket (one worker each) reads its row group from every staging file, permutes the rows
            with a seeded generator and writes one output shard. Memory: one bucket, i.e. corpus / n_buckets.

A uniform bucket per row followed by a uniform permutation inside each bucket is a uniform permutation of the
corpus. Rows are never edited: token and document IDs travel together. Before the record is published every
output shard is re-read and the fingerprint of all output rows (count, wrapped sum and XOR of a 64-bit hash per
row: equal for equal multisets, in any order) must equal that of the source rows.

`row_shuffle.json` (required by every reader, `formats/dataset_store.py::assert_row_shuffled`) records the
source, the digest of its metadata, the seed, the bucket count and the fingerprint.

Parity: param_decomp/infra/row_shuffle.py:1-310 (two passes through a staging directory, order-independent
fingerprint check, `row_shuffle.json`); the hash construction and file layout here are this package's own.

`python -m param_decomp_b200.data.row_shuffle <src_dir> <dst_dir> --seed 0 [--buckets N] [--workers W]`
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os
import shutil
from concurrent.futures import ProcessPoolExecutor
from dataclasses import dataclass
from pathlib import Path

import numpy as np

from param_decomp_b200.formats import dataset_store as ds

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


@dataclass(frozen=True)
class Fingerprint:
    """Order-independent summary of a multiset of rows."""

    rows: int
    hash_sum: int
    hash_xor: int

    def __add__(self, other: "Fingerprint") -> "Fingerprint":
        return Fingerprint(self.rows + other.rows, (self.hash_sum + other.hash_sum) & 0xFFFFFFFFFFFFFFFF,
                           self.hash_xor ^ other.hash_xor)


EMPTY = Fingerprint(0, 0, 0)


def _mix(x: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser, elementwise on uint64."""
    with np.errstate(over="ignore"):
        x = (x ^ (x >> np.uint64(30))) * _M1
        x = (x ^ (x >> np.uint64(27))) * _M2
        return x ^ (x >> np.uint64(31))


def fingerprint(token_ids: np.ndarray, document_ids: np.ndarray) -> Fingerprint:
    """Row hash: a position-keyed mix of every token and document id, chained so that neither swapping two
    positions nor moving an id between the two columns leaves it unchanged."""
    assert token_ids.shape == document_ids.shape and token_ids.ndim == 2
    if token_ids.shape[0] == 0:
        return EMPTY
    with np.errstate(over="ignore"):
        pos = (np.arange(token_ids.shape[1], dtype=np.uint64) + np.uint64(1)) * _GOLDEN
        a = _mix(token_ids.astype(np.uint64) + pos[None, :])
        b = _mix(document_ids.astype(np.uint64) * np.uint64(3) + pos[None, :] * np.uint64(5) + np.uint64(1))
        h = _mix(a.sum(axis=1, dtype=np.uint64) ^ _mix(b.sum(axis=1, dtype=np.uint64)))
        return Fingerprint(int(h.shape[0]), int(h.sum(dtype=np.uint64)), int(np.bitwise_xor.reduce(h)))


def _read_shard(path: Path) -> tuple[np.ndarray, np.ndarray]:
    import pyarrow.parquet as pq

    table = pq.read_table(path)
    assert set(table.column_names) == {"input_ids", "document_ids"}, f"{path}: needs input_ids and document_ids"

    def col(name: str) -> np.ndarray:
        c = table.column(name).combine_chunks()
        flat = c.flatten().to_numpy(zero_copy_only=False)
        assert len(c) > 0 and flat.size % len(c) == 0, f"{path}: ragged {name}"
        return flat.reshape(len(c), -1).astype(np.int32, copy=False)

    return col("input_ids"), col("document_ids")


def _table(tok: np.ndarray, doc: np.ndarray):
    import pyarrow as pa

    width = tok.shape[1]

    def lists(a: np.ndarray):
        offsets = pa.array(np.arange(0, (a.shape[0] + 1) * width, width, dtype=np.int32))
        return pa.ListArray.from_arrays(offsets, pa.array(np.ascontiguousarray(a, np.int32).reshape(-1)))

    return pa.table({"input_ids": lists(tok), "document_ids": lists(doc)})


def _scatter_one(args: tuple[str, str, int, int, int]) -> tuple[int, int, int]:
    src, staging, index, seed, n_buckets = args
    import pyarrow.parquet as pq

    tok, doc = _read_shard(Path(src))
    fp = fingerprint(tok, doc)
    bucket = np.random.default_rng([seed, 0, index]).integers(0, n_buckets, size=tok.shape[0])
    order = np.argsort(bucket, kind="stable")
    tok, doc, bucket = tok[order], doc[order], bucket[order]
    present, starts = np.unique(bucket, return_index=True)
    ends = list(starts[1:]) + [tok.shape[0]]
    out = Path(staging) / f"scatter_{index:05d}.parquet"
    tmp = out.with_suffix(".tmp")
    with pq.ParquetWriter(tmp, _table(tok[:0], doc[:0]).schema) as w:
        for s, e in zip(starts, ends):
            w.write_table(_table(tok[s:e], doc[s:e]), row_group_size=int(e - s))
    os.replace(tmp, out)
    out.with_suffix(".json").write_text(json.dumps({"buckets": [int(b) for b in present]}))
    return fp.rows, fp.hash_sum, fp.hash_xor


def _gather_one(args: tuple[str, str, int, int, int, int]) -> tuple[int, int, int]:
    staging, dst, b, seed, n_sources, rows_per_group = args
    import pyarrow.parquet as pq

    toks, docs = [], []
    for i in range(n_sources):
        f = Path(staging) / f"scatter_{i:05d}.parquet"
        present = json.loads(f.with_suffix(".json").read_text())["buckets"]
        if b not in present:
            continue
        t = pq.ParquetFile(f).read_row_group(present.index(b))
        width = len(t.column("input_ids")[0])
        toks.append(t.column("input_ids").combine_chunks().flatten().to_numpy(zero_copy_only=False).reshape(-1, width))
        docs.append(t.column("document_ids").combine_chunks().flatten().to_numpy(zero_copy_only=False).reshape(-1, width))
    if not toks:
        return 0, 0, 0
    tok, doc = np.concatenate(toks), np.concatenate(docs)
    perm = np.random.default_rng([seed, 1, b]).permutation(tok.shape[0])
    tok, doc = tok[perm], doc[perm]
    out = Path(dst) / f"shard_{b:05d}.parquet"
    tmp = out.with_suffix(".tmp")
    pq.write_table(_table(tok, doc), tmp, row_group_size=rows_per_group)
    os.replace(tmp, out)
    fp = fingerprint(*_read_shard(out))  # re-read what was written, not what was meant
    return fp.rows, fp.hash_sum, fp.hash_xor


def _sum(parts: list[tuple[int, int, int]]) -> Fingerprint:
    total = EMPTY
    for p in parts:
        total = total + Fingerprint(*p)
    return total


def row_shuffle(src_dir: Path, dst_dir: Path, seed: int, n_buckets: int | None = None, workers: int = 1,
                rows_per_group: int = 8192, staging_dir: Path | None = None) -> Fingerprint:
    """Write `dst_dir` = the rows of `src_dir` in a seeded uniform order, with `meta.json` carried over and
    `row_shuffle.json` recording how. `n_buckets` = number of output shards (default: as many as the source)."""
    src_dir, dst_dir = Path(src_dir), Path(dst_dir)
    assert src_dir.resolve() != dst_dir.resolve(), "shuffle into a new directory; datasets are immutable"
    meta = ds.read_dataset_meta(src_dir)
    sources = sorted(src_dir.glob("*.parquet"))
    assert sources, f"no *.parquet under {src_dir}"
    n_buckets = n_buckets or len(sources)
    dst_dir.mkdir(parents=True, exist_ok=True)
    assert not list(dst_dir.glob("*.parquet")), f"{dst_dir} already holds shards"
    staging = Path(staging_dir) if staging_dir is not None else dst_dir / ".row_shuffle_staging"
    staging.mkdir(parents=True, exist_ok=True)

    def run(fn, jobs):
        if workers <= 1:
            return [fn(j) for j in jobs]
        with ProcessPoolExecutor(max_workers=workers) as pool:
            return list(pool.map(fn, jobs))

    try:
        before = _sum(run(_scatter_one, [(str(f), str(staging), i, seed, n_buckets) for i, f in enumerate(sources)]))
        after = _sum(run(_gather_one, [(str(staging), str(dst_dir), b, seed, len(sources), rows_per_group)
                                       for b in range(n_buckets)]))
    finally:
        shutil.rmtree(staging, ignore_errors=True)
    assert after == before, f"shuffled rows differ from the source rows: {before} -> {after}"
    ds.write_dataset_meta(dst_dir, meta)
    record = {
        "method": "bucket_scatter_gather", "seed": seed, "n_buckets": n_buckets, "n_rows": before.rows,
        "source": str(src_dir), "source_meta_sha256": hashlib.sha256((src_dir / ds.DATASET_META_FILENAME).read_bytes()).hexdigest(),
        "fingerprint": {"rows": before.rows, "hash_sum": before.hash_sum, "hash_xor": before.hash_xor},
    }
    tmp = dst_dir / f".{ds.ROW_SHUFFLE_FILENAME}.tmp"
    tmp.write_text(json.dumps(record, indent=1) + "\n")
    os.replace(tmp, dst_dir / ds.ROW_SHUFFLE_FILENAME)
    return before


def dataset_fingerprint(data_dir: Path) -> Fingerprint:
    return _sum([tuple(fingerprint(*_read_shard(f)).__dict__.values()) for f in sorted(Path(data_dir).glob("*.parquet"))])


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("src_dir", type=Path)
    ap.add_argument("dst_dir", type=Path)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--buckets", type=int, default=None)
    ap.add_argument("--workers", type=int, default=max(1, (os.cpu_count() or 2) // 2))
    ap.add_argument("--rows-per-group", type=int, default=8192)
    args = ap.parse_args()
    fp = row_shuffle(args.src_dir, args.dst_dir, args.seed, args.buckets, args.workers, args.rows_per_group)
    print(json.dumps({"rows": fp.rows, "hash_sum": fp.hash_sum, "hash_xor": fp.hash_xor}))


if __name__ == "__main__":
    main()
