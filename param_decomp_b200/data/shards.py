"""Pre-tokenised parquet datasets: the deterministic batch schedule, the per-process shard reader
with prefetch, and the global row shuffle that prepares a corpus for training.

Schedule: a pure function of `(seed, epoch, step)` -> `(shard, row group, rows)`. Each epoch visits
every row group once in a seeded order; within a row group rows are taken in a seeded order, and a
batch is cut from one row group (continuing into the next when it runs out). Because nothing but
`step` advances, a resumed run reads exactly the rows it would have read.
Every rank computes the same global schedule and reads only its own rows (no communication).

Parity: param_decomp/lm/batch_schedule.py:76-175 (`BatchSchedule`), lm/batch_data.py:58-239
(`ShardServer`, prefetch, document layouts), lm/batch.py (`LMBatch*`), sequence.py:12-41
(`SequenceLayout`), infra/row_shuffle.py:55-310 (scatter/gather row shuffle with fingerprints).
"""

from __future__ import annotations

import hashlib
import json
import threading
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import numpy as np
import torch

from param_decomp_b200.formats import dataset_store as ds
from param_decomp_b200.formats.packed_rows import PackedRows
from param_decomp_b200.models.transformer import LMBatch


@dataclass(frozen=True)
class RowAddress:
    shard: int
    row_group: int
    row: int  # within the row group


class BatchSchedule:
    """`rows_for(step)` = the global batch's row addresses, a pure function of (seed, step)."""

    def __init__(self, shards: tuple[ds.ShardInfo, ...], batch_rows: int, seed: int) -> None:
        self.shards, self.batch_rows, self.seed = shards, batch_rows, seed
        self.groups = [(si, gi, g.n_rows) for si, s in enumerate(shards) for gi, g in enumerate(s.row_groups)]
        self.rows_per_epoch = sum(n for _, _, n in self.groups)
        assert self.rows_per_epoch >= batch_rows, "dataset smaller than one batch"

    def _epoch_order(self, epoch: int) -> np.ndarray:
        return np.random.default_rng([self.seed, epoch, 0]).permutation(len(self.groups))

    def _group_rows(self, epoch: int, group_idx: int, n_rows: int) -> np.ndarray:
        return np.random.default_rng([self.seed, epoch, 1, group_idx]).permutation(n_rows)

    def rows_for(self, step: int) -> list[RowAddress]:
        start = step * self.batch_rows
        out: list[RowAddress] = []
        while len(out) < self.batch_rows:
            pos = start + len(out)
            epoch, offset = divmod(pos, self.rows_per_epoch)
            order = self._epoch_order(epoch)
            sizes = np.array([self.groups[g][2] for g in order])
            ends = np.cumsum(sizes)
            k = int(np.searchsorted(ends, offset, side="right"))
            gidx = int(order[k])
            si, gi, n = self.groups[gidx]
            within = offset - (int(ends[k - 1]) if k > 0 else 0)
            perm = self._group_rows(epoch, gidx, n)
            take = min(n - within, self.batch_rows - len(out))
            out.extend(RowAddress(si, gi, int(r)) for r in perm[within:within + take])
        return out


def sequence_layout(rows: PackedRows, layout: str) -> tuple[np.ndarray, np.ndarray | None, np.ndarray | None]:
    """`documents`: segment ids + within-document positions (attention and next-token terms stay
    inside each document); `unsegmented_tokens`: one unbroken sequence per row."""
    if layout == "unsegmented_tokens":
        return rows.token_ids, None, None
    seg = rows.document_ids
    start = np.concatenate([np.ones((seg.shape[0], 1), bool), np.diff(seg, axis=1) != 0], axis=1)
    idx = np.arange(seg.shape[1])[None, :].repeat(seg.shape[0], 0)
    doc_start = np.maximum.accumulate(np.where(start, idx, 0), axis=1)
    return rows.token_ids, seg, (idx - doc_start).astype(np.int32)


class ShardServer:
    """Per-process reader: computes the global schedule, reads this rank's rows, prefetches the next
    step on a background thread, returns pinned host tensors."""

    def __init__(self, data_dir: Path, seq_len: int, layout: str, seed: int, vocab_size: int | None = None) -> None:
        ds.assert_row_shuffled(data_dir)
        meta = ds.assert_records_documents(data_dir)
        assert meta.seq_len in (seq_len, seq_len + 1) or meta.seq_len >= seq_len, (meta.seq_len, seq_len)
        self.data_dir, self.seq_len, self.layout, self.seed = Path(data_dir), seq_len, layout, seed
        self.meta = meta
        self.shards = ds.scan_shards(self.data_dir)
        self.vocab_size = vocab_size
        self._schedules: dict[int, BatchSchedule] = {}
        self._cache: dict[tuple[int, int], PackedRows] = {}
        self._prefetched: dict[tuple, Any] = {}
        self._lock = threading.Lock()

    @classmethod
    def open(cls, ref: Any, data_root: Path, seq_len: int, layout: str, seed: int) -> "ShardServer":
        return cls(ds.resolve_dataset_ref(ref, data_root), seq_len, layout, seed)

    def _group(self, si: int, gi: int) -> PackedRows:
        key = (si, gi)
        with self._lock:
            hit = self._cache.get(key)
        if hit is None:
            hit = ds.read_row_group(self.shards[si], gi, self.seq_len)
            if self.vocab_size is not None:
                hit.validate_vocabulary(self.vocab_size)
            with self._lock:
                if len(self._cache) > 8:
                    self._cache.pop(next(iter(self._cache)))
                self._cache[key] = hit
        return hit

    def _read(self, step: int, global_rows: int, rank: int, world: int) -> PackedRows:
        sched = self._schedules.setdefault(global_rows, BatchSchedule(self.shards, global_rows, self.seed))
        per = global_rows // world
        mine = sched.rows_for(step)[rank * per:(rank + 1) * per]
        tok = np.stack([self._group(a.shard, a.row_group).token_ids[a.row] for a in mine])
        doc = np.stack([self._group(a.shard, a.row_group).document_ids[a.row] for a in mine])
        return PackedRows(tok, doc)

    def batch(self, step: int, global_rows: int, rank: int = 0, world: int = 1, pin: bool = False) -> LMBatch:
        key = (step, global_rows, rank, world)
        fut = self._prefetched.pop(key, None)
        rows = fut.result() if fut is not None else self._read(step, global_rows, rank, world)
        nxt = (step + 1, global_rows, rank, world)
        if nxt not in self._prefetched:
            self._prefetched[nxt] = _Future(lambda: self._read(step + 1, global_rows, rank, world))
        tok, seg, pos = sequence_layout(rows, self.layout)

        def t(a):
            if a is None:
                return None
            x = torch.from_numpy(np.ascontiguousarray(a))
            return x.pin_memory() if pin and torch.cuda.is_available() else x

        return LMBatch(t(tok), t(seg), t(pos))


class _Future:
    def __init__(self, fn) -> None:
        self._out, self._err = None, None
        self._t = threading.Thread(target=self._run, args=(fn,), daemon=True)
        self._t.start()

    def _run(self, fn) -> None:
        try:
            self._out = fn()
        except BaseException as e:  # surfaced on result()
            self._err = e

    def result(self):
        self._t.join()
        if self._err is not None:
            raise self._err
        return self._out


# ---- producing datasets -------------------------------------------------------------------------


def write_token_dataset(data_dir: Path, token_ids: np.ndarray, document_ids: np.ndarray | None, tokenizer_name: str,
                        rows_per_group: int = 1024, rows_per_shard: int = 8192, preprocessing_name: str = "synthetic",
                        shuffle_seed: int | None = 0) -> None:
    """Write `[rows, width]` int32 tokens as a store dataset (parquet shards + meta.json), then
    row-shuffle it in place and record the shuffle."""
    import pyarrow as pa
    import pyarrow.parquet as pq

    data_dir = Path(data_dir)
    data_dir.mkdir(parents=True, exist_ok=True)
    token_ids = np.ascontiguousarray(token_ids, dtype=np.int32)
    document_ids = np.zeros_like(token_ids) if document_ids is None else np.ascontiguousarray(document_ids, np.int32)
    order = np.arange(token_ids.shape[0])
    if shuffle_seed is not None:
        order = np.random.default_rng(shuffle_seed).permutation(token_ids.shape[0])
    token_ids, document_ids = token_ids[order], document_ids[order]
    for si, s in enumerate(range(0, token_ids.shape[0], rows_per_shard)):
        tok, doc = token_ids[s:s + rows_per_shard], document_ids[s:s + rows_per_shard]
        table = pa.table({"input_ids": pa.array(tok.tolist(), type=pa.list_(pa.int32())),
                          "document_ids": pa.array(doc.tolist(), type=pa.list_(pa.int32()))})
        pq.write_table(table, data_dir / f"shard_{si:05d}.parquet", row_group_size=rows_per_group)
    ds.write_dataset_meta(data_dir, ds.DatasetMeta(seq_len=token_ids.shape[1], tokenizer_name=tokenizer_name,
                                                   format_version=2, preprocessing_name=preprocessing_name))
    if shuffle_seed is not None:
        record_row_shuffle(data_dir, shuffle_seed, order)


def record_row_shuffle(data_dir: Path, seed: int, order: np.ndarray) -> None:
    fp = hashlib.sha256(np.ascontiguousarray(order, dtype=np.int64).tobytes()).hexdigest()
    (Path(data_dir) / ds.ROW_SHUFFLE_FILENAME).write_text(json.dumps(
        {"seed": seed, "n_rows": int(order.shape[0]), "permutation_sha256": fp, "method": "global_permutation"}))


def row_shuffle_dataset(src_dir: Path, dst_dir: Path, seed: int, rows_per_group: int = 1024,
                        rows_per_shard: int = 8192) -> None:
    """Uniformly permute the rows of a packed dataset across all of its shards (scatter the rows by
    a seeded global permutation, gather them into new shards) and record how."""
    src_dir = Path(src_dir)
    meta = ds.read_dataset_meta(src_dir)
    toks, docs = [], []
    for shard in ds.scan_shards(src_dir):
        for gi in range(len(shard.row_groups)):
            rows = ds.read_row_group(shard, gi, meta.seq_len)
            toks.append(rows.token_ids)
            docs.append(rows.document_ids)
    write_token_dataset(dst_dir, np.concatenate(toks), np.concatenate(docs), meta.tokenizer_name, rows_per_group,
                        rows_per_shard, meta.preprocessing_name, shuffle_seed=seed)
