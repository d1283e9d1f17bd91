"""Turn local text into a published dataset of the store: tokenize, pack with document boundaries, row-shuffle.

Training never tokenizes or streams: the deterministic batch schedule reads a fixed set of int32 parquet shards.
This tool produces them, offline, from files already on disk (there is no hub access: source files and the
tokenizer's files are local paths).

Two steps, as the reference's tool:

  tokenize   each source file (parquet with a string column, `.jsonl` with that key, or `.txt` with one document
             per line) -> `<staging>/shard_<NNNNN>.parquet`, rows of paired `input_ids` / `document_ids` of
             length `seq_len` in packing order, plus `meta.json`. One source file is one unit of work: an output
             shard that already exists is skipped, so a killed invocation continues where it stopped, and
             `--task i --n-tasks n` lets n invocations split the files.
  finish     `<staging>` -> `<dataset dir>`: the same rows uniformly shuffled across the whole dataset
             (`data/row_shuffle.py`), with the `row_shuffle.json` every reader requires.

Document policy (`bos_eos`): each document becomes BOS, its text encoded WITHOUT special-token parsing (a literal
`<|end_of_text|>` in the text stays text), EOS, all under one document id; empty text gives BOS, EOS. Long
documents continue across rows without extra boundary tokens; the incomplete final row of each source file is
dropped. With `--llama3` the tokenizer must be a Llama 3 base tokenizer (BOS 128000, EOS 128001, 128256 entries,
no normalizer) and the preprocessing name is `llama3-bos-eos-v1`.

Parity: param_decomp/experiments/lm/data.py:18-45 (`pack_documents`), experiments/lm/llama3/data.py:33-123 (the
Llama 3 base-text policy), experiments/lm/llama3/prestage_tokenized.py (tokenize / finish, resumable per file).

`python -m param_decomp_b200.data.prestage tokenize --source <dir> --tokenizer-dir <dir> --out-dir <staging>
    --seq-len 513 [--column text] [--llama3] [--task 0 --n-tasks 1] [--workers 8]`
`python -m param_decomp_b200.data.prestage finish <staging> <data_root>/datasets/<name> [--seed 0]`
"""

from __future__ import annotations

import argparse
import json
import os
from collections.abc import Iterable, Iterator, Sequence
from concurrent.futures import ProcessPoolExecutor
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import numpy as np

from param_decomp_b200.formats import dataset_store as ds
from param_decomp_b200.formats.packed_rows import PackedRows

LLAMA3_PREPROCESSING_NAME = "llama3-bos-eos-v1"
BOS_EOS_PREPROCESSING_NAME = "bos-eos-v1"
SOURCE_SUFFIXES = (".parquet", ".jsonl", ".txt")


def pack_documents(documents: Sequence[Sequence[int]], max_length: int) -> PackedRows:
    """Concatenate the documents and cut rows of `max_length`; a row can hold several documents or a fragment of
    one. Document ids are local to this call (attention never crosses rows). The incomplete final row is dropped.
    Boundary tokens must already belong to their documents."""
    assert max_length > 0
    lengths = np.fromiter((len(d) for d in documents), dtype=np.int64, count=len(documents))
    assert (lengths > 0).all(), "encoded documents must contain at least one token"
    total = int(lengths.sum())
    flat = np.empty(total, dtype=np.int64)
    at = 0
    for d in documents:
        flat[at:at + len(d)] = d
        at += len(d)
    assert total == 0 or (flat.min() >= 0 and flat.max() <= np.iinfo(np.int32).max), "token ids must be non-negative int32"
    doc = np.repeat(np.arange(len(documents), dtype=np.int64), lengths)
    n = total // max_length * max_length
    tok_rows = flat[:n].astype(np.int32).reshape(-1, max_length)
    doc_rows = doc[:n].astype(np.int32).reshape(-1, max_length)
    return PackedRows(tok_rows, doc_rows)


@dataclass(frozen=True)
class BosEosPolicy:
    """BOS + literal text + EOS under one document id."""

    tokenizer: Any
    bos: int
    eos: int
    ordinary_below: int | None  # every text token must be below this id (special tokens sit above), when known
    name: str = BOS_EOS_PREPROCESSING_NAME

    def encode_document(self, text: str) -> tuple[int, ...]:
        try:
            ids = self.tokenizer.encode(text, add_special_tokens=False, split_special_tokens=True)
        except TypeError:  # a tokenizer without the switch: it has no special-token parsing to turn off
            ids = self.tokenizer.encode(text, add_special_tokens=False)
        if self.ordinary_below is not None:
            assert all(0 <= t < self.ordinary_below for t in ids), "document text must encode entirely as ordinary tokens"
        return (self.bos, *ids, self.eos)


def load_policy(tokenizer_dir: Path, llama3: bool) -> BosEosPolicy:
    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(str(tokenizer_dir), local_files_only=True)
    if llama3:
        assert tok.bos_token_id == 128000, "Llama 3 requires BOS token ID 128000"
        assert tok.eos_token_id == 128001, "Llama 3 requires EOS token ID 128001"
        assert len(tok) == 128256, "Llama 3 requires a 128256-token vocabulary"
        vocab = tok.get_vocab()
        for spelling, tid in (("<|begin_of_text|>", 128000), ("<|end_of_text|>", 128001), ("<|eot_id|>", 128009)):
            assert vocab.get(spelling) == tid, f"unexpected Llama 3 token: {spelling}"
        assert tok.backend_tokenizer.normalizer is None, "Llama 3 raw text must not be normalized"
        return BosEosPolicy(tok, 128000, 128001, 128000, LLAMA3_PREPROCESSING_NAME)
    assert tok.bos_token_id is not None and tok.eos_token_id is not None, (
        "the bos_eos policy needs a tokenizer that defines BOS and EOS")
    return BosEosPolicy(tok, int(tok.bos_token_id), int(tok.eos_token_id), None)


def read_documents(path: Path, column: str) -> Iterator[str]:
    """One string per document; a missing or null text is an empty document."""
    if path.suffix == ".parquet":
        import pyarrow as pa
        import pyarrow.parquet as pq

        f = pq.ParquetFile(path)
        assert column in f.schema_arrow.names, f"{path}: missing text column {column!r}"
        assert pa.types.is_string(f.schema_arrow.field(column).type) or pa.types.is_large_string(
            f.schema_arrow.field(column).type), f"{path}: {column!r} must be a string column"
        for batch in f.iter_batches(batch_size=1000, columns=[column]):
            for v in batch.column(0).to_pylist():
                yield v or ""
    elif path.suffix == ".jsonl":
        with path.open() as fh:
            for line in fh:
                if line.strip():
                    yield json.loads(line).get(column) or ""
    elif path.suffix == ".txt":
        with path.open() as fh:
            for line in fh:
                yield line.rstrip("\n")
    else:
        raise ValueError(f"{path}: source files are {SOURCE_SUFFIXES}")


def source_files(source: Path) -> list[Path]:
    source = Path(source)
    if source.is_file():
        return [source]
    files = sorted(p for p in source.rglob("*") if p.suffix in SOURCE_SUFFIXES and p.is_file())
    assert files, f"no {SOURCE_SUFFIXES} files under {source}"
    return files


def _batched(it: Iterable[str], n: int) -> Iterator[list[str]]:
    buf: list[str] = []
    for x in it:
        buf.append(x)
        if len(buf) == n:
            yield buf
            buf = []
    if buf:
        yield buf


def tokenize_file(policy: BosEosPolicy, path: Path, out: Path, seq_len: int, column: str,
                  rows_per_group: int = 8192) -> int:
    """One source file -> one shard; returns the rows written. Documents are packed as ONE stream per file, so
    only the file's final incomplete row is dropped. The shard appears under its name only when complete."""
    import pyarrow.parquet as pq

    from param_decomp_b200.data.row_shuffle import _table

    carry_tok = np.zeros(0, np.int64)
    carry_doc = np.zeros(0, np.int64)
    next_doc = 0
    tmp = out.with_suffix(".tmp")
    writer = None
    n_rows = 0
    try:
        for texts in _batched(read_documents(path, column), 1000):
            docs = [policy.encode_document(t) for t in texts]
            lengths = np.fromiter((len(d) for d in docs), np.int64, len(docs))
            tok = np.concatenate([carry_tok, np.fromiter((t for d in docs for t in d), np.int64, int(lengths.sum()))])
            doc = np.concatenate([carry_doc, np.repeat(np.arange(next_doc, next_doc + len(docs), dtype=np.int64), lengths)])
            next_doc += len(docs)
            n = tok.shape[0] // seq_len * seq_len
            if n:
                rows_t = tok[:n].astype(np.int32).reshape(-1, seq_len)
                rows_d = doc[:n].reshape(-1, seq_len)
                rows_d = (rows_d - rows_d[:, :1]).astype(np.int32)  # ids local to the row: attention never crosses rows
                PackedRows(rows_t, rows_d)  # validates the store's invariants
                table = _table(rows_t, rows_d)
                if writer is None:
                    writer = pq.ParquetWriter(tmp, table.schema)
                writer.write_table(table, row_group_size=rows_per_group)
                n_rows += rows_t.shape[0]
            carry_tok, carry_doc = tok[n:], doc[n:]
        if writer is None:  # a file too short for one row still leaves a (rowless) marker so it is not redone
            writer = pq.ParquetWriter(tmp, _table(np.zeros((0, seq_len), np.int32), np.zeros((0, seq_len), np.int32)).schema)
    finally:
        if writer is not None:
            writer.close()
    os.replace(tmp, out)
    return n_rows


def _tokenize_job(args: tuple[str, bool, str, str, int, str]) -> tuple[str, int]:
    tokenizer_dir, llama3, src, out, seq_len, column = args
    return out, tokenize_file(load_policy(Path(tokenizer_dir), llama3), Path(src), Path(out), seq_len, column)


def tokenize(source: Path, tokenizer_dir: Path, out_dir: Path, seq_len: int, column: str = "text", llama3: bool = False,
             task: int = 0, n_tasks: int = 1, workers: int = 1, tokenizer_name: str | None = None) -> list[Path]:
    """Writes this task's share of `<out_dir>/shard_<NNNNN>.parquet` (index = position of the source file in the
    sorted file list, so tasks never collide) and `meta.json`. Existing shards are left alone."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    policy = load_policy(Path(tokenizer_dir), llama3)  # fail on a wrong tokenizer before any work
    files = source_files(source)
    ds.write_dataset_meta(out_dir, ds.DatasetMeta(
        seq_len=seq_len, tokenizer_name=tokenizer_name or Path(tokenizer_dir).name, format_version=2,
        preprocessing_name=policy.name, end_of_document_token_id=policy.eos))
    jobs = []
    for i, f in enumerate(files):
        out = out_dir / f"shard_{i:05d}.parquet"
        if i % n_tasks == task and not out.exists():
            jobs.append((str(tokenizer_dir), llama3, str(f), str(out), seq_len, column))
    if workers <= 1:
        done = [_tokenize_job(j) for j in jobs]
    else:
        with ProcessPoolExecutor(max_workers=workers) as pool:
            done = list(pool.map(_tokenize_job, jobs))
    (out_dir / f"tokenize_task_{task:05d}_of_{n_tasks:05d}.json").write_text(json.dumps(
        {"source": str(source), "n_source_files": len(files), "written": {Path(o).name: n for o, n in done}}))
    return [Path(o) for o, _ in done]


def finish(staging_dir: Path, dataset_dir: Path, seed: int = 0, workers: int = 1, producer_revision: str | None = None,
           n_buckets: int | None = None) -> None:
    """Publish: every source file must have its shard; rowless shards are left out; rows are shuffled across the
    whole dataset."""
    from param_decomp_b200.data.row_shuffle import row_shuffle

    import pyarrow.parquet as pq

    staging_dir = Path(staging_dir)
    records = sorted(staging_dir.glob("tokenize_task_*.json"))
    assert records, f"{staging_dir}: no tokenize step has finished here"
    n_files = json.loads(records[0].read_text())["n_source_files"]
    shards = sorted(staging_dir.glob("shard_*.parquet"))
    assert len(shards) == n_files, f"{len(shards)} of {n_files} source files are tokenized; run the missing tasks first"
    for s in shards:  # rowless markers would break the readers' row-group arithmetic
        if pq.ParquetFile(s).metadata.num_rows == 0:
            s.unlink()
    row_shuffle(staging_dir, dataset_dir, seed, n_buckets=n_buckets, workers=workers)
    if producer_revision is not None:
        (Path(dataset_dir) / "producer.json").write_text(json.dumps({"producer_revision": producer_revision}))


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    t = sub.add_parser("tokenize")
    t.add_argument("--source", type=Path, required=True)
    t.add_argument("--tokenizer-dir", type=Path, required=True)
    t.add_argument("--tokenizer-name", type=str, default=None)
    t.add_argument("--out-dir", type=Path, required=True)
    t.add_argument("--seq-len", type=int, required=True)
    t.add_argument("--column", type=str, default="text")
    t.add_argument("--llama3", action="store_true")
    t.add_argument("--task", type=int, default=0)
    t.add_argument("--n-tasks", type=int, default=1)
    t.add_argument("--workers", type=int, default=max(1, (os.cpu_count() or 2) // 2))
    f = sub.add_parser("finish")
    f.add_argument("staging_dir", type=Path)
    f.add_argument("dataset_dir", type=Path)
    f.add_argument("--seed", type=int, default=0)
    f.add_argument("--workers", type=int, default=max(1, (os.cpu_count() or 2) // 2))
    f.add_argument("--producer-revision", type=str, default=None)
    args = ap.parse_args()
    if args.cmd == "tokenize":
        done = tokenize(args.source, args.tokenizer_dir, args.out_dir, args.seq_len, args.column, args.llama3,
                        args.task, args.n_tasks, args.workers, args.tokenizer_name)
        print(f"wrote {len(done)} shards under {args.out_dir}")
    else:
        finish(args.staging_dir, args.dataset_dir, args.seed, args.workers, args.producer_revision)
        print(f"published {args.dataset_dir}")


if __name__ == "__main__":
    main()
