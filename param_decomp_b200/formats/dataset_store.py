"""The dataset-store contract: `<data_root>/datasets/<name>/{*.parquet, meta.json, row_shuffle.json}`.

Parity: param_decomp_formats/dataset_store.py:33-157 and datasets.py:34-110 (shard scan, row-group
reads cut to `seq_len`, the `DatasetRef` union configs name shards by).
"""

from __future__ import annotations

import json
import os
from collections.abc import Callable, Sequence
from dataclasses import dataclass
from pathlib import Path
from typing import Annotated, Literal, Self

import numpy as np
from pydantic import Discriminator, Field, NonNegativeInt, PositiveInt, model_validator

from param_decomp_b200.formats.base import BaseConfig
from param_decomp_b200.formats.packed_rows import PackedRows

DATASET_META_FILENAME = "meta.json"
ROW_SHUFFLE_FILENAME = "row_shuffle.json"


def dataset_dir(data_root: Path, name: str) -> Path:
    return Path(data_root) / "datasets" / name


class NamedDataset(BaseConfig):
    kind: Literal["name"] = "name"
    name: str

    @model_validator(mode="after")
    def _flat(self) -> Self:
        bad = self.name in ("", ".", "..") or any(ch in self.name for ch in "/\\*?[")
        assert not bad, f"dataset names are flat store names: {self.name!r}"
        return self


class DatasetDir(BaseConfig):
    kind: Literal["dir"] = "dir"
    dir: Path

    @model_validator(mode="after")
    def _abs(self) -> Self:
        assert self.dir.is_absolute(), f"ad-hoc shard dirs are absolute paths: {self.dir}"
        return self


DatasetRef = Annotated[NamedDataset | DatasetDir, Discriminator("kind")]
DataLayout = Literal["documents", "unsegmented_tokens"]


def resolve_dataset_ref(ref: NamedDataset | DatasetDir, data_root: Path) -> Path:
    return dataset_dir(data_root, ref.name) if isinstance(ref, NamedDataset) else ref.dir


class DatasetIdentity(BaseConfig):
    seq_len: PositiveInt
    tokenizer_name: str = Field(min_length=1)


class DatasetMeta(DatasetIdentity):
    format_version: Literal[2]
    preprocessing_name: str = Field(min_length=1)
    end_of_document_token_id: NonNegativeInt | None = None


def read_dataset_identity(data_dir: Path) -> DatasetIdentity:
    raw = json.loads((Path(data_dir) / DATASET_META_FILENAME).read_text())
    return DatasetIdentity(seq_len=raw["seq_len"], tokenizer_name=raw["tokenizer_name"])


def read_dataset_meta(data_dir: Path) -> DatasetMeta:
    path = Path(data_dir) / DATASET_META_FILENAME
    assert path.exists(), f"no {DATASET_META_FILENAME} in {data_dir}: dataset dirs are self-describing"
    return DatasetMeta.model_validate_json(path.read_text())


def assert_records_documents(data_dir: Path) -> DatasetMeta:
    path = Path(data_dir) / DATASET_META_FILENAME
    assert not path.exists() or "format_version" in json.loads(path.read_text()), (
        f"{data_dir} is a token-only dataset with no document IDs"
    )
    return read_dataset_meta(data_dir)


def assert_row_shuffled(data_dir: Path) -> None:
    assert (Path(data_dir) / ROW_SHUFFLE_FILENAME).exists(), (
        f"{data_dir} records no row shuffle ({ROW_SHUFFLE_FILENAME}): contiguous rows of a packed "
        "corpus are a few long documents, not a sample"
    )


def write_dataset_meta(data_dir: Path, meta: DatasetMeta) -> None:
    """Atomic publish: write a temp file, hard-link it into place, tolerate an identical winner."""
    data_dir = Path(data_dir)
    data_dir.mkdir(parents=True, exist_ok=True)
    path = data_dir / DATASET_META_FILENAME
    tmp = data_dir / f".meta.{os.getpid()}.tmp"
    tmp.write_text(meta.model_dump_json() + "\n")
    try:
        os.link(tmp, path)
    except FileExistsError:
        assert read_dataset_meta(data_dir) == meta, f"dataset metadata differs in {data_dir}"
    finally:
        tmp.unlink()


# ---- parquet shards ------------------------------------------------------------------------


@dataclass(frozen=True)
class RowGroupInfo:
    start_row: int
    n_rows: int


@dataclass(frozen=True)
class ShardInfo:
    path: Path
    row_groups: tuple[RowGroupInfo, ...]

    @property
    def n_rows(self) -> int:
        return sum(g.n_rows for g in self.row_groups)


def scan_shards(data_dir: Path) -> tuple[ShardInfo, ...]:
    import pyarrow.parquet as pq

    files = sorted(Path(data_dir).glob("*.parquet"))
    assert files, f"no *.parquet under {data_dir}"
    out = []
    for f in files:
        md = pq.ParquetFile(f).metadata
        groups, start = [], 0
        for i in range(md.num_row_groups):
            n = md.row_group(i).num_rows
            groups.append(RowGroupInfo(start, n))
            start += n
        out.append(ShardInfo(f, tuple(groups)))
    return tuple(out)


def _id_column(table, name: str, seq_len: int) -> np.ndarray:
    import pyarrow as pa

    col = table.column(name).combine_chunks()
    ok_type = pa.types.is_list(col.type) or pa.types.is_large_list(col.type) or pa.types.is_fixed_size_list(col.type)
    assert ok_type and col.type.value_type == pa.int32(), f"{name} must be an int32 list column"
    assert col.null_count == 0, f"{name} has null rows"
    flat = col.flatten().to_numpy(zero_copy_only=False)
    n = len(col)
    assert n > 0 and flat.size % n == 0, f"{name} rows must have equal lengths"
    width = flat.size // n
    assert width in (seq_len, seq_len + 1), f"{name} rows have seq {width}, config says {seq_len}"
    return flat.reshape(n, width)


OpenShard = Callable[[Path], object]


def _default_open(path: Path):
    import pyarrow.parquet as pq

    return pq.ParquetFile(path)


def read_row_group(shard: ShardInfo, idx: int, seq_len: int, open_shard: OpenShard = _default_open) -> PackedRows:
    table = open_shard(shard.path).read_row_group(idx)
    assert set(table.column_names) == {"input_ids", "document_ids"}, (
        f"{shard.path}: shards require input_ids and document_ids"
    )
    tok = _id_column(table, "input_ids", seq_len)[:, :seq_len]
    doc = _id_column(table, "document_ids", seq_len)[:, :seq_len]
    return PackedRows(np.ascontiguousarray(tok), np.ascontiguousarray(doc))


def read_shard_rows(shard: ShardInfo, rows: Sequence[int], seq_len: int, open_shard: OpenShard = _default_open) -> PackedRows:
    assert all(0 <= r < shard.n_rows for r in rows), (rows, shard.n_rows)
    starts = np.array([g.start_row for g in shard.row_groups])
    which = np.searchsorted(starts, rows, side="right") - 1
    cache = {int(g): read_row_group(shard, int(g), seq_len, open_shard) for g in set(which.tolist())}
    local = np.asarray(rows) - starts[which]
    tok = np.stack([cache[int(g)].token_ids[int(i)] for g, i in zip(which, local)])
    doc = np.stack([cache[int(g)].document_ids[int(i)] for g, i in zip(which, local)])
    return PackedRows(tok, doc)
