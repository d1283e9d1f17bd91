import numpy as np
import pytest

from param_decomp_b200.data.shards import BatchSchedule, ShardServer, row_shuffle_dataset, write_token_dataset
from param_decomp_b200.data.synthetic import ZipfTokenSource
from param_decomp_b200.formats import dataset_store as ds
from param_decomp_b200.formats.packed_rows import PackedRows


def make(tmp_path, rows=300, width=17):
    rng = np.random.default_rng(0)
    tok = rng.integers(0, 100, size=(rows, width), dtype=np.int32)
    doc = np.cumsum(rng.random((rows, width)) < 0.2, axis=1).astype(np.int32)
    write_token_dataset(tmp_path / "datasets" / "toy", tok, doc, "tok", rows_per_group=32, rows_per_shard=128)
    return tok, doc


def test_schedule_is_pure_and_covers_an_epoch(tmp_path):
    tok, _ = make(tmp_path)
    shards = ds.scan_shards(tmp_path / "datasets" / "toy")
    s1, s2 = BatchSchedule(shards, 20, seed=3), BatchSchedule(shards, 20, seed=3)
    assert s1.rows_for(7) == s2.rows_for(7)
    seen = [a for step in range(15) for a in s1.rows_for(step)]
    assert len(set(seen)) == 300  # one epoch = every row exactly once
    assert BatchSchedule(shards, 20, seed=4).rows_for(0) != s1.rows_for(0)


def test_ranks_partition_the_global_batch(tmp_path):
    make(tmp_path)
    d = tmp_path / "datasets" / "toy"
    whole = ShardServer(d, 16, "unsegmented_tokens", seed=1).batch(5, 8).tokens
    parts = [ShardServer(d, 16, "unsegmented_tokens", seed=1).batch(5, 8, r, 4).tokens for r in range(4)]
    assert whole.shape == (8, 16) and (np.concatenate([p.numpy() for p in parts]) == whole.numpy()).all()


def test_document_layout_positions(tmp_path):
    make(tmp_path)
    b = ShardServer(tmp_path / "datasets" / "toy", 16, "documents", seed=1).batch(0, 4)
    seg, pos = b.segment_ids.numpy(), b.positions.numpy()
    assert (pos[:, 0] == 0).all()
    same = seg[:, 1:] == seg[:, :-1]
    assert (pos[:, 1:][same] == pos[:, :-1][same] + 1).all() and (pos[:, 1:][~same] == 0).all()


def test_unshuffled_dataset_is_refused_and_shuffle_records(tmp_path):
    tok, doc = make(tmp_path)
    raw = tmp_path / "datasets" / "raw"
    write_token_dataset(raw, tok, doc, "tok", shuffle_seed=None)
    with pytest.raises(AssertionError):
        ShardServer(raw, 16, "unsegmented_tokens", seed=0)
    row_shuffle_dataset(raw, tmp_path / "datasets" / "shuf", seed=5)
    ds.assert_row_shuffled(tmp_path / "datasets" / "shuf")
    got = ShardServer(tmp_path / "datasets" / "shuf", 17, "unsegmented_tokens", seed=0)
    assert sum(s.n_rows for s in got.shards) == 300


def test_packed_rows_validation():
    with pytest.raises(AssertionError):
        PackedRows(np.zeros((2, 3), np.int32), np.array([[0, 2, 2], [0, 0, 0]], np.int32))
    PackedRows.from_unsegmented_sequences(np.ones((2, 3), np.int32)).validate_vocabulary(2)


def test_zipf_source_partition_and_law():
    src = ZipfTokenSource(1000, 64, 1.1, seed=0)
    whole = src.batch(3, 8).tokens
    parts = [src.batch(3, 8, r, 2).tokens for r in range(2)]
    assert (np.concatenate([p.numpy() for p in parts]) == whole.numpy()).all()
    big = src.rows(0, 0, 256, 256).ravel()
    counts = np.sort(np.bincount(big, minlength=1000))[::-1]
    assert counts[0] > 5 * counts[50]  # heavy head
