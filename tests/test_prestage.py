"""Dataset production: packing with document boundaries, resumable per-file tokenization, the out-of-core row
shuffle with its multiset fingerprint, and the published dataset read back through the training loader."""
import json

import numpy as np
import pytest

from param_decomp_b200.data import prestage, row_shuffle
from param_decomp_b200.data.shards import ShardServer
from param_decomp_b200.formats import dataset_store as ds


def test_pack_documents_keeps_boundaries_and_drops_the_tail():
    rows = prestage.pack_documents([(1, 2, 3), (4,), (5, 6, 7, 8, 9)], max_length=4)
    assert rows.token_ids.tolist() == [[1, 2, 3, 4], [5, 6, 7, 8]]
    assert rows.document_ids.tolist() == [[0, 0, 0, 1], [2, 2, 2, 2]]
    assert prestage.pack_documents([(1, 2)], max_length=4).token_ids.shape == (0, 4)
    with pytest.raises(AssertionError):
        prestage.pack_documents([()], max_length=4)


def test_fingerprint_is_order_free_and_sensitive():
    rng = np.random.default_rng(0)
    tok = rng.integers(0, 1000, (64, 9)).astype(np.int32)
    doc = np.cumsum(rng.integers(0, 2, (64, 9)), axis=1).astype(np.int32)
    fp = row_shuffle.fingerprint(tok, doc)
    perm = rng.permutation(64)
    assert row_shuffle.fingerprint(tok[perm], doc[perm]) == fp
    assert row_shuffle.fingerprint(tok[:32], doc[:32]) + row_shuffle.fingerprint(tok[32:], doc[32:]) == fp
    swapped = tok.copy()
    swapped[0, [0, 1]] = swapped[0, [1, 0]]
    if swapped[0, 0] != swapped[0, 1]:
        assert row_shuffle.fingerprint(swapped, doc) != fp
    bumped = doc.copy()
    bumped[3] += 1
    assert row_shuffle.fingerprint(tok, bumped) != fp
    assert row_shuffle.fingerprint(tok[:, :0].reshape(0, 0)[:0].reshape(0, 9), doc[:0]) == row_shuffle.EMPTY


def _tiny_tokenizer(path):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    vocab = {c: i for i, c in enumerate("abcdefghijklmnopqrstuvwxyz ")}
    vocab.update({"[UNK]": 27, "<s>": 28, "</s>": 29})
    tok = Tokenizer(models.WordLevel(vocab, unk_token="[UNK]"))
    tok.pre_tokenizer = pre_tokenizers.Split("", "isolated")
    PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="[UNK]", bos_token="<s>", eos_token="</s>").save_pretrained(str(path))


def _write_sources(src):
    import pyarrow as pa
    import pyarrow.parquet as pq

    src.mkdir()
    rng = np.random.default_rng(1)
    words = ["alpha", "beta", "gamma", "delta", "epsilon", "zeta"]
    docs = [" ".join(rng.choice(words, size=int(rng.integers(1, 12)))) for _ in range(600)]
    pq.write_table(pa.table({"text": docs[:250], "other": list(range(250))}), src / "a.parquet")
    (src / "b.jsonl").write_text("".join(json.dumps({"text": d}) + "\n" for d in docs[250:450]) + json.dumps({"text": None}) + "\n")
    (src / "c.txt").write_text("\n".join(docs[450:]) + "\n")
    return docs


def test_tokenize_resume_finish_and_load(tmp_path):
    tok_dir, src, staging = tmp_path / "tok", tmp_path / "src", tmp_path / "staging"
    _tiny_tokenizer(tok_dir)
    docs = _write_sources(src)
    # two tasks split the three files; the second invocation of task 0 finds its shards and writes nothing
    first = prestage.tokenize(src, tok_dir, staging, seq_len=17, task=0, n_tasks=2, tokenizer_name="tiny-chars")
    assert [p.name for p in first] == ["shard_00000.parquet", "shard_00002.parquet"]
    assert prestage.tokenize(src, tok_dir, staging, seq_len=17, task=0, n_tasks=2, tokenizer_name="tiny-chars") == []
    with pytest.raises(AssertionError, match="2 of 3"):
        prestage.finish(staging, tmp_path / "early")
    prestage.tokenize(src, tok_dir, staging, seq_len=17, task=1, n_tasks=2, tokenizer_name="tiny-chars")
    assert not list(staging.glob("*.tmp"))

    tok0, doc0 = row_shuffle._read_shard(staging / "shard_00000.parquet")
    stream = [t for d in docs[:250] for t in (28, *[ord(c) - 97 if c != " " else 26 for c in d], 29)]
    assert tok0.reshape(-1).tolist() == stream[:tok0.size] and len(stream) - tok0.size < 17
    assert (doc0[:, 0] == 0).all() and ((np.diff(doc0, axis=1) == 0) | (np.diff(doc0, axis=1) == 1)).all()
    assert ((tok0 == 28).sum(axis=1) >= np.diff(doc0, axis=1).sum(axis=1)).all()  # every boundary starts with BOS

    before = row_shuffle.dataset_fingerprint(staging)
    out = tmp_path / "root" / "datasets" / "tiny"
    prestage.finish(staging, out, seed=5, producer_revision="abc123")
    assert row_shuffle.dataset_fingerprint(out) == before
    record = json.loads((out / ds.ROW_SHUFFLE_FILENAME).read_text())
    assert record["seed"] == 5 and record["fingerprint"]["rows"] == before.rows
    meta = ds.read_dataset_meta(out)
    assert (meta.seq_len, meta.tokenizer_name, meta.preprocessing_name, meta.end_of_document_token_id) == (
        17, "tiny-chars", "bos-eos-v1", 29)
    ds.assert_row_shuffled(out)
    # the rows are no longer in packing order, and the training loader serves them with document segments
    shuffled = np.concatenate([row_shuffle._read_shard(f)[0] for f in sorted(out.glob("*.parquet"))])
    packed = np.concatenate([row_shuffle._read_shard(f)[0] for f in sorted(staging.glob("*.parquet"))])
    assert shuffled.shape == packed.shape and not np.array_equal(shuffled, packed)
    server = ShardServer.open(ds.NamedDataset(name="tiny"), tmp_path / "root", 16, "documents", seed=0)
    batch = server.batch(0, 8)
    assert batch.tokens.shape == (8, 16) and batch.segment_ids is not None


def test_row_shuffle_is_seeded_and_uses_worker_processes(tmp_path):
    from param_decomp_b200.data.shards import write_token_dataset

    rng = np.random.default_rng(2)
    tok = rng.integers(0, 500, (3000, 12)).astype(np.int32)
    write_token_dataset(tmp_path / "src", tok, None, "t", rows_per_group=256, rows_per_shard=700, shuffle_seed=None)
    a = row_shuffle.row_shuffle(tmp_path / "src", tmp_path / "a", seed=1, n_buckets=5, workers=2, rows_per_group=128)
    row_shuffle.row_shuffle(tmp_path / "src", tmp_path / "b", seed=1, n_buckets=5)
    row_shuffle.row_shuffle(tmp_path / "src", tmp_path / "c", seed=2, n_buckets=5)
    rows = {k: np.concatenate([row_shuffle._read_shard(f)[0] for f in sorted((tmp_path / k).glob("*.parquet"))]) for k in "abc"}
    assert a.rows == 3000 and np.array_equal(rows["a"], rows["b"]) and not np.array_equal(rows["a"], rows["c"])
    assert sorted(map(tuple, rows["a"].tolist())) == sorted(map(tuple, tok.tolist()))
    # no row stays next to its packing-order neighbour more often than chance allows
    index = {tuple(r): i for i, r in enumerate(tok.tolist())}
    pos = np.array([index[tuple(r)] for r in rows["a"].tolist()])
    assert (np.abs(np.diff(pos)) == 1).mean() < 0.01
    assert not (tmp_path / "a" / ".row_shuffle_staging").exists()


def test_a_prestaged_dataset_trains_with_document_boundaries(tmp_path):
    """Text -> tokenize -> finish -> a decomposition run that reads the published dataset by name with
    `layout: documents`: attention and losses stay inside a document, and the prompt encoder finds the tokenizer
    the dataset names under `<data_root>/tokenizers/`."""
    import copy

    import __graft_entry__ as ge
    from param_decomp_b200.config.experiments import LMExperimentConfig
    from param_decomp_b200.experiments.lm.prompt_encoder import resolve_prompt_encoder
    from param_decomp_b200.experiments.lm.training import train_lm

    root = tmp_path / "root"
    tok_dir = root / "tokenizers" / "tiny-chars"
    tok_dir.mkdir(parents=True)
    _tiny_tokenizer(tok_dir)
    _write_sources(tmp_path / "src")
    prestage.tokenize(tmp_path / "src", tok_dir, tmp_path / "staging", seq_len=17, tokenizer_name="tiny-chars")
    prestage.finish(tmp_path / "staging", root / "datasets" / "tiny", seed=1)

    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"].update(backend="eager_torch", sharding="ddp")
    c["target"].update(weights_dtype="float32", attention_implementation="xla")
    c["target"]["spec"]["arch"] = {"family": "glu_transformer", "n_layer": 1, "d_model": 32, "n_head": 2, "d_ff": 48,
                                   "vocab_size": 30}
    c["decomposition"]["sites"]["cs"] = {"q": 8, "down": 8}
    c["decomposition"]["ci"] = {"type": "layerwise_mlp", "hidden_dims": [8]}
    c["data"] = {"train": {"kind": "name", "name": "tiny"}, "eval": {"kind": "name", "name": "tiny"},
                 "layout": "documents", "seq_len": 16}
    c["pd"].update(batch_size=4, steps=2)
    c["cadence"] = {"train_log_every": 1, "checkpointing": {"kind": "none"}}
    c["eval"] = None
    cfg = LMExperimentConfig.model_validate(c)
    res = train_lm(cfg, root, device="cpu")
    assert res.final_step == 2 and res.last_metrics["train/loss/total"] == res.last_metrics["train/loss/total"]
    enc = resolve_prompt_encoder(cfg.target.spec, cfg.data.train, root, 30)
    assert enc.source.endswith("tokenizers/tiny-chars") and enc("ab") == [0, 1]
