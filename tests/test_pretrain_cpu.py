"""The pretrainer's run mechanics on CPU: exact resume from the trainer state, retention of the newest
`keep_last` files, validation on the train rows when no held-out split is given, and two data-parallel
`gloo` ranks reproducing the one-process run."""
import os
import signal
import threading
import time

import torch
import torch.multiprocessing as mp
from safetensors.torch import load_file

from param_decomp_b200.models.loaders import latest_checkpoint
from param_decomp_b200.pretrain.train import PretrainConfig, pretrain


def _cfg(**over) -> PretrainConfig:
    raw = dict(run_name="tiny", seed=3, dtype="float32", attention_implementation="xla", global_batch=4,
               num_iterations=6, warmup_iters=2, learning_rate=1e-2, learning_rate_decay_frac=0.1, weight_decay=0.1,
               grad_clip=1.0, log_every=1, val_every=3, val_steps=3, save_every=2, keep_last=2,
               model=dict(model_type="LlamaSimpleMLP", n_layer=1, n_head=2, n_embd=16, n_intermediate=32,
                          vocab_size=61, n_ctx=8))
    raw.update(over)
    return PretrainConfig.model_validate(raw)


def _final(entry) -> dict:
    return load_file(str(latest_checkpoint(entry)))


def test_resume_is_exact_and_old_files_are_pruned(tmp_path):
    whole = pretrain(_cfg(), tmp_path / "a", run_id="t-00000001")
    part = pretrain(_cfg(), tmp_path / "b", run_id="t-00000001", max_iterations=4)
    assert sorted(p.name for p in (part / "ckpts").glob("state_step_*.pt")) == ["state_step_2.pt", "state_step_4.pt"]
    again = pretrain(_cfg(), tmp_path / "b", run_id="t-00000001")
    assert again == part
    a, b = _final(whole), _final(part)
    assert all(torch.equal(a[k], b[k]) for k in a), "a resumed run must land on the uninterrupted run's weights"
    assert sorted(p.name for p in (part / "ckpts").glob("state_step_*.pt")) == ["state_step_4.pt", "state_step_6.pt"]
    assert sorted(p.name for p in part.glob("model_step_*.safetensors")) == ["model_step_6.safetensors"]
    # a state file cut short by a kill is skipped for the one before it
    (part / "ckpts" / "state_step_6.pt").write_bytes(b"\x00" * 10)
    pretrain(_cfg(), tmp_path / "b", run_id="t-00000001")
    assert all(torch.equal(a[k], _final(part)[k]) for k in a)


def test_validation_without_a_held_out_split_reads_the_train_rows(tmp_path):
    entry = pretrain(_cfg(val_data=None, num_iterations=3), tmp_path, run_id="t-00000002")
    assert "\"val_loss\"" in (entry / "metrics.jsonl").read_text()


def test_sigterm_saves_state_at_the_next_iteration_boundary(tmp_path):
    cfg = _cfg(num_iterations=100000, save_every=100000, val_every=100000, log_every=1000)
    threading.Timer(3.0, lambda: os.kill(os.getpid(), signal.SIGTERM)).start()
    t0 = time.time()
    entry = pretrain(cfg, tmp_path, run_id="t-00000003")
    assert time.time() - t0 < 120
    states = list((entry / "ckpts").glob("state_step_*.pt"))
    assert len(states) == 1 and 0 < int(states[0].stem.split("_")[-1]) < 100000


def _dp_rank(rank: int, world: int, root: str, port: int) -> None:
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    pretrain(_cfg(dp=2), root, run_id="t-00000004")


def test_two_data_parallel_ranks_match_one_process(tmp_path):
    one = pretrain(_cfg(), tmp_path / "one", run_id="t-00000004")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_dp_rank, args=(2, str(tmp_path / "two"), port), nprocs=2, join=True)
    a = _final(one)
    b = _final(tmp_path / "two" / "pretrain_cache" / "spd-t-00000004")
    for k in a:
        torch.testing.assert_close(a[k], b[k], atol=2e-5, rtol=1e-4)
