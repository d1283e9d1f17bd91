"""Failure detection and recovery, with every failure made on the host (no device is faulted, trapped or hung):
a stalled step seen by the watchdog thread, a SIGTERM that reaches one rank of two, a checkpoint damaged on disk,
a checkpoint directory left half-written."""
import copy
import os
import signal
import socket
import subprocess
import sys
import tempfile
import textwrap
import time
from pathlib import Path

import torch
import torch.multiprocessing as mp

import __graft_entry__ as ge
from param_decomp_b200.config.experiments import LMExperimentConfig
from param_decomp_b200.core import checkpoint as ckpt


def _cfg(steps: int = 6, world: int = 1, watchdog: float | None = None, save_every: int = 2) -> LMExperimentConfig:
    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"]["backend"] = "eager_torch"
    c["runtime"]["mesh"] = {"replicate": 1, "fsdp": world, "tp": 1}
    c["runtime"]["sharding"] = "ddp"
    if watchdog is not None:
        c["runtime"]["step_watchdog_s"] = watchdog
    c["target"]["weights_dtype"] = "float32"
    c["target"]["attention_implementation"] = "xla"
    c["data"]["seq_len"] = 8
    c["pd"]["batch_size"] = 4
    c["pd"]["steps"] = steps
    c["cadence"] = {"train_log_every": 1, "checkpointing": {"kind": "periodic", "save_every": save_every,
                                                            "retention": {"kind": "keep_all"}}}
    c["eval"] = None
    return LMExperimentConfig.model_validate(c)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_watchdog_turns_a_stalled_step_into_a_saved_exit(tmp_path, monkeypatch):
    """The data source hangs for longer than the limit on one step: the watchdog marks the run preempted, the loop
    saves and leaves at its next boundary, and the run resumes from there."""
    from param_decomp_b200.experiments.lm import build as build_mod
    from param_decomp_b200.experiments.lm.training import train_lm

    real_build = build_mod.build_lm_run

    def slow_build(*a, **k):
        run = real_build(*a, **k)
        sample = run.sample_train

        def stalling(step: int):
            if step == 2:
                time.sleep(4.5)  # a stall on the host (between one and two limits); nothing is waiting on a device
            return sample(step)

        return run.__class__(**{**run.__dict__, "sample_train": stalling}) if hasattr(run, "__dict__") else run

    monkeypatch.setattr("param_decomp_b200.experiments.lm.training.build_lm_run", slow_build)
    res = train_lm(_cfg(steps=50, watchdog=3.0, save_every=100), tmp_path, run_id="p-0000f001", device="cpu")
    assert res.stopped_by_sigterm and res.final_step == 3  # the stalled step completed, then the run left
    assert ckpt.latest_step(tmp_path / "runs" / "p-0000f001") == 3
    monkeypatch.setattr("param_decomp_b200.experiments.lm.training.build_lm_run", real_build)
    again = train_lm(_cfg(steps=50, watchdog=3.0, save_every=100), tmp_path, run_id="p-0000f001", device="cpu",
                     max_steps_this_entry=1)
    assert again.final_step == 4


def test_watchdog_second_stage_leaves_the_process(tmp_path):
    """A loop that never comes back to a boundary: after the second limit the process exits with the watchdog's
    code (run in a child: the exit is `os._exit`)."""
    code = textwrap.dedent("""
        import sys, time
        sys.path.insert(0, %r)
        from param_decomp_b200.core.run import StepWatchdog
        fired = []
        w = StepWatchdog(0.4, on_stall=lambda: fired.append(1)).start()
        time.sleep(5)      # never beats
        sys.exit(0)        # not reached
    """ % str(Path(ge.__file__).resolve().parent))
    t0 = time.monotonic()
    p = subprocess.run([sys.executable, "-c", code], timeout=120)
    assert p.returncode == 75 and time.monotonic() - t0 < 60


def _sigterm_worker(rank: int, world: int, port: int, root: str, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    import threading

    from param_decomp_b200.experiments.lm.training import train_lm

    if rank == 1:  # the signal reaches ONE rank only
        threading.Thread(target=lambda: (time.sleep(6.0), os.kill(os.getpid(), signal.SIGTERM)), daemon=True).start()
    res = train_lm(_cfg(steps=100000, world=world, save_every=10**6), Path(root), run_id="p-0000f002", device="cpu")
    out[rank] = (res.stopped_by_sigterm, res.final_step)


def test_sigterm_on_one_rank_stops_every_rank_at_the_same_step():
    with tempfile.TemporaryDirectory() as root:
        out = mp.Manager().dict()
        mp.spawn(_sigterm_worker, args=(2, _free_port(), root, out), nprocs=2, join=True)
        assert out[0][0] and out[1][0] and out[0][1] == out[1][1] and 0 < out[0][1] < 100000
        assert ckpt.latest_step(Path(root) / "runs" / "p-0000f002") == out[0][1]


def test_damaged_and_half_written_checkpoints_are_skipped(tmp_path):
    from param_decomp_b200.experiments.lm.training import train_lm

    train_lm(_cfg(steps=6), tmp_path, run_id="p-0000f003", device="cpu", max_steps_this_entry=5)
    run_dir = tmp_path / "runs" / "p-0000f003"
    assert ckpt.list_steps(run_dir) == [2, 4]
    # a directory whose write never finished (no rename) is not a checkpoint
    (ckpt.ckpt_root(run_dir) / "6.tmp").mkdir()
    assert ckpt.list_steps(run_dir) == [2, 4]
    # the newest checkpoint is truncated on disk (a copy that was cut short)
    f = ckpt.ckpt_root(run_dir) / "4" / ckpt.TRAINING_FILE
    data = f.read_bytes()
    f.write_bytes(data[: len(data) // 2])
    assert not ckpt.is_readable(run_dir, 4) and ckpt.is_readable(run_dir, 2)
    assert ckpt.latest_readable_step(run_dir) == 2
    states: list = []
    res = train_lm(_cfg(steps=6), tmp_path, run_id="p-0000f003", device="cpu", max_steps_this_entry=1, state_out=states)
    assert res.final_step == 3  # resumed from step 2, not from the damaged step 4


def _dying_rank_worker(rank: int, world: int, port: int, root: str, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from param_decomp_b200.experiments.lm import training
    from param_decomp_b200.experiments.lm.training import train_lm

    real_build = training.build_lm_run

    def build(*a, **k):
        run = real_build(*a, **k)
        sample = run.sample_train

        def failing(step: int):
            if rank == 1 and step == 3:
                raise RuntimeError("the data source of rank 1 failed")  # between two steps, nothing in flight
            return sample(step)

        return run.__class__(**{**run.__dict__, "sample_train": failing})

    training.build_lm_run = build
    t0 = time.monotonic()
    try:
        train_lm(_cfg(steps=1000, world=world, save_every=10**6), Path(root), run_id="p-0000f004", device="cpu")
        out[rank] = ("finished", time.monotonic() - t0)
    except BaseException as e:  # noqa: BLE001
        out[rank] = (type(e).__name__ + ": " + str(e)[:80], time.monotonic() - t0)


def test_a_rank_that_raises_between_steps_ends_the_others_quickly():
    """Rank 1's data source raises before step 3. It leaves without waiting at a barrier; rank 0 learns of it at
    its next host-side consensus (the peer's connection is gone) and ends with an error within seconds, not after
    the process group's ten-minute timeout."""
    with tempfile.TemporaryDirectory() as root:
        out = mp.Manager().dict()
        ctx = mp.get_context("spawn")
        port = _free_port()
        procs = [ctx.Process(target=_dying_rank_worker, args=(r, 2, port, root, out)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=240)
        alive = [p.is_alive() for p in procs]
        for p in procs:
            if p.is_alive():
                p.terminate()
        assert not any(alive), "a rank was still waiting for its dead peer"
        assert out[1][0].startswith("RuntimeError: the data source of rank 1 failed")
        assert out[0][0] != "finished" and out[0][1] < 120, out[0]
