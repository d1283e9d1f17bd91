"""Data-parallel LM training with the ZeRO-style sharded optimizer on CPU (gloo, 2 ranks): a run interrupted
after its checkpoint resumes to the same parameters as the uninterrupted run, and the checkpoint is readable
by a single process with the replicated optimizer (per-parameter moments, gathered masters)."""
import copy
import os
import socket
import tempfile
from pathlib import Path

import torch
import torch.multiprocessing as mp

import __graft_entry__ as ge
from param_decomp_b200.config.experiments import LMExperimentConfig

STEPS = 6
FULL_ID, PART_ID = "p-0000eeee", "p-0000ffff"


def _cfg(world: int) -> LMExperimentConfig:
    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"]["backend"] = "eager_torch"
    c["runtime"]["mesh"] = {"replicate": 1, "fsdp": world, "tp": 1}
    c["runtime"]["sharding"] = "owner"  # -> sharded AdamW over the data group (collective form on CPU)
    c["target"]["weights_dtype"] = "float32"
    c["target"]["attention_implementation"] = "xla"
    c["target"]["spec"]["arch"] = {"family": "glu_transformer", "n_layer": 2, "d_model": 32, "n_head": 2, "d_ff": 48,
                                   "vocab_size": 100}
    c["decomposition"]["sites"]["cs"] = {"q": 16, "o": 16, "gate": 24, "down": 16}
    c["decomposition"]["ci"] = {"type": "layerwise_mlp", "hidden_dims": [16]}
    c["data"]["seq_len"] = 8
    c["pd"]["batch_size"] = 4
    c["pd"]["steps"] = STEPS
    c["cadence"] = {"train_log_every": 1, "checkpointing": {"kind": "periodic", "save_every": 3, "retention": {"kind": "keep_all"}}}
    c["eval"] = None
    return LMExperimentConfig.model_validate(c)


def _free_ports(n: int) -> tuple:
    socks = [socket.socket() for _ in range(n)]
    try:
        for s in socks:
            s.bind(("127.0.0.1", 0))
        return tuple(s.getsockname()[1] for s in socks)  # distinct: all bound at the same time
    finally:
        for s in socks:
            s.close()


def _worker(rank: int, world: int, ports: tuple, root: str, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(ports[0]))
    from param_decomp_b200.experiments.lm.training import train_lm

    def run(run_id, max_steps=None):
        states: list = []
        train_lm(_cfg(world), Path(root), run_id=run_id, device="cpu", max_steps_this_entry=max_steps, state_out=states)
        st = states[0]
        if hasattr(st.components_opt, "refresh_full_fp32") and torch.distributed.is_initialized():
            st.components_opt.refresh_full_fp32()
        return st

    full = run(FULL_ID)
    os.environ["MASTER_PORT"] = str(ports[1])
    run(PART_ID, max_steps=4)  # saved at the top of step 3, stops after step 4 (steps 3.. are redone on re-entry)
    os.environ["MASTER_PORT"] = str(ports[2])
    resumed = run(PART_ID)
    assert hasattr(full.components_opt, "gather_state"), "the config must select the sharded optimizer"
    out[rank] = ([p.detach().clone() for p in full.components.parameters()],
                 [p.detach().clone() for p in resumed.components.parameters()], full.step, resumed.step)


def test_sharded_optimizer_resume_and_layout_independent_checkpoint():
    from param_decomp_b200.core import checkpoint as ckpt
    from param_decomp_b200.core.objective import build_objective
    from param_decomp_b200.core.run import init_train_state
    from param_decomp_b200.experiments.lm.build import build_lm_run

    with tempfile.TemporaryDirectory() as root:
        world, ports = 2, _free_ports(3)  # one rendezvous per training entry
        out = mp.Manager().dict()
        mp.spawn(_worker, args=(world, ports, root, out), nprocs=world, join=True)
        for r in range(world):
            full, resumed, s1, s2 = out[r]
            assert s1 == s2 == STEPS
            for a, b in zip(full, resumed):
                assert torch.allclose(a, b, atol=1e-6)
        # the two-rank sharded run follows the single-process run with the replicated optimizer
        from param_decomp_b200.experiments.lm.training import train_lm

        single: list = []
        train_lm(_cfg(1), Path(root), run_id="p-00001111", device="cpu", state_out=single)
        for a, b in zip(out[0][0], single[0].components.parameters()):
            assert torch.allclose(a, b.detach(), atol=2e-5), float((a - b).abs().max())
        # one process, replicated optimizer, reads the 2-rank checkpoint
        cfg = _cfg(1)
        run = build_lm_run(cfg, None, "cpu")
        obj = build_objective(cfg.pd)
        st = init_train_state(run.model, run.ci_fn, cfg.pd, obj, "cpu", cfg.pd.batch_size, cfg.data.seq_len)
        run_dir = Path(root) / "runs" / FULL_ID
        ckpt.restore_state(run_dir, STEPS, st)
        assert st.step == STEPS
        for a, b in zip(out[0][0], st.components.parameters()):
            assert torch.allclose(a, b.detach(), atol=1e-6)
        mus = [k for k in st.components_opt.state if k.endswith("/mu")]
        assert len(mus) == len(list(st.components.parameters())) and all(float(st.components_opt.state[k].abs().sum()) > 0 for k in mus)
