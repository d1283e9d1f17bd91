"""Expert-split training through the engine on CPU (gloo, 2 ranks on the mesh's tp axis): the same
config on a `tp = 2` mesh follows the single-process run step for step - losses, clipped updates of
replicated and split leaves - and writes checkpoints in the global layout that either run can resume."""
import copy
import os
import socket
import tempfile
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as ge
from param_decomp_b200.config.experiments import LMExperimentConfig
from param_decomp_b200.core.checkpoint import DECOMPOSITION_FILE, TRAINING_FILE

STEPS = 4
SPLIT_ID, SINGLE_ID = "p-0000aaaa", "p-0000bbbb"


def _cfg(tp: int, mode: str = "allreduce", n_experts: int = 5, k: int = 2, batch: int = 4) -> LMExperimentConfig:
    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"]["backend"] = "eager_torch"
    c["runtime"]["mesh"] = {"replicate": 1, "fsdp": 1, "tp": tp}
    c["runtime"]["sharding"] = "ddp"
    c["target"]["weights_dtype"] = "float32"
    c["target"]["attention_implementation"] = "xla"
    c["target"]["spec"]["arch"] = {"family": "moe", "n_layer": 2, "d_model": 32, "n_head": 2, "d_ff": 16,
                                   "vocab_size": 100, "n_experts": n_experts, "experts_per_token": k}  # 5 experts on 2 ranks: one dummy
    c["decomposition"]["sites"] = {"kind": "moe", "layers": {"kind": "all"},
                                   "cs": {"q": 8, "experts_gate": 20, "experts_up": 20, "experts_down": 20}}
    c["decomposition"]["ci"] = {"type": "layerwise_mlp", "hidden_dims": [16]}
    c["data"]["seq_len"] = 8
    c["pd"]["batch_size"] = batch
    c["pd"]["steps"] = STEPS
    c["cadence"] = {"train_log_every": 1, "checkpointing": {"kind": "periodic", "save_every": 2, "retention": {"kind": "keep_all"}}}
    c["eval"] = None
    if mode == "all_to_all":
        c["target"]["expert_implementation"] = "all_to_all"
    return LMExperimentConfig.model_validate(c)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _train(cfg, root: Path, run_id: str, max_steps=None):
    from param_decomp_b200.experiments.lm.training import train_lm

    states: list = []
    res = train_lm(cfg, root, run_id=run_id, device="cpu", max_steps_this_entry=max_steps, state_out=states)
    return res, states[0]


def _worker(rank: int, world: int, port: int, root: str, mode: str, out, n_experts: int = 5, k: int = 2, batch: int = 4):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    torch.manual_seed(0)
    res, state = _train(_cfg(world, mode, n_experts, k, batch), Path(root), SPLIT_ID)
    shard = state.expert_shard
    assert shard is not None and shard.world == world
    local = {n: p.detach().clone() for n, p in state.components.named_parameters()}
    out[rank] = (dict(res.last_metrics), local, shard.lo, shard.n_real,
                 {n: p.detach().clone() for n, p in state.ci_fn.named_parameters()})
    assert not dist.is_initialized()  # train_lm tears its own process group down


@pytest.mark.parametrize("mode,n_experts,k,world,batch", [("allreduce", 5, 2, 2, 4), ("all_to_all", 5, 2, 2, 4),
                                                         ("all_to_all", 4, 2, 3, 6), ("all_to_all", 2, 2, 3, 6), ("allreduce", 2, 2, 2, 4)])
def test_expert_split_engine_matches_single_process(mode, n_experts, k, world, batch):
    """`allreduce`: tokens replicated over the pair; `all_to_all`: each rank takes half of the batch and jobs
    travel to their expert's owner (`target.expert_implementation: all_to_all`). With four experts on three ranks (padded to six, two per rank) the
    last rank owns only padding experts and receives no job at all (42 experts on 8 ranks do the same to the
    last rank). Two experts on two or three ranks leave ONE expert per rank: the sites stay blocked (narrow CI,
    routed taps) although a rank's bank has a single block."""
    from safetensors import safe_open

    with tempfile.TemporaryDirectory() as root:
        port = _free_port()
        out = mp.Manager().dict()
        mp.spawn(_worker, args=(world, port, root, mode, out, n_experts, k, batch), nprocs=world, join=True)

        res, ref = _train(_cfg(1, "allreduce", n_experts, k, batch), Path(root), SINGLE_ID)
        ref_params = dict(ref.components.named_parameters())
        for k in ("loss/total", "loss/FaithfulnessLoss", "loss/StochasticReconLoss", "loss/ImportanceMinimalityLoss",
                  "grad_norms/summary/components", "grad_norms/summary/ci_fns"):
            got = sum(out[r][0]["train/" + k] for r in range(world)) / world  # (per-rank batch shards under all_to_all)
            want = res.last_metrics["train/" + k]
            assert abs(got - want) <= 2e-4 * abs(want) + 1e-7, (k, got, want)
            if mode == "allreduce":
                assert abs(out[0][0]["train/" + k] - out[1][0]["train/" + k]) <= 1e-5 * abs(want) + 1e-8
        for r in range(world):
            _, local, lo, n_real, ci_params = out[r]
            for name, p in local.items():
                g = ref_params[name].detach()
                if p.shape == g.shape:  # replicated leaf (dense site): identical on every rank
                    assert torch.allclose(p, g, atol=2e-6), name
                else:  # [sites, E_loc, ...]: this rank's experts; dummies untouched
                    assert torch.allclose(p[:, :n_real], g[:, lo:lo + n_real], atol=2e-6), name
                    assert float(p[:, n_real:].abs().sum()) == 0.0
            for name, p in ref.ci_fn.named_parameters():
                assert torch.allclose(ci_params[name], p.detach(), atol=2e-6), name

        # the split run's checkpoint holds global stacks, equal to the single-process file
        for item in (DECOMPOSITION_FILE, TRAINING_FILE):
            paths = sorted(Path(root).rglob(item))
            split_f = [p for p in paths if SPLIT_ID in str(p)][-1]
            single_f = Path(str(split_f).replace(SPLIT_ID, SINGLE_ID))
            with safe_open(str(split_f), framework="pt") as fs, safe_open(str(single_f), framework="pt") as f1:
                assert set(fs.keys()) == set(f1.keys())
                for k in fs.keys():
                    assert fs.get_tensor(k).shape == f1.get_tensor(k).shape, k
                    assert torch.allclose(fs.get_tensor(k), f1.get_tensor(k), atol=2e-6), k
