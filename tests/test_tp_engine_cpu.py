"""Component-split (tensor-parallel) training through the engine on CPU (gloo, 2 ranks on the mesh's tp
axis): every site's component axis is divided over the ranks; the run follows the single-process run
step for step and writes the same checkpoint files."""
import copy
import os
import socket
import tempfile
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

import __graft_entry__ as ge
from param_decomp_b200.config.experiments import LMExperimentConfig
from param_decomp_b200.core.checkpoint import DECOMPOSITION_FILE, TRAINING_FILE

STEPS = 4
SPLIT_ID, SINGLE_ID = "p-0000cccc", "p-0000dddd"


def _cfg(tp: int, losses: str, fsdp: int = 1, sp: bool = False) -> LMExperimentConfig:
    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"]["backend"] = "eager_torch"
    c["runtime"]["mesh"] = {"replicate": 1, "fsdp": fsdp, "tp": tp}
    c["runtime"]["sharding"] = "owner" if fsdp > 1 else "ddp"  # fsdp > 1: ZeRO-style sharded AdamW over the batch axes
    if sp:
        c["runtime"]["sequence_sharding"] = "sequence_parallel"
    c["target"]["weights_dtype"] = "float32"
    c["target"]["attention_implementation"] = "xla"
    c["target"]["spec"]["arch"] = {"family": "glu_transformer", "n_layer": 2, "d_model": 32, "n_head": 2, "d_ff": 48,
                                   "vocab_size": 100}
    c["decomposition"]["sites"] = {"kind": "glu_transformer", "layers": {"kind": "all"},
                                   "cs": {"q": 32, "o": 16, "gate": 48, "down": 32}}
    c["decomposition"]["ci"] = {"type": "layerwise_mlp", "hidden_dims": [16]}
    c["data"]["seq_len"] = 8
    c["pd"]["batch_size"] = 4
    c["pd"]["steps"] = STEPS
    if losses == "pgd":  # a persistent adversary: sources live on the whole sites, their gradients re-assemble
        c["pd"]["loss_metrics"] = [
            {"type": "ImportanceMinimalityLoss", "coeff": 1e-3, "gamma": 1.0},
            {"type": "PersistentPGDReconLoss", "coeff": 1.0, "source_shape": "bc", "n_warmup_steps": 1,
             "optimizer": {"type": "adam", "lr_schedule": 0.05}},
            {"type": "FaithfulnessLoss", "coeff": 10.0},
        ]
    c["cadence"] = {"train_log_every": 1, "checkpointing": {"kind": "periodic", "save_every": 2, "retention": {"kind": "keep_all"}}}
    c["eval"] = None
    if losses == "stochastic" and fsdp == 1:  # evaluations run on the split stacks too
        c["eval"] = {"batch_size": 4, "n_steps": 1, "every": 2, "slow_every": 4,
                     "metrics": [{"type": "CI_L0", "groups": None},
                                 {"type": "PGDReconLoss", "init": "random", "source_shape": "c", "n_steps": 2, "step_size": 0.1}]}
    return LMExperimentConfig.model_validate(c)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _train(cfg, root: Path, run_id: str):
    from param_decomp_b200.experiments.lm.training import train_lm

    states: list = []
    res = train_lm(cfg, root, run_id=run_id, device="cpu", state_out=states)
    return res, states[0]


def _worker(rank: int, world: int, port: int, root: str, losses: str, fsdp: int, out, sp: bool = False):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from param_decomp_b200.parallel import group_ops

    calls = {"n": 0}
    real_gather = group_ops.gather_sequence

    def counting_gather(x, group):
        calls["n"] += 1
        assert x.shape[1] * 2 == 8  # [B, T / 2, d] shards of the 8-token window
        return real_gather(x, group)

    group_ops.gather_sequence = counting_gather
    res, state = _train(_cfg(world // fsdp, losses, fsdp, sp), Path(root), SPLIT_ID)
    group_ops.gather_sequence = real_gather
    assert (calls["n"] > 0) == sp, calls
    assert state.expert_shard is not None and state.expert_shard.by_component
    if hasattr(state.components_opt, "gather_state"):
        assert fsdp > 1
    else:
        assert fsdp == 1
    out[rank] = (dict(res.last_metrics), {n: p.detach().clone() for n, p in state.components.named_parameters()},
                 {n: p.detach().clone() for n, p in state.ci_fn.named_parameters()})


@pytest.mark.parametrize("losses,fsdp,sp", [("stochastic", 1, False), ("pgd", 1, False), ("stochastic", 2, False),
                                            ("stochastic", 1, True), ("pgd", 1, True)])
def test_component_split_engine_matches_single_process(losses, fsdp, sp):
    """`fsdp = 2`: a 2 x 2 mesh - the batch over two data shards with the sharded optimizer, the components over
    two tp ranks. `sp`: `runtime.sequence_sharding: sequence_parallel` - masked passes carry the residual stream
    position-sharded over the tp pair between blocks; nothing in the results may change."""
    from safetensors import safe_open

    with tempfile.TemporaryDirectory() as root:
        tp = 2
        world, port = tp * fsdp, _free_port()
        out = mp.Manager().dict()
        mp.spawn(_worker, args=(world, port, root, losses, fsdp, out, sp), nprocs=world, join=True)
        res, ref = _train(_cfg(1, losses), Path(root), SINGLE_ID)
        keys = [k for k in res.last_metrics if k.startswith("train/loss/") or k.startswith("train/grad_norms/")]
        assert len(keys) >= 4
        for k in keys:
            got = sum(out[r][0][k] for r in range(world)) / world  # (data shards see their own rows)
            want = res.last_metrics[k]
            assert abs(got - want) <= 3e-4 * abs(want) + 1e-7, (k, got, want)
        ref_params = dict(ref.components.named_parameters())
        for r in range(world):
            _, local, ci_params = out[r]
            for name, p in local.items():
                g = ref_params[name].detach()
                ax = -1 if name.startswith("V") else -2
                w = g.shape[ax] // tp
                assert torch.allclose(p, g.narrow(ax, (r % tp) * w, w), atol=3e-6), name
            for name, p in ref.ci_fn.named_parameters():
                assert torch.allclose(ci_params[name], p.detach(), atol=3e-6), name
        if losses == "stochastic" and fsdp == 1:
            import json

            def last_eval(run_id):
                path = next(p for p in Path(root).rglob("metrics.jsonl") if run_id in str(p))
                rows = [json.loads(x) for x in path.read_text().splitlines()]
                return [{k: v for k, v in r.items() if k.startswith("eval/")} for r in rows if any(k.startswith("eval/") for k in r)][-1]

            a, b = last_eval(SPLIT_ID), last_eval(SINGLE_ID)
            assert set(a) == set(b) and any(k.startswith("eval/l0/") for k in a) and "eval/loss/PGDReconLoss_2step" in a
            for k in a:
                assert abs(a[k] - b[k]) <= 1e-3 * abs(b[k]) + 1e-6, (k, a[k], b[k])
        for item in (DECOMPOSITION_FILE, TRAINING_FILE):
            split_f = [p for p in sorted(Path(root).rglob(item)) if SPLIT_ID in str(p)][-1]
            single_f = Path(str(split_f).replace(SPLIT_ID, SINGLE_ID))
            with safe_open(str(split_f), framework="pt") as fs, safe_open(str(single_f), framework="pt") as f1:
                assert set(fs.keys()) == set(f1.keys())
                for k in fs.keys():
                    assert fs.get_tensor(k).shape == f1.get_tensor(k).shape, k
                    a, b = fs.get_tensor(k).float(), f1.get_tensor(k).float()
                    if k.startswith("adversaries/") or k.startswith("opt/"):
                        # sign-like Adam steps amplify rounding noise where a gradient is ~0: compare in the mean
                        assert float((a - b).abs().mean()) <= 1e-3 * (float(b.abs().mean()) + 1e-3), k
                    else:
                        assert torch.allclose(a, b, atol=3e-6), k


def _resume_worker(rank: int, world: int, ports: tuple, root: str, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(ports[0]))
    from param_decomp_b200.experiments.lm.training import train_lm

    def run(run_id, max_steps=None):
        states: list = []
        train_lm(_cfg(world, "pgd"), Path(root), run_id=run_id, device="cpu", max_steps_this_entry=max_steps, state_out=states)
        return states[0]

    full = run("p-0000aaa1")
    os.environ["MASTER_PORT"] = str(ports[1])
    run("p-0000aaa2", max_steps=3)  # checkpoint at step 2, stopped after step 3
    os.environ["MASTER_PORT"] = str(ports[2])
    resumed = run("p-0000aaa2")
    same = all(torch.allclose(a, b, atol=1e-6) for a, b in zip(list(full.components.parameters()) + list(full.ci_fn.parameters()),
                                                                list(resumed.components.parameters()) + list(resumed.ci_fn.parameters())))
    out[rank] = (same, full.step, resumed.step)


def test_component_split_run_resumes_from_its_global_checkpoint():
    """A tp-split run (persistent adversary included) interrupted after its checkpoint reaches the same
    parameters as the uninterrupted one: the global-layout file is cut back to each rank's slice."""
    from test_sharded_resume_cpu import _free_ports

    with tempfile.TemporaryDirectory() as root:
        out = mp.Manager().dict()
        mp.spawn(_resume_worker, args=(2, _free_ports(3), root, out), nprocs=2, join=True)
        assert all(v == (True, STEPS, STEPS) for v in out.values()), dict(out)
