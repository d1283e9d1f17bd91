"""Data-parallel correctness on CPU (gloo, 2 ranks) against the single-process run of the same config:

* the ZeRO-style sharded optimizer after a faithfulness warm-up (the warm-up must not detach the parameters'
  gradients from the optimizer's flat buffer);
* adversary sources under data parallelism: batch-shared (`c`) sources - persistent and fresh - stay identical
  on every rank and follow the single-process trajectory, per-row (`bc`) sources are drawn at their global rows
  and a checkpoint stores them for the whole batch;
* the L_p minimality term uses the global-batch mean inside its logarithm.
"""
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

STEPS = 3


def _cfg(world: int, losses: list, sharding: str, warmup: int = 0, save: bool = False) -> LMExperimentConfig:
    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"]["backend"] = "eager_torch"
    c["runtime"]["mesh"] = {"replicate": 1, "fsdp": world, "tp": 1}
    c["runtime"]["sharding"] = sharding
    c["target"]["weights_dtype"] = "float32"
    c["target"]["attention_implementation"] = "xla"
    c["target"]["spec"]["arch"] = {"family": "glu_transformer", "n_layer": 2, "d_model": 32, "n_head": 2, "d_ff": 48,
                                   "vocab_size": 100}
    c["decomposition"]["sites"]["cs"] = {"q": 16, "o": 16, "gate": 24, "down": 16}
    c["decomposition"]["ci"] = {"type": "layerwise_mlp", "hidden_dims": [16]}
    c["data"]["seq_len"] = 8
    c["pd"]["batch_size"] = 4
    c["pd"]["steps"] = STEPS
    c["pd"]["loss_metrics"] = losses
    c["pd"]["faithfulness_warmup_steps"] = warmup
    c["pd"]["faithfulness_warmup_lr"] = 1e-2
    ck = ({"kind": "periodic", "save_every": STEPS, "retention": {"kind": "keep_all"}} if save else {"kind": "none"})
    c["cadence"] = {"train_log_every": 1, "checkpointing": ck}
    c["eval"] = None
    if save:  # an evaluation probe with batch-shared (`c`) sources at the last step
        c["eval"] = {"batch_size": 4, "n_steps": 1, "every": STEPS, "slow_every": STEPS,
                     "metrics": [{"type": "PGDReconLoss", "init": "random", "source_shape": "c", "n_steps": 3,
                                  "step_size": 0.1}]}
    return LMExperimentConfig.model_validate(c)


BASE = [{"type": "ImportanceMinimalityLoss", "coeff": 1e-3, "gamma": 1.0},
        {"type": "StochasticReconLoss", "coeff": 1.0},
        {"type": "FaithfulnessLoss", "coeff": 10.0}]


def _pgd_losses(shape: str) -> list:
    return [{"type": "ImportanceMinimalityLoss", "coeff": 1e-3, "gamma": 1.0},
            {"type": "PersistentPGDReconLoss", "coeff": 1.0, "source_shape": shape, "n_warmup_steps": 1,
             "optimizer": {"type": "sgd", "lr_schedule": 0.05}},
            {"type": "PGDReconLoss", "coeff": 0.5, "init": "random", "source_shape": shape, "n_steps": 2, "step_size": 0.1},
            {"type": "FaithfulnessLoss", "coeff": 10.0}]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _train(cfg, root, run_id):
    from param_decomp_b200.experiments.lm.training import train_lm

    states: list = []
    res = train_lm(cfg, Path(root) if root else None, run_id=run_id, device="cpu", state_out=states)
    st = states[0]
    return res, st


def _snapshot(res, st):
    if hasattr(st.components_opt, "refresh_full_fp32") and torch.distributed.is_initialized():
        st.components_opt.refresh_full_fp32()
    adv = {t: {k: v.detach().clone() for k, v in a._local_state().items()} for t, a in st.adversaries.items()}
    return (dict(res.last_metrics), [p.detach().clone() for p in st.components.parameters()], adv)


def _worker(rank: int, world: int, port: int, root: str, kind: str, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from param_decomp_b200.experiments.lm.training import train_lm

    if kind == "warmup":
        cfg = _cfg(world, BASE, "owner", warmup=2)
    elif kind == "muon":
        cfg = _muon_cfg(world)
    else:
        cfg = _cfg(world, _pgd_losses(kind), "ddp", save=True)
    states: list = []
    res = train_lm(cfg, Path(root), run_id="p-0000aaaa", device="cpu", state_out=states)
    st = states[0]
    if kind == "warmup":
        assert hasattr(st.components_opt, "gather_state"), "the config must select the sharded optimizer"
    if kind == "muon":
        from param_decomp_b200.parallel.sharded_muon import StackShardedMuon

        assert isinstance(st.components_opt, StackShardedMuon)
        mom = st.components_opt.state["V.q/mom"]
        assert mom.shape[0] * world == st.components.V["q"].shape[0]  # momentum of this rank's matrices only
    # the process group is gone after train_lm: the sharded masters were gathered by its final save / log step
    adv = {t: {k: v.detach().clone() for k, v in a._local_state().items()} for t, a in st.adversaries.items()}
    out[rank] = (dict(res.last_metrics), [p.detach().clone() for p in st.components.parameters()], adv)


def test_sharded_optimizer_trains_after_faithfulness_warmup():
    with tempfile.TemporaryDirectory() as root:
        out = mp.Manager().dict()
        mp.spawn(_worker, args=(2, _free_port(), root, "warmup", out), nprocs=2, join=True)
        res, st = _train(_cfg(1, BASE, "owner", warmup=2), root, "p-0000bbbb")
        ref_metrics, ref_params, _ = _snapshot(res, st)
        for r in range(2):
            metrics, params, _ = out[r]
            assert metrics["train/grad_norms/summary/components"] > 0.0
            assert metrics["train/loss/total"] == pytest.approx(ref_metrics["train/loss/total"], rel=1e-4)
            assert metrics["train/grad_norms/summary/components"] == pytest.approx(ref_metrics["train/grad_norms/summary/components"], rel=1e-3)


def _eval_value(root, run_id: str, key: str) -> float:
    import json

    lines = [json.loads(l) for l in (Path(root) / "runs" / run_id / "metrics.jsonl").read_text().splitlines()]
    vals = [l[key] for l in lines if key in l]
    assert vals, (key, sorted({k for l in lines for k in l}))
    return vals[-1]


@pytest.mark.parametrize("shape", ["bc"])
def test_adversary_sources_under_data_parallel(shape):
    from param_decomp_b200.core import checkpoint as ckpt

    with tempfile.TemporaryDirectory() as root:
        out = mp.Manager().dict()
        mp.spawn(_worker, args=(2, _free_port(), root, shape, out), nprocs=2, join=True)
        res, st = _train(_cfg(1, _pgd_losses(shape), "ddp", save=True), root, "p-0000cccc")
        ref_metrics, ref_params, ref_adv = _snapshot(res, st)
        # evaluation probe with batch-shared sources: the ranks ascend ONE source on the global-batch gradient
        assert _eval_value(root, "p-0000aaaa", "eval/loss/PGDReconLoss_3step") == pytest.approx(
            _eval_value(root, "p-0000cccc", "eval/loss/PGDReconLoss_3step"), rel=2e-3)  # sign steps amplify rounding
        (term,) = ref_adv.keys()
        for key, ref in ref_adv[term].items():
            a, b = out[0][2][term][key], out[1][2][term][key]
            if ref.shape[0] == 1:  # batch-shared: every rank holds the single-process source
                assert torch.equal(a, b), key
                assert torch.allclose(a, ref, atol=2e-5), (key, float((a - ref).abs().max()))
            else:  # per-row: each rank holds its rows of the single-process tensor
                assert torch.allclose(torch.cat([a, b]), ref, atol=2e-5), (key, float((torch.cat([a, b]) - ref).abs().max()))
        for r in range(2):
            assert out[r][0]["train/loss/total"] == pytest.approx(ref_metrics["train/loss/total"], rel=2e-4)
        # the checkpoint holds the sources of the global batch
        tensors, _ = ckpt._read(Path(root) / "runs" / "p-0000aaaa" / "ckpts" / str(STEPS) / ckpt.TRAINING_FILE)
        for key, ref in ref_adv[term].items():
            saved = tensors[f"adversaries/{term}/{key}"]
            assert saved.shape == ref.shape, (key, saved.shape, ref.shape)
            assert torch.allclose(saved.float(), ref.float(), atol=2e-5)
        # ... and a single process restores all of them, a 2-rank job its own rows
        st.adversaries[term].load_state_dict({k[len(f"adversaries/{term}/"):]: v for k, v in tensors.items()
                                              if k.startswith(f"adversaries/{term}/")}, 0, 1)
        half = copy.deepcopy(st.adversaries[term])
        for name in half.sources:
            if half.sources[name].shape[0] > 1:
                n = half.sources[name].shape[0] // 2
                half.sources[name], half.delta[name] = half.sources[name][:n], half.delta[name][:n]
        half.state = {}
        half.load_state_dict({k[len(f"adversaries/{term}/"):]: v for k, v in tensors.items()
                              if k.startswith(f"adversaries/{term}/")}, 1, 2)
        for name, v in half.sources.items():
            full = st.adversaries[term].sources[name]
            assert torch.equal(v, full if full.shape[0] == 1 else full[full.shape[0] // 2:])


def test_lp_minimality_uses_global_mean():
    from param_decomp_b200.core import losses

    torch.manual_seed(0)
    ci = {"s": torch.rand(8, 5)}
    whole = losses.lp_importance_minimality(ci, 0.9, 1e-6, 0.5)
    halves = [{"s": ci["s"][:4]}, {"s": ci["s"][4:]}]
    means = [(h["s"].float() + 1e-6).pow(0.9).mean(0) for h in halves]
    glob = (means[0] + means[1]) / 2
    got = losses.lp_importance_minimality(halves[0], 0.9, 1e-6, 0.5, world_size=2, mean_over_ranks=lambda m: glob)
    assert float(got) == pytest.approx(float(whole), rel=1e-6)


def _muon_cfg(world: int) -> LMExperimentConfig:
    c = _cfg(world, BASE, "owner", save=True).model_dump(mode="json")
    c["pd"]["components_optimizer"] = {"type": "muon", "lr_schedule": 1e-2, "ns_dtype": "float32", "grad_clip_norm": 1.0}
    c["eval"] = None
    return LMExperimentConfig.model_validate(c)


def test_muon_with_newton_schulz_split_over_ranks_matches_replicated_muon():
    """`sharding: owner` + Muon: each rank orthogonalises and keeps momentum for its slice of every stack; the run
    follows the single-process Muon run, and the checkpoint holds whole momenta."""
    from param_decomp_b200.core import checkpoint as ckpt

    with tempfile.TemporaryDirectory() as root:
        out = mp.Manager().dict()
        mp.spawn(_worker, args=(2, _free_port(), root, "muon", out), nprocs=2, join=True)
        res, st = _train(_muon_cfg(1), root, "p-0000dddd")
        ref_metrics, ref_params, _ = _snapshot(res, st)
        for r in range(2):
            metrics, params, _ = out[r]
            assert metrics["train/loss/total"] == pytest.approx(ref_metrics["train/loss/total"], rel=2e-4)
            for a, b in zip(params, ref_params):
                assert torch.allclose(a, b, atol=5e-5), float((a - b).abs().max())
        tensors, _ = ckpt._read(Path(root) / "runs" / "p-0000aaaa" / "ckpts" / str(STEPS) / ckpt.TRAINING_FILE)
        single, _ = ckpt._read(Path(root) / "runs" / "p-0000dddd" / "ckpts" / str(STEPS) / ckpt.TRAINING_FILE)
        key = "opt/components/V.q/mom"
        assert tensors[key].shape == single[key].shape and torch.allclose(tensors[key], single[key], atol=5e-5)


def _tms_cfg():
    import yaml

    from param_decomp_b200.config.experiments import TMSExperimentConfig

    root = Path(ge.__file__).resolve().parent
    raw = yaml.safe_load((root / "param_decomp_b200/experiments/configs/tms_5-2.yaml").read_text())
    raw["pd"].update({"steps": 5, "batch_size": 64, "faithfulness_warmup_steps": 0})
    raw["target"]["pretrain"]["steps"] = 10
    raw["cadence"] = {"train_log_every": 1, "checkpointing": {"kind": "none"}}
    raw["eval"] = None
    return TMSExperimentConfig.model_validate(raw)


def _tms_worker(rank: int, world: int, port: int, root: str, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from param_decomp_b200.experiments.tms.run import run_tms

    states: list = []
    res = run_tms(_tms_cfg(), Path(root), run_id="p-0000a7a5", state_out=states)
    out[rank] = (dict(res.last_metrics), [p.detach().clone() for p in states[0].components.parameters()])


def test_toy_root_runs_data_parallel_and_matches_single_process():
    """The TMS root under a 2-process launch (the form the 2-GPU toy benchmark uses): every rank takes its rows of
    the seeded global batch, gradients are averaged, and the run follows the single-process run."""
    from param_decomp_b200.experiments.tms.run import run_tms

    with tempfile.TemporaryDirectory() as root:
        out = mp.Manager().dict()
        mp.spawn(_tms_worker, args=(2, _free_port(), root, out), nprocs=2, join=True)
        states: list = []
        res = run_tms(_tms_cfg(), Path(root), run_id="p-0000a7a6", state_out=states)
        for r in range(2):
            metrics, params = out[r]
            assert metrics["train/loss/total"] == pytest.approx(res.last_metrics["train/loss/total"], rel=1e-4)
            for a, b in zip(params, states[0].components.parameters()):
                assert torch.allclose(a, b.detach(), atol=2e-5), float((a - b).abs().max())


def _odd_muon_cfg(world: int, steps: int = 4) -> LMExperimentConfig:
    """Three layers: every stack holds three matrices, padded to four under a two-rank Newton-Schulz split."""
    c = _muon_cfg(world).model_dump(mode="json")
    c["target"]["spec"]["arch"]["n_layer"] = 3
    c["pd"]["steps"] = steps
    c["cadence"] = {"train_log_every": 1, "checkpointing": {"kind": "periodic", "save_every": 2, "retention": {"kind": "keep_all"}}}
    c["eval"] = None
    return LMExperimentConfig.model_validate(c)


def _odd_muon_worker(rank: int, world: int, port: int, root: str, out, run_id: str = "p-0000b0b0", max_steps=3):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from param_decomp_b200.experiments.lm.training import train_lm

    states: list = []
    # (first entry: checkpoint at step 2, stopped after step 3)
    res = train_lm(_odd_muon_cfg(world), Path(root), run_id=run_id, device="cpu", max_steps_this_entry=max_steps, state_out=states)
    st = states[0]
    out[rank] = (st.components.V["q"].shape[0], st.step, res.last_metrics.get("train/loss/total"),
                 [p.detach()[:3].clone() for p in st.components.parameters()])


def test_padded_stacks_resume_on_another_layout():
    """Stacks of three matrices are padded to four when two ranks split the Newton-Schulz work; the checkpoint written
    by that layout holds the three real entries only, so a single process (no padding) resumes it and ends where an
    uninterrupted single-process run ends."""
    from param_decomp_b200.core import checkpoint as ckpt

    with tempfile.TemporaryDirectory() as root:
        out = mp.Manager().dict()
        mp.spawn(_odd_muon_worker, args=(2, _free_port(), root, out), nprocs=2, join=True)
        assert out[0][:2] == (4, 3) and out[1][:2] == (4, 3)  # padded to the group size while training
        tensors, _ = ckpt._read(Path(root) / "runs" / "p-0000b0b0" / "ckpts" / "2" / ckpt.TRAINING_FILE)
        assert tensors["opt/components/V.q/mom"].shape[0] == 3  # pads never reach the file
        # the same pinned config in a single process: every mesh axis collapses to 1, no padding
        res, st = _train(_odd_muon_cfg(2), root, "p-0000b0b0")  # resumes at step 2
        assert st.step == 4 and st.components.V["q"].shape[0] == 3
        ref_res, ref = _train(_odd_muon_cfg(1), root, "p-0000b0b1")
        assert res.last_metrics["train/loss/total"] == pytest.approx(ref_res.last_metrics["train/loss/total"], rel=3e-4)
        for a, b in zip(st.components.parameters(), ref.components.parameters()):
            assert torch.allclose(a, b, atol=1e-4), float((a - b).abs().max())
        # and the other way round: a single-process (unpadded) checkpoint resumed by the padded two-rank layout
        from param_decomp_b200.experiments.lm.training import train_lm

        train_lm(_odd_muon_cfg(2), Path(root), run_id="p-0000b0b2", device="cpu", max_steps_this_entry=3)
        out2 = mp.Manager().dict()
        mp.spawn(_odd_muon_worker, args=(2, _free_port(), root, out2, "p-0000b0b2", None), nprocs=2, join=True)
        for r in range(2):
            n_stack, step, loss, params = out2[r]
            assert (n_stack, step) == (4, 4)
            assert loss == pytest.approx(ref_res.last_metrics["train/loss/total"], rel=3e-4)
            for a, b in zip(params, ref.components.parameters()):
                assert torch.allclose(a, b.detach(), atol=1e-4), float((a - b).abs().max())
