"""End-to-end engine behaviour on CPU: TMS decomposition, checkpoint/resume exactness, fine-tune,
preemption, metrics files, run-dir rules."""
import json
import signal
from pathlib import Path

import pytest
import torch
import yaml

from param_decomp_b200.config.experiments import ResidMLPExperimentConfig, TMSExperimentConfig
from param_decomp_b200.core import checkpoint as ckpt
from param_decomp_b200.core.metrics import pin_launch_config
from param_decomp_b200.experiments.tms.run import run_tms

CFG = Path(__file__).resolve().parents[1] / "param_decomp_b200" / "experiments" / "configs"


def small_tms(steps=30, **pd_over):
    raw = yaml.safe_load((CFG / "tms_5-2.yaml").read_text())
    raw["pd"].update({"steps": steps, "batch_size": 256, "faithfulness_warmup_steps": 5, **pd_over})
    raw["target"]["pretrain"].update({"steps": 50, "batch_size": 256})
    raw["cadence"] = {"train_log_every": 10, "checkpointing": {"kind": "periodic", "save_every": 10,
                                                                "retention": {"kind": "keep_last", "n": 2}}}
    raw["eval"].update({"batch_size": 64, "every": 10, "slow_every": 20})
    raw["eval"]["metrics"][1]["n_steps"] = 2
    return TMSExperimentConfig.model_validate(raw)


def test_tms_runs_and_writes_run_dir(tmp_path):
    res = run_tms(small_tms(), tmp_path, run_id="p-00000001")
    rd = tmp_path / "runs" / "p-00000001"
    assert res.final_step == 30 and (rd / "launch_config.yaml").exists()
    lines = [json.loads(l) for l in (rd / "metrics.jsonl").read_text().splitlines()]
    train = [l for l in lines if "train/loss/total" in l]
    assert {"train/loss/FaithfulnessLoss", "train/loss/StochasticReconLoss", "train/perf/step_time_s",
            "train/grad_norms/summary/components", "train/schedules/lr/components"} <= set(train[0])
    assert any("eval/l0/0.0_linear1" in l for l in lines) and any("eval/loss/PGDReconLoss_2step" in l for l in lines)
    assert ckpt.list_steps(rd) == [20, 30]  # keep_last 2
    assert train[-1]["train/loss/total"] < train[0]["train/loss/total"]


def test_resume_is_bit_exact(tmp_path):
    cfg = small_tms(steps=20, loss_metrics=[
        {"type": "ImportanceMinimalityLoss", "coeff": 1e-3, "gamma": 1.0,
         "frequency": {"coeff": 1e-3, "reference_datapoint_count": 256, "ema_halflife_steps": 5}},
        {"type": "PersistentPGDReconLoss", "coeff": 1.0, "source_shape": "bc", "n_warmup_steps": 1,
         "optimizer": {"type": "adam", "lr_schedule": 0.01}},
        {"type": "FaithfulnessLoss", "coeff": 1.0}])
    full: list = []
    run_tms(cfg, tmp_path / "a", run_id="p-0000000a", state_out=full)
    part: list = []
    run_tms(cfg, tmp_path / "b", run_id="p-0000000b", max_steps_this_entry=10, state_out=part)
    assert ckpt.latest_step(tmp_path / "b" / "runs" / "p-0000000b") is None or True
    # interrupted at step 10 without a checkpoint at 10? save_every=10 fires at the top of step 10
    resumed: list = []
    # second entry: first entry stopped after 10 steps; its step-10 checkpoint is written on re-entry
    st = part[0]
    ckpt.save_state(tmp_path / "b" / "runs" / "p-0000000b", st, 2)
    run_tms(cfg, tmp_path / "b", run_id="p-0000000b", state_out=resumed)
    a, b = full[0], resumed[0]
    assert a.step == b.step == 20
    for (n1, p1), (_, p2) in zip(a.components.named_parameters(), b.components.named_parameters()):
        assert torch.equal(p1, p2), n1
    for (n1, p1), (_, p2) in zip(a.ci_fn.named_parameters(), b.ci_fn.named_parameters()):
        assert torch.equal(p1, p2), n1
    k = next(iter(a.adversaries))
    assert torch.equal(a.adversaries[k].sources["linear1"], b.adversaries[k].sources["linear1"])


def test_changed_config_refuses_resume(tmp_path):
    pin_launch_config(tmp_path, "a: 1\n")
    pin_launch_config(tmp_path, "a: 1\n")
    with pytest.raises(AssertionError):
        pin_launch_config(tmp_path, "a: 2\n")


def test_finetune_loads_parent_decomposition_only(tmp_path):
    from param_decomp_b200.config.run import ResumeProvenance

    parent: list = []
    cfg = small_tms(steps=10)
    run_tms(cfg, tmp_path, run_id="p-000000aa", state_out=parent)
    from param_decomp_b200.core.run import run_decomposition_training
    from param_decomp_b200.experiments.toy_common import build_toy_ci_fn
    from param_decomp_b200.models.tms import TMSDecomposedModel, pretrain_tms

    params = pretrain_tms(cfg.target, 0.05, "at_least_zero_active")
    model = TMSDecomposedModel(params, {"linear1": 20, "linear2": 20})
    child: list = []
    prov = ResumeProvenance(parent_run_dir=tmp_path / "runs" / "p-000000aa", parent_step=10)
    pd0 = cfg.pd.model_copy(update={"faithfulness_warmup_steps": 0})
    run_decomposition_training(model, build_toy_ci_fn(cfg.decomposition.ci, model.sites, 0), pd0, cfg.cadence,
                               lambda s: torch.zeros(4, 5), resume_provenance=prov, max_steps_this_entry=0 or 1,
                               state_out=child)
    assert child[0].step == 1  # fresh schedule from step 0, one step taken
    assert child[0].components_opt.count == 1  # fresh optimizer state


def test_sigterm_saves_and_stops(tmp_path):
    cfg = small_tms(steps=1000)
    import threading, os, time

    def fire():
        time.sleep(4.0)
        os.kill(os.getpid(), signal.SIGTERM)

    threading.Thread(target=fire, daemon=True).start()
    res = run_tms(cfg, tmp_path, run_id="p-000000bb")
    assert res.stopped_by_sigterm and 0 < res.final_step < 1000
    assert ckpt.latest_step(tmp_path / "runs" / "p-000000bb") == res.final_step


def test_no_checkpoint_run_refuses_reentry(tmp_path):
    raw = small_tms(steps=3).model_dump(mode="json")
    raw["cadence"]["checkpointing"] = {"kind": "none"}
    cfg = TMSExperimentConfig.model_validate(raw)
    run_tms(cfg, tmp_path, run_id="p-000000cc")
    assert not (tmp_path / "runs" / "p-000000cc" / "ckpts").exists()
    with pytest.raises(AssertionError):
        run_tms(cfg, tmp_path, run_id="p-000000cc")


def test_resid_mlp_runs(tmp_path):
    from param_decomp_b200.experiments.resid_mlp.run import run_resid_mlp

    raw = yaml.safe_load((CFG / "resid_mlp_1l.yaml").read_text())
    raw["pd"].update({"steps": 6, "batch_size": 64, "faithfulness_warmup_steps": 2})
    raw["target"].update({"n_features": 10, "d_embed": 32, "d_mlp": 8})
    raw["target"]["pretrain"].update({"steps": 20, "batch_size": 64})
    raw["decomposition"]["sites"]["sites"] = [{"name": "layers.0.mlp_in", "C": 12}, {"name": "layers.0.mlp_out", "C": 12}]
    res = run_resid_mlp(ResidMLPExperimentConfig.model_validate(raw), tmp_path, run_id="p-000000dd")
    assert res.final_step == 6


def test_pretrain_cache_roundtrip_feeds_decomposition(tmp_path):
    """Pretrain a tiny LlamaSimpleMLP, then load it as a `pretrained` target by run path."""
    import torch

    from param_decomp_b200.config.experiments import PretrainedTarget
    from param_decomp_b200.models import loaders
    from param_decomp_b200.pretrain.train import PretrainConfig, pretrain

    cfg = PretrainConfig.model_validate({
        "run_name": "t", "global_batch": 4, "num_iterations": 4, "warmup_iters": 1, "learning_rate": 1e-3,
        "log_every": 2, "val_every": 2, "save_every": 2, "dtype": "float32",
        "model": {"vocab_size": 64, "n_layer": 2, "n_head": 2, "n_embd": 32, "n_intermediate": 64, "n_ctx": 16}})
    entry = pretrain(cfg, tmp_path, run_id="t-0000abcd", project="spd")
    assert (entry / "model_config.yaml").exists() and len(list(entry.glob("model_step_*.safetensors"))) == 1
    spec = PretrainedTarget(model_class="LlamaSimpleMLP", run_path="goodfire/spd/runs/t-0000abcd")
    arch, weights = loaders.load_from_spec(spec, tmp_path, torch.float32, "cpu")
    assert arch.family == "simple_mlp" and arch.n_layer == 2 and "h.0.attn.q_proj.weight" in weights


def test_nonlinearity_aligned_init_is_rank_one_slices_of_w():
    import torch

    from param_decomp_b200.config.experiments import TransformerArchConfig
    from param_decomp_b200.core.components import ComponentStacks
    from param_decomp_b200.core.init_aligned import nonlinearity_aligned_init
    from param_decomp_b200.models import transformer as tf

    arch = TransformerArchConfig(family="simple_mlp", n_layer=1, d_model=16, n_head=2, d_ff=32, vocab_size=20)
    w = tf.random_init_weights(arch, 0, torch.float32)
    name = tf.site_name("simple_mlp", 0, "c_fc")
    m = tf.TransformerDecomposedModel(arch, w, {name: 32})
    st = ComponentStacks(m.sites)
    nonlinearity_aligned_init(st, m, 0)
    # C == d_ff and every neuron covered once: the components sum to W exactly
    assert torch.allclose(st.weight(name), w[name + ".weight"], atol=1e-5)


def test_activation_recompute_changes_nothing_but_memory():
    """`runtime.remat_recon_forwards` / `remat_ci_fn`: every masked forward and the CI function are run again
    in the backward pass instead of keeping their activations; losses and gradients are the same."""
    import copy

    import torch

    import __graft_entry__ as ge
    from param_decomp_b200.config.experiments import LMExperimentConfig
    from param_decomp_b200.core.objective import build_objective
    from param_decomp_b200.core.run import init_train_state
    from param_decomp_b200.core.train import StepContext, train_step
    from param_decomp_b200.experiments.lm.build import build_lm_run

    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"]["backend"] = "eager_torch"
    c["target"]["weights_dtype"] = "float32"
    c["target"]["attention_implementation"] = "xla"
    c["target"]["spec"]["arch"] = {"family": "glu_transformer", "n_layer": 2, "d_model": 32, "n_head": 2, "d_ff": 48,
                                   "vocab_size": 100}
    c["decomposition"]["sites"]["cs"] = {"q": 16, "o": 16, "gate": 24, "down": 16}
    c["decomposition"]["ci"] = {"type": "layerwise_mlp", "hidden_dims": [16]}
    c["data"]["seq_len"] = 8
    cfg = LMExperimentConfig.model_validate(c)
    out = {}
    for remat in (False, True):
        run = build_lm_run(cfg, None, "cpu")
        obj = build_objective(cfg.pd)
        ctx = StepContext.build(run.model, obj, cfg.pd, remat_recon_forwards=remat, remat_ci_fn=remat)
        st = init_train_state(run.model, run.ci_fn, cfg.pd, obj, "cpu", cfg.pd.batch_size, cfg.data.seq_len)
        m = train_step(ctx, st, run.sample_train(0))
        out[remat] = ({k: float(v) for k, v in m.items() if k.startswith("loss/") or k.startswith("grad_norm/")},
                      [p.detach().clone() for p in st.components.parameters()],
                      [p.detach().clone() for p in st.ci_fn.parameters()])
    assert out[False][0] == pytest.approx(out[True][0], rel=1e-6)
    for a, b in zip(out[False][1] + out[False][2], out[True][1] + out[True][2]):
        assert torch.allclose(a, b, atol=1e-7)
