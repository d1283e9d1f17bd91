"""Metric naming grammar, config / checkpoint migrations, canonical weight addressing."""
import json
import tempfile
from pathlib import Path

import pytest
import torch
import yaml

from param_decomp_b200.infra import metric_names as MN
from param_decomp_b200.infra import migrations as MG
from param_decomp_b200.infra.weight_addressing import address_of, align_sites


def test_weight_addresses_align_families():
    assert address_of("layers.3.self_attn.k_proj").label == "layer-03-02-attn-k"
    assert address_of("h.1.mlp.c_fc") == address_of("layers.1.mlp.up_proj")
    assert address_of("layers.0.mlp.experts_down").role == "experts.out"
    assert address_of("linear1").role == "mlp.in" and address_of("layers.2.mlp_out").role == "mlp.out"
    with pytest.raises(ValueError):
        address_of("embed.weight")
    pairs = align_sites(["h.0.mlp.c_fc", "h.0.attn.q_proj", "h.1.mlp.down_proj"],
                        ["layers.0.self_attn.q_proj", "layers.0.mlp.up_proj", "layers.1.mlp.down_proj", "layers.1.mlp.gate_proj"])
    assert pairs == [("h.0.attn.q_proj", "layers.0.self_attn.q_proj"), ("h.0.mlp.c_fc", "layers.0.mlp.up_proj"),
                     ("h.1.mlp.down_proj", "layers.1.mlp.down_proj")]


def test_grouped_names_and_collisions():
    k = MN.grouped_metric_key
    assert k("train/loss/StochasticReconLoss").path == "train-loss/stochastic-recon-loss"
    assert k("train/schedules/lr_components").path == "train-schedules/lr-components"
    assert k("train/perf/step_time_s").path == "train-performance/step-time-s"
    assert k("eval/l0/layers.2.self_attn.q_proj").path == "eval-ci-l0/layer-02-01-attn-q"
    assert k("eval/ce_unrecovered/rounded_masked").path == "eval-reconstruction-ce-unrecovered/rounded-masked"
    assert k("eval/SlowPGDReconLoss_640step").path == "eval-reconstruction-pgd/slow-pgdrecon-loss-00640-steps"
    assert k("eval/ci_mean/h.0.mlp.c_fc/n_dead").path == "eval-ci-mean-n-dead/layer-00-06-mlp-in"
    assert k("train/uv_norm_ratio['layers.0.mlp.up_proj']").path == "train-uv-norm-ratio/layer-00-06-mlp-in"
    with pytest.raises(ValueError):
        k("weird")
    names = MN.MetricNames("grouped")
    a = names.metric("eval/l0/h.0.mlp.c_fc")
    assert names.metric("eval/l0/h.0.mlp.c_fc") == a
    with pytest.raises(ValueError):
        names.metric("eval/l0/layers.0.mlp.up_proj")  # a different local key with the same canonical address
    assert MN.MetricNames("legacy").metric("anything/at all") == "anything/at all"
    MN.validate_resume_schema({"wandb": {"metric_schema": "v2"}}, "grouped")
    with pytest.raises(ValueError):
        MN.validate_resume_schema({}, "grouped")


def test_every_key_of_a_run_is_in_the_grammar():
    from param_decomp_b200.config.experiments import TMSExperimentConfig
    from param_decomp_b200.experiments.tms.run import run_tms

    root = Path(__file__).resolve().parents[1]
    raw = yaml.safe_load((root / "param_decomp_b200/experiments/configs/tms_5-2.yaml").read_text())
    raw["pd"].update({"steps": 2, "batch_size": 64, "faithfulness_warmup_steps": 0})
    raw["target"]["pretrain"]["steps"] = 10
    raw["cadence"] = {"train_log_every": 1, "checkpointing": {"kind": "none"}}
    cfg = TMSExperimentConfig.model_validate(raw)
    with tempfile.TemporaryDirectory() as d:
        res = run_tms(cfg, Path(d), run_id="p-00001234")
        keys = {k for l in (res.run_dir / "metrics.jsonl").read_text().splitlines() for k in json.loads(l) if k != "step"}
    names = MN.MetricNames("grouped")
    mapped = {names.metric(k) for k in keys}
    assert len(mapped) == len(keys) and all("/" in m for m in mapped)


def test_config_migrations_produce_loadable_configs():
    old_sched = {"start_val": 0.01, "fn_type": "cosine", "final_val_frac": 0.1, "warmup_pct": 0.05}
    new = MG.migrate_schedule(old_sched)
    assert new == {"max_val": 0.01, "points": [{"at": 0.0, "frac": 0.0}, {"at": 0.05, "frac": 1.0},
                                               {"at": 1.0, "frac": 0.1, "interp": "cosine"}]}
    raw = {"pd": {"ci_config": {"type": "layerwise_mlp", "hidden_dims": [8]},
                  "decomposition_targets": [{"module_pattern": "model.layers.18.mlp.gate_proj", "C": 64},
                                            {"module_pattern": "layers.19.mlp.gate_proj", "C": 64}],
                  "components_optimizer": {"lr_schedule": old_sched}},
           "data": {"train": {"name": "corpus"}}, "wandb": {"project": "p", "metric_schema": "v2"}}
    out = MG.migrate_raw(raw)
    assert out["decomposition"]["sites"] == {"kind": "glu_transformer", "layers": {"kind": "list", "indices": [18, 19]},
                                             "cs": {"gate": 64}}
    assert out["decomposition"]["ci"]["type"] == "layerwise_mlp" and "ci_config" not in out["pd"]
    assert out["pd"]["components_optimizer"]["lr_schedule"]["points"][-1]["interp"] == "cosine"
    assert out["data"]["layout"] == "documents" and out["wandb"]["metric_schema"] == "grouped"
    assert MG.migrate_raw(out) == out  # idempotent
    # a current config passes through unchanged, and `from_file` applies the migrations
    from param_decomp_b200.config.experiments import TMSExperimentConfig

    root = Path(__file__).resolve().parents[1]
    cur = yaml.safe_load((root / "param_decomp_b200/experiments/configs/tms_5-2.yaml").read_text())
    assert MG.migrate_raw(cur) == cur
    legacy = dict(cur)
    legacy["pd"] = dict(cur["pd"])
    legacy["pd"]["components_optimizer"] = {"lr_schedule": {"start_val": 1e-3, "fn_type": "constant"}}
    with tempfile.TemporaryDirectory() as d:
        p = Path(d) / "old.yaml"
        p.write_text(yaml.dump(legacy))
        cfg = TMSExperimentConfig.from_file(p)
    assert cfg.pd.components_optimizer.lr_schedule.max_val == pytest.approx(1e-3)


def test_ci_attention_checkpoint_migration():
    old = {"ci_fn/backbone.blocks.0.wq.weight": torch.ones(2, 2), "ci_fn/backbone.blocks.0.qk_norm_scales.1": torch.ones(2),
           "ci_fn/backbone.blocks.0.ffn.w1.weight": torch.zeros(1), "opt/ci_fn/backbone.blocks.0.wo.bias/mu": torch.zeros(2),
           "step": torch.tensor(3)}
    new = MG.migrate_ci_attention_keys(old)
    assert set(new) == {"ci_fn/backbone.blocks.0.attn.wq.weight", "ci_fn/backbone.blocks.0.attn.k_gain",
                        "ci_fn/backbone.blocks.0.ffn.w1.weight", "opt/ci_fn/backbone.blocks.0.attn.wo.bias/mu", "step"}
    assert MG.migrate_ci_attention_keys(new) == new
    with pytest.raises(AssertionError):
        MG.migrate_ci_attention_keys({**old, **new})
    from safetensors.torch import load_file, save_file

    with tempfile.TemporaryDirectory() as d:
        src, dst = Path(d) / "3", Path(d) / "3-new"
        src.mkdir()
        save_file({k: v.contiguous() for k, v in old.items()}, str(src / "decomposition.safetensors"), metadata={"format": "x"})
        MG.migrate_checkpoint_step(src, dst)
        assert set(load_file(str(dst / "decomposition.safetensors"))) == set(new)


def test_written_keys_use_the_reference_spellings():
    from param_decomp_b200.infra.reference_keys import reference_key, reference_keys

    pairs = {
        "train/loss/total": "train/loss/total",
        "train/loss/FaithfulnessLoss": "train/loss/FaithfulnessLoss",
        "train/grad_norm/components": "train/grad_norms/summary/components",
        "train/grad_norm/ci_fn": "train/grad_norms/summary/ci_fns",
        "train/grad_norm/total": "train/grad_norms/summary/total",
        "train/schedules/gamma": "train/schedules/gamma_imp",
        "train/schedules/lr_components": "train/schedules/lr/components",
        "train/schedules/lr_ci_fn": "train/schedules/lr/ci_fn",
        "train/perf/step_time_s": "train/perf/step_time_s",
        "eval/kl/ci_masked": "eval/ce_kl/kl_ci_masked",
        "eval/ce_difference/stoch_masked": "eval/ce_kl/ce_difference_stoch_masked",
        "eval/ce/target": "eval/ce_kl/ce_target",
        "eval/PGDReconLoss_20step": "eval/loss/PGDReconLoss_20step",
        "eval/SlowPGDReconLoss_640step/hidden_acts_reconstruction": "eval/loss/SlowPGDReconLoss_640step/hidden_acts_reconstruction",
        "eval/l0/0.0_layers.0.mlp.up_proj": "eval/l0/0.0_layers.0.mlp.up_proj",
        "eval/ArithmeticCIGrid/probe/kl/ci_masked": "eval/ArithmeticCIGrid/probe/ce_kl/kl_ci_masked",
        "train/nontarget/loss/ImportanceMinimalityLoss": "train/loss/nontarget/imp",
        "train/nontarget/loss/StochasticReconSubsetLoss": "train/loss/nontarget/StochasticReconSubsetLoss",
    }
    for ours, theirs in pairs.items():
        assert reference_key(ours) == theirs, ours
    assert set(reference_keys(dict.fromkeys(pairs, 1.0))) == set(pairs.values())
    from param_decomp_b200.infra.reference_keys import internal_key

    assert all(internal_key(theirs) == ours for ours, theirs in pairs.items())
    # the grouped names are derived from the internal keys, thresholded L0 keys included
    k = MN.grouped_metric_key
    assert k("eval/l0/0.1_layers.2.self_attn.q_proj").path == "eval-ci-l0-gt-0p1/layer-02-01-attn-q"


def test_sink_mirrors_the_written_keys_or_the_grouped_names(tmp_path, monkeypatch):
    """`legacy`: W&B receives what `metrics.jsonl` receives (the reference's spellings); `grouped`: the two-level
    names derived from the internal keys."""
    import sys
    import types

    from param_decomp_b200.config.run import WandbConfig
    from param_decomp_b200.core.metrics import MetricsSink

    logged: list[dict] = []
    fake = types.ModuleType("wandb")
    fake.init = lambda **kw: types.SimpleNamespace(log=lambda rec, step=None: logged.append(dict(rec)), finish=lambda: None)
    monkeypatch.setitem(sys.modules, "wandb", fake)
    monkeypatch.setenv("WANDB_MODE", "offline")
    record = {"loss/total": 2.5, "grad_norm/ci_fn": 0.5, "schedules/lr_components": 1e-3}
    for schema, want in (("legacy", {"train/loss/total", "train/grad_norms/summary/ci_fns", "train/schedules/lr/components"}),
                         ("grouped", {"train-loss/total", "train-grad-norm/ci-fn", "train-schedules/lr-components"})):
        logged.clear()
        run_dir = tmp_path / schema
        sink = MetricsSink.for_run(run_dir, 0, WandbConfig(project="p", metric_schema=schema), "r", {})
        written = sink.log(3, record)
        sink.close()
        assert set(written) == {"train/loss/total", "train/grad_norms/summary/ci_fns", "train/schedules/lr/components"}
        assert set(json.loads((run_dir / "metrics.jsonl").read_text())) == set(written) | {"step"}
        assert len(logged) == 1 and set(logged[0]) == want, logged
