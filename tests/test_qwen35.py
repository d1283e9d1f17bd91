"""Qwen3.5-style hybrid target: delta-rule forms agree, the model steps through the engine."""
import math

import torch

from param_decomp_b200.config.experiments import LMExperimentConfig
from param_decomp_b200.core.objective import build_objective
from param_decomp_b200.core.run import init_train_state
from param_decomp_b200.core.train import StepContext, train_step
from param_decomp_b200.experiments.lm.build import build_lm_run
from param_decomp_b200.models import ports, qwen35

ARCH = dict(family="qwen35_moe", n_layer=4, d_model=32, n_head=4, n_kv_head=2, head_dim=16, d_ff=16, vocab_size=101,
            max_seq_len=24, n_experts=6, experts_per_token=2, full_attention_interval=2, partial_rotary_factor=0.5,
            linear_num_key_heads=2, linear_key_head_dim=8, linear_num_value_heads=4, linear_value_head_dim=8,
            linear_conv_kernel_dim=4, shared_expert_intermediate=24)


def _config(cs: dict) -> LMExperimentConfig:
    base = LMExperimentConfig.from_file("param_decomp_b200/experiments/configs/lm_moe4l_e42.yaml")
    raw = base.model_dump(mode="json")
    raw["target"]["spec"]["arch"] = ARCH
    raw["target"]["weights_dtype"] = "float32"
    raw["target"]["attention_implementation"] = "xla"
    raw["decomposition"]["sites"] = {"kind": "qwen36_moe", "layers": {"kind": "all"}, "cs": cs}
    raw["decomposition"]["ci"] = {"type": "layerwise_mlp", "hidden_dims": [16]}
    raw["data"]["seq_len"] = 24
    raw["pd"]["batch_size"] = 4
    raw["runtime"]["backend"] = "eager_torch"
    return LMExperimentConfig.model_validate(raw)


def test_delta_rule_forms_agree_and_are_causal():
    torch.manual_seed(0)
    B, T, H, dk, dv = 2, 150, 3, 16, 24
    q, k, v = torch.randn(B, T, H, dk), torch.randn(B, T, H, dk), torch.randn(B, T, H, dv)
    g, beta = -torch.rand(B, T, H) * 2, torch.rand(B, T, H)
    a = ports.gated_delta_rule(q, k, v, g, beta, "sequential")
    b = ports.gated_delta_rule(q, k, v, g, beta, "chunkwise")
    assert torch.allclose(a, b, atol=1e-5)
    v2 = v.clone()
    v2[:, 100:] += 1.0  # the future does not reach the past
    c = ports.gated_delta_rule(q, k, v2, g, beta, "chunkwise")
    assert torch.allclose(c[:, :100], b[:, :100], atol=1e-6) and not torch.allclose(c[:, 100:], b[:, 100:])


def test_site_grammar():
    cfg = _config({"gdn_q": 8, "attn_o": 8, "experts_down": 12, "shared_up": 8})
    run = build_lm_run(cfg, None, "cpu")
    names = [s.name for s in run.model.sites]
    assert "layers.0.linear_attn.in_proj_qkv.q" in names and "layers.1.linear_attn.in_proj_qkv.q" not in names
    assert "layers.1.self_attn.o_proj" in names and "layers.0.self_attn.o_proj" not in names
    blocked = [s for s in run.model.sites if s.blocked]
    assert len(blocked) == 4 and all(s.n_blocks == 6 and s.C_block == 2 for s in blocked)
    assert qwen35.site_dims(cfg.target.spec.arch, "attn_q") == (32, 2 * 4 * 16)


def test_hybrid_model_trains_on_cpu():
    cs = {k: (12 if k.startswith("experts_") else 8) for k in qwen35.KIND_ORDER}
    cfg = _config(cs)
    run = build_lm_run(cfg, None, "cpu")
    assert len(run.model.sites) == 2 * 7 + 2 * 4 + 4 * 6
    obj = build_objective(cfg.pd)
    ctx = StepContext.build(run.model, obj, cfg.pd, lazy_masks=True)
    state = init_train_state(run.model, run.ci_fn, cfg.pd, obj, torch.device("cpu"), 4, 24)
    losses = []
    for s in range(3):
        m = train_step(ctx, state, run.sample_train(s))
        losses.append(float(m["loss/total"]))
    assert all(l == l and l < float("inf") for l in losses)
    # masked pass with every mask at one and no delta reproduces ... the component model, which at
    # init differs from the target; the clean pass must be reproducible and pinned routing reused
    batch = run.sample_train(0)
    a = run.model.clean_forward(batch)
    b = run.model.clean_forward(batch)
    assert torch.equal(a.output, b.output) and set(a.aux["routing"]) == {0, 1, 2, 3}


def test_pretrained_hybrid_target_roundtrip(tmp_path):
    """Pretrain a tiny hybrid model for a few iterations, then decompose it as a `pretrained_qwen35_moe` target
    resolved by run path through the pretrain cache."""
    from param_decomp_b200.pretrain.train import PretrainConfig, pretrain

    pcfg = PretrainConfig.model_validate({
        "run_name": "t", "global_batch": 4, "num_iterations": 3, "warmup_iters": 1, "learning_rate": 1e-3,
        "log_every": 1, "val_every": 3, "save_every": 3, "dtype": "float32",
        "model": {"model_type": "Qwen35Moe", "vocab_size": 101, "n_layer": 4, "n_head": 4, "n_embd": 32,
                  "n_intermediate": 16, "n_ctx": 24, "hybrid": ARCH}})
    entry = pretrain(pcfg, tmp_path, run_id="t-0000beef", project="spd")
    assert (entry / "model_config.yaml").exists() and len(list(entry.glob("model_step_*.safetensors"))) == 1
    import json

    lines = [json.loads(x) for x in (entry / "metrics.jsonl").read_text().splitlines()]
    losses = [r["train_loss"] for r in lines if "train_loss" in r]
    assert len(losses) == 3 and all(math.isfinite(v) for v in losses)

    cfg = _config({"gdn_q": 8, "attn_o": 8, "experts_down": 12, "shared_up": 8})
    raw = cfg.model_dump(mode="json")
    raw["target"]["spec"] = {"kind": "pretrained_qwen35_moe", "run_path": "goodfire/spd/runs/t-0000beef"}
    cfg = LMExperimentConfig.model_validate(raw)
    run = build_lm_run(cfg, tmp_path, "cpu")
    assert run.arch.family == "qwen35_moe" and run.arch.n_experts == 6
    obj = build_objective(cfg.pd)
    ctx = StepContext.build(run.model, obj, cfg.pd)
    st = init_train_state(run.model, run.ci_fn, cfg.pd, obj, "cpu", cfg.pd.batch_size, cfg.data.seq_len)
    m = train_step(ctx, st, run.sample_train(0))
    assert math.isfinite(float(m["loss/total"]))
