import copy

import pytest
import torch

from param_decomp_b200.config.experiments import LMExperimentConfig
from param_decomp_b200.core.ci_fn.transformer import CIAttention, ComponentConditioning
from param_decomp_b200.experiments.lm.build import build_lm_run



def tiny(ci: dict, family="glu_transformer", cs=None) -> LMExperimentConfig:
    import __graft_entry__ as ge

    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["decomposition"]["ci"] = ci
    c["runtime"]["backend"] = "eager_torch"
    c["target"]["spec"]["arch"].update({"d_model": 64, "n_head": 2, "d_ff": 96, "vocab_size": 200, "n_layer": 4})
    c["decomposition"]["sites"]["cs"] = cs or {"q": 16, "o": 16, "gate": 24, "down": 24}
    c["data"]["seq_len"] = 16
    c["pd"]["batch_size"] = 2
    return LMExperimentConfig.model_validate(c)


ATT = {"kind": "mha", "n_heads": 2, "implementation": "xla", "mask": "causal"}


@pytest.mark.parametrize("ci", [
    {"type": "global_transformer", "d_model": 32, "n_blocks": 2, "attention": {**ATT, "qk_norm": "rms"},
     "ffn": {"kind": "gelu", "hidden": 48}, "input_tap": {"kind": "residual_boundaries", "offsets": [0, 2, 4]},
     "final_norm": "rms",
     "component_conditioning": {"kind": "affine_clipped_component_activation", "output_scale_init": 1.0,
                                "calibration": {"min_n_tokens": 8}}},
    {"type": "chunkwise_transformer", "d_model": 32, "n_blocks": 1, "blocks_per_chunk": 2,
     "attention": {"kind": "gqa", "n_heads": 4, "n_kv_heads": 2, "implementation": "xla", "mask": "bidirectional",
                   "sink": "learned", "logit_softcap": 30.0},
     "ffn": {"kind": "swiglu", "hidden": 48}, "input_tap": "all_block_taps"},
    {"type": "global_mlp", "hidden_dims": [24], "input_tap": "all_block_resids"},
])
def test_lm_ci_archs_emit_per_site_ci_and_train(ci):
    from param_decomp_b200.core.objective import build_objective
    from param_decomp_b200.core.run import init_train_state
    from param_decomp_b200.core.train import StepContext, train_step

    cfg = tiny(ci)
    run = build_lm_run(cfg, None, "cpu")
    obj = build_objective(cfg.pd)
    ctx = StepContext.build(run.model, obj, cfg.pd)
    st = init_train_state(run.model, run.ci_fn, cfg.pd, obj, "cpu", 2, 16)
    before = [p.detach().clone() for p in run.ci_fn.parameters()]
    m = train_step(ctx, st, run.sample_train(0))
    assert torch.isfinite(m["loss/total"])
    changed = sum(int(not torch.equal(a, b)) for a, b in zip(before, run.ci_fn.parameters()))
    assert changed > 0


def test_attention_is_confined_to_documents():
    torch.manual_seed(0)
    att = CIAttention(32, 2, None, "bidirectional", False, None, False, 10000.0, torch.Generator().manual_seed(0))
    x = torch.randn(1, 8, 32)
    seg = torch.tensor([[0, 0, 0, 0, 1, 1, 1, 1]])
    pos = torch.tensor([[0, 1, 2, 3, 0, 1, 2, 3]])
    y = att(x, pos, seg)
    x2 = x.clone()
    x2[:, 4:] = torch.randn(1, 4, 32)  # changing document 1 must not change document 0's output
    y2 = att(x2, pos, seg)
    assert torch.allclose(y[:, :4], y2[:, :4], atol=1e-6) and not torch.allclose(y[:, 4:], y2[:, 4:])


def test_component_conditioning_calibration():
    cc = ComponentConditioning({"s": 4}, 1.0)
    h = torch.arange(1, 1001, dtype=torch.float32)[:, None].repeat(1, 4) * torch.tensor([1.0, 2.0, 3.0, 4.0])
    cc.calibrate({"s": h})
    assert torch.allclose(cc.a_pos["s"], 1.0 / (999 * torch.tensor([1.0, 2.0, 3.0, 4.0])), rtol=1e-5)
    out = cc("s", h[:3])
    assert out.shape == (3, 4) and (out >= 0).all()
