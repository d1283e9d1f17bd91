"""The hybrid target against the HuggingFace implementations it is loaded from: a tiny random
Qwen3.5-MoE (fused `in_proj_qkv`) and Qwen3-Next (`in_proj_qkvz` grouped per key head) model is
written as a snapshot, read through the loader, and must give the same logits."""
import json

import pytest
import torch

from param_decomp_b200.config.experiments import HFTarget, PretrainedQwen35MoeTarget
from param_decomp_b200.models import loaders, qwen35
from param_decomp_b200.models.transformer import LMBatch

transformers = pytest.importorskip("transformers")

TINY = dict(vocab_size=101, hidden_size=32, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
            moe_intermediate_size=16, shared_expert_intermediate_size=24, num_experts=6, num_experts_per_tok=2,
            linear_num_key_heads=2, linear_key_head_dim=8, linear_num_value_heads=4, linear_value_head_dim=8,
            linear_conv_kernel_dim=4, full_attention_interval=2, max_position_embeddings=64)


def _hf_model(kind: str):
    if kind == "qwen3_5_moe":
        from transformers.models.qwen3_5_moe.configuration_qwen3_5_moe import Qwen3_5MoeTextConfig as Cfg
        from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import Qwen3_5MoeForCausalLM as Model

        cfg = Cfg(**TINY)
    else:
        from transformers.models.qwen3_next.configuration_qwen3_next import Qwen3NextConfig as Cfg
        from transformers.models.qwen3_next.modeling_qwen3_next import Qwen3NextForCausalLM as Model

        cfg = Cfg(**TINY, intermediate_size=48, decoder_sparse_step=1, mlp_only_layers=[])
    torch.manual_seed(0)
    m = Model(cfg).eval()
    with torch.no_grad():  # move norms, decay parameters and the (empty-initialised) expert banks off their defaults
        for n, p in m.named_parameters():
            if "norm" in n or "A_log" in n or "dt_bias" in n:
                p.add_(0.3 * torch.randn_like(p))
            elif "experts." in n and p.dim() == 3:
                p.normal_(0, 0.2)
    return m, json.loads(cfg.to_json_string())


def _logits(arch, weights, tok):
    model = qwen35.Qwen35DecomposedModel(arch, {k: v.float() for k, v in weights.items()}, {}, backend="eager_torch",
                                         attention="xla")
    with torch.no_grad():
        return model.logits(model.clean_forward(LMBatch(tok)).output)


@pytest.mark.parametrize("kind", ["qwen3_5_moe", "qwen3_next"])
def test_snapshot_loads_and_matches_hf_logits(kind, tmp_path):
    from safetensors.torch import save_file

    try:
        m, cfg = _hf_model(kind)
    except ImportError as e:  # an older transformers without this family
        pytest.skip(str(e))
    snap = tmp_path / "hf_snapshots" / f"tiny--{kind}"
    snap.mkdir(parents=True)
    (snap / "config.json").write_text(json.dumps(cfg))
    sd = {k: v.detach().clone().contiguous() for k, v in m.state_dict().items()}
    save_file(sd, str(snap / "model.safetensors"))
    arch, w = loaders.load_from_spec(HFTarget(model_class="auto", model_name=f"tiny/{kind}"), tmp_path, torch.float32, "cpu")
    assert arch.family == "qwen35_moe" and arch.full_attention_interval == 2 and arch.partial_rotary_factor == 0.25
    tok = torch.randint(0, 101, (2, 24), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = m(tok).logits
    assert torch.allclose(_logits(arch, w, tok), ref, atol=2e-5)

    # one matrix per expert (the on-disk form of the original checkpoints) maps to the same banks
    per = {}
    for k, v in sd.items():
        if k.endswith("mlp.experts.gate_up_proj"):
            for e in range(v.shape[0]):
                per[k.replace("gate_up_proj", f"{e}.gate_proj.weight")] = v[e, :arch.d_ff].clone()
                per[k.replace("gate_up_proj", f"{e}.up_proj.weight")] = v[e, arch.d_ff:].clone()
        elif k.endswith("mlp.experts.down_proj"):
            for e in range(v.shape[0]):
                per[k.replace("down_proj", f"{e}.down_proj.weight")] = v[e].clone()
        else:
            per[k] = v
    w2 = loaders.remap_hf_qwen35(per, arch)
    assert set(w2) == set(w) and all(torch.equal(w2[k], w[k]) for k in w)

    # the pretrain-cache entry in this package's own key grammar round-trips
    entry = loaders.pretrain_cache_dir(tmp_path, "goodfire/proj/runs/abc123")
    loaders.save_qwen35_cache(entry, arch, w, step=7)
    arch3, w3 = loaders.load_from_spec(PretrainedQwen35MoeTarget(run_path="goodfire/proj/runs/abc123"), tmp_path,
                                       torch.float32, "cpu")
    assert arch3 == arch and all(torch.equal(w3[k], w[k]) for k in w)
