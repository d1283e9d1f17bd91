"""Llama- and Qwen3-style dense targets against the HuggingFace implementations: a tiny random model
is saved as a snapshot, read through the loader, and must give the same logits."""
import json

import pytest
import torch

from param_decomp_b200.config.experiments import HFTarget
from param_decomp_b200.models import loaders
from param_decomp_b200.models import transformer as tf

transformers = pytest.importorskip("transformers")


def _hf(kind: str):
    common = dict(vocab_size=97, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=2, max_position_embeddings=64, rms_norm_eps=1e-6, tie_word_embeddings=False)
    if kind == "llama":
        from transformers import LlamaConfig, LlamaForCausalLM

        cfg = LlamaConfig(**common, rope_theta=10000.0)
        model = LlamaForCausalLM(cfg)
    else:
        from transformers import Qwen3Config, Qwen3ForCausalLM

        cfg = Qwen3Config(**common, head_dim=16, rope_theta=10000.0)
        model = Qwen3ForCausalLM(cfg)
    torch.manual_seed(0)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "norm" in n:
                p.add_(0.3 * torch.randn_like(p))
    return model.eval(), json.loads(cfg.to_json_string())


@pytest.mark.parametrize("kind", ["llama", "qwen3"])
def test_dense_snapshot_matches_hf_logits(kind, tmp_path):
    from safetensors.torch import save_file

    m, cfg = _hf(kind)
    snap = tmp_path / "hf_snapshots" / f"tiny--{kind}"
    snap.mkdir(parents=True)
    (snap / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.detach().clone().contiguous() for k, v in m.state_dict().items()}, str(snap / "model.safetensors"))
    arch, w = loaders.load_from_spec(HFTarget(model_class="auto", model_name=f"tiny/{kind}"), tmp_path, torch.float32, "cpu")
    assert arch.qk_norm == (kind == "qwen3")
    model = tf.TransformerDecomposedModel(arch, w, {}, backend="eager_torch", attention="xla")
    tok = torch.randint(0, 97, (2, 20), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = m(tok).logits
        out = model.logits(model.clean_forward(tf.LMBatch(tok)).output)
    assert torch.allclose(out, ref, atol=2e-5), float((out - ref).abs().max())


def test_qwen3_moe_snapshot_matches_hf_logits(tmp_path):
    """The plain top-k mixture-of-experts target against HuggingFace Qwen3-MoE (softmax router, renormalised top-k,
    SwiGLU experts, q/k norms), through the snapshot loader."""
    from safetensors.torch import save_file

    from param_decomp_b200.models import moe

    try:
        from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM
    except ImportError as e:
        pytest.skip(str(e))
    cfg = Qwen3MoeConfig(vocab_size=97, hidden_size=32, intermediate_size=48, moe_intermediate_size=16, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, head_dim=16, num_experts=6, num_experts_per_tok=2,
                         norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], max_position_embeddings=64,
                         rms_norm_eps=1e-6, tie_word_embeddings=False)
    torch.manual_seed(0)
    m = Qwen3MoeForCausalLM(cfg).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" in n:
                p.add_(0.3 * torch.randn_like(p))
            elif "experts." in n and p.dim() == 3:
                p.normal_(0, 0.2)
    snap = tmp_path / "hf_snapshots" / "tiny--qwen3moe"
    snap.mkdir(parents=True)
    (snap / "config.json").write_text(cfg.to_json_string())
    save_file({k: v.detach().clone().contiguous() for k, v in m.state_dict().items()}, str(snap / "model.safetensors"))
    arch, w = loaders.load_from_spec(HFTarget(model_class="auto", model_name="tiny/qwen3moe"), tmp_path, torch.float32, "cpu")
    assert arch.family == "moe" and arch.n_experts == 6 and arch.norm_topk_prob
    model = moe.MoEDecomposedModel(arch, w, {}, backend="eager_torch", attention="xla")
    tok = torch.randint(0, 97, (2, 20), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = m(tok).logits
        out = model.logits(model.clean_forward(tf.LMBatch(tok)).output)
    assert torch.allclose(out, ref, atol=2e-5), float((out - ref).abs().max())
