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
