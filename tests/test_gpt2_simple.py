"""The pretrainer's other two dense model types: `GPT2Simple` (learned positions, LayerNorm with bias, plain
multi-head attention, two-matrix GELU(tanh) MLP, tied head) and `LlamaSimple` (RoPE, RMSNorm, SwiGLU). Forward parity
against a plain restatement of the reference's model math (param_decomp/pretrain/models.py:144-207), the
pretrain-cache round trip in the reference's key grammar, and a decomposition step on the loaded target."""
import math

import pytest
import torch
import torch.nn.functional as F


def _gpt2_oracle(w: dict, tokens: torch.Tensor, n_head: int, eps: float) -> torch.Tensor:
    def ln(x, wt, b):
        mean = x.mean(-1, keepdim=True)
        var = ((x - mean) ** 2).mean(-1, keepdim=True)
        return wt * ((x - mean) * torch.rsqrt(var + eps)) + b

    B, T = tokens.shape
    x = w["wte.weight"][tokens] + w["wpe.weight"][torch.arange(T)]
    d = x.shape[-1]
    hd = d // n_head
    n_layer = 1 + max(int(k.split(".")[1]) for k in w if k.startswith("h."))
    for i in range(n_layer):
        h = ln(x, w[f"h.{i}.ln_1.weight"], w[f"h.{i}.ln_1.bias"])
        q, k, v = (F.linear(h, w[f"h.{i}.attn.{n}_proj.weight"]).view(B, T, n_head, hd).transpose(1, 2) for n in "qkv")
        s = (q @ k.transpose(-1, -2)) / math.sqrt(hd)
        s = s.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), float("-inf"))
        a = (s.softmax(-1) @ v).transpose(1, 2).reshape(B, T, d)
        x = x + F.linear(a, w[f"h.{i}.attn.o_proj.weight"])
        h = ln(x, w[f"h.{i}.ln_2.weight"], w[f"h.{i}.ln_2.bias"])
        x = x + F.linear(F.gelu(F.linear(h, w[f"h.{i}.mlp.c_fc.weight"]), approximate="tanh"), w[f"h.{i}.mlp.down_proj.weight"])
    return F.linear(ln(x, w["ln_f.weight"], w["ln_f.bias"]), w["wte.weight"])


def test_gpt2_simple_forward_matches_the_reference_math():
    from param_decomp_b200.config.experiments import TransformerArchConfig
    from param_decomp_b200.models import loaders
    from param_decomp_b200.models import transformer as tf

    arch = TransformerArchConfig(family="simple_mlp", n_layer=2, d_model=32, n_head=4, d_ff=128, vocab_size=50,
                                 max_seq_len=16, rms_eps=1e-5, tie_embeddings=True, norm_kind="layer", positional="learned")
    w = tf.random_init_weights(arch, 3, torch.float32)
    g = torch.Generator().manual_seed(0)
    for k in w:  # non-trivial norm scales and shifts
        if k.endswith("norm.weight") or k.endswith("norm.bias"):
            w[k] = w[k] + 0.3 * torch.randn(w[k].shape, generator=g)
    assert "pos_embed.weight" in w and "lm_head.weight" not in w and "layers.0.attn_norm.bias" in w
    model = tf.TransformerDecomposedModel(arch, w, {}, backend="eager_torch", attention="xla")
    tokens = torch.randint(0, 50, (3, 12), generator=g)
    ours = model.logits(model._run(tf.LMBatch(tokens), None, None, (), want_taps=False).output)
    theirs_keys = {theirs: w[ours_k] for ours_k, theirs in loaders._cache_keys("GPT2Simple", 2).items()}
    want = _gpt2_oracle(theirs_keys, tokens, 4, 1e-5)
    assert torch.allclose(ours, want, atol=2e-5), float((ours - want).abs().max())


@pytest.mark.parametrize("model_type", ["GPT2Simple", "LlamaSimple"])
def test_pretrain_cache_roundtrip_of_the_other_model_types(tmp_path, model_type):
    import copy

    import __graft_entry__ as ge
    from param_decomp_b200.config.experiments import LMExperimentConfig, PretrainedTarget
    from param_decomp_b200.experiments.lm.training import train_lm
    from param_decomp_b200.models import loaders
    from param_decomp_b200.pretrain.train import PretrainConfig, pretrain
    from safetensors import safe_open

    model = {"model_type": model_type, "vocab_size": 64, "n_layer": 2, "n_head": 2, "n_embd": 32, "n_ctx": 16}
    if model_type == "LlamaSimple":
        model.update({"n_intermediate": 48, "n_key_value_heads": 1})
    cfg = PretrainConfig.model_validate({
        "run_name": "t", "global_batch": 4, "num_iterations": 6, "warmup_iters": 1, "learning_rate": 3e-3,
        "log_every": 1, "val_every": 3, "save_every": 6, "dtype": "float32", "model": model})
    entry = pretrain(cfg, tmp_path, run_id="t-0000aaaa", project="spd")
    with safe_open(str(next(entry.glob("model_step_*.safetensors"))), framework="pt") as f:
        keys = set(f.keys())
    if model_type == "GPT2Simple":
        assert {"wte.weight", "wpe.weight", "ln_f.bias", "h.0.ln_1.bias", "h.1.mlp.c_fc.weight"} <= keys and "lm_head.weight" not in keys
    else:
        assert {"wte.weight", "h.0.rms_1.weight", "h.1.mlp.gate_proj.weight", "h.0.attn.k_proj.weight"} <= keys
    spec = PretrainedTarget(model_class=model_type, run_path="goodfire/spd/runs/t-0000aaaa")
    arch, weights = loaders.load_from_spec(spec, tmp_path, torch.float32, "cpu")
    assert arch.family == ("simple_mlp" if model_type == "GPT2Simple" else "glu_transformer")
    assert (arch.norm_kind, arch.positional) == (("layer", "learned") if model_type == "GPT2Simple" else ("rms", "rope"))
    # the loaded target decomposes: two steps through the engine on the eager backend
    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"]["backend"] = "eager_torch"
    c["target"] = {"spec": {"kind": "pretrained", "model_class": model_type, "run_path": "goodfire/spd/runs/t-0000aaaa"},
                   "attention_implementation": "xla", "output_edge": {"kind": "materialized"}, "weights_dtype": "float32"}
    if model_type == "GPT2Simple":
        c["decomposition"]["sites"] = {"kind": "simple_mlp", "layers": {"kind": "all"}, "cs": {"q_proj": 8, "c_fc": 16, "down_proj": 8}}
    else:
        c["decomposition"]["sites"] = {"kind": "glu_transformer", "layers": {"kind": "all"}, "cs": {"q": 8, "gate": 16, "down": 8}}
    c["decomposition"]["ci"] = {"type": "layerwise_mlp", "hidden_dims": [16]}
    c["data"]["seq_len"] = 8
    c["pd"]["batch_size"] = 2
    c["pd"]["steps"] = 2
    c["cadence"] = {"train_log_every": 1, "checkpointing": {"kind": "none"}}
    c["eval"] = None
    res = train_lm(LMExperimentConfig.model_validate(c), tmp_path, run_id="p-0000eeee", device="cpu")
    assert res.final_step == 2 and math.isfinite(res.last_metrics["train/loss/total"])
