"""Frozen-target weight sources: HuggingFace safetensors snapshots (Llama-3.1, Qwen3, the Qwen3.5 /
Qwen3-Next hybrid mixture-of-experts family) and the in-house pretrain cache (LlamaSimpleMLP /
LlamaSimple / GPT2Simple checkpoints, hybrid mixture-of-experts checkpoints).

All loaders return `(TransformerArchConfig, {internal key: tensor})` with the key grammar of
`models/transformer.py` (`embed.weight`, `layers.{i}.attn_norm.weight`, site weights named by the
family's site grammar, `final_norm.weight`, `lm_head.weight`).

Pretrain cache entry: `<data_root>/pretrain_cache/<project>-<run_id>/{model_config.yaml,
model_step_<N>.safetensors}`; a `run_path` is `entity/project[/runs]/run_id`.

Parity: param_decomp/targets/llama31.py:23-76, targets/qwen3.py:37-218,
targets/llama_simple_mlp.py:202-348, targets/transformer.py:2308-2358 (HF snapshot reading),
pretrain/cache.py:21-74, infra/pretrain_cache.py:44-124.
"""

from __future__ import annotations

import json
import re
from pathlib import Path
from typing import Any

import torch
import yaml
from safetensors import safe_open
from torch import Tensor

from param_decomp_b200.config.experiments import (
    HFTarget,
    HFWeightsInVendored,
    PretrainedQwen35MoeTarget,
    PretrainedTarget,
    TransformerArchConfig,
)
from param_decomp_b200.models import transformer as tf


def parse_run_path(run_path: str) -> tuple[str, str]:
    """`entity/project[/runs]/run_id` -> `(project, run_id)`."""
    parts = [p for p in run_path.split("/") if p]
    if len(parts) == 4 and parts[2] == "runs":
        parts = [parts[0], parts[1], parts[3]]
    assert len(parts) == 3, f"run_path must be entity/project[/runs]/run_id, got {run_path!r}"
    return parts[1], parts[2]


def pretrain_cache_dir(data_root: Path, run_path: str) -> Path:
    project, run_id = parse_run_path(run_path)
    return Path(data_root) / "pretrain_cache" / f"{project}-{run_id}"


def latest_checkpoint(entry: Path) -> Path:
    files = sorted(entry.glob("model_step_*.safetensors"), key=lambda p: int(re.findall(r"\d+", p.stem)[-1]))
    assert files, f"no model_step_<N>.safetensors in {entry} (offline: the cache entry must already exist)"
    return files[-1]


def read_safetensors(paths: list[Path], dtype: torch.dtype, device) -> dict[str, Tensor]:
    out = {}
    for p in paths:
        with safe_open(str(p), framework="pt") as f:
            for k in f.keys():
                out[k] = f.get_tensor(k).to(dtype).to(device)
    return out


def _llama3_rope_scaling(cfg: dict[str, Any]):
    """`rope_scaling: {rope_type: llama3, factor, low_freq_factor, high_freq_factor,
    original_max_position_embeddings}` of a HuggingFace config, or None."""
    rs = cfg.get("rope_scaling") or {}
    if (rs.get("rope_type") or rs.get("type")) != "llama3":
        return None
    from param_decomp_b200.config.experiments import Llama3RopeScalingConfig

    return Llama3RopeScalingConfig(
        factor=rs.get("factor", 8.0), low_freq_factor=rs.get("low_freq_factor", 1.0),
        high_freq_factor=rs.get("high_freq_factor", 4.0),
        original_max_position_embeddings=rs.get("original_max_position_embeddings", 8192))


def arch_from_hf_config(cfg: dict[str, Any], family: str = "glu_transformer") -> TransformerArchConfig:
    return TransformerArchConfig(
        rope_scaling=_llama3_rope_scaling(cfg),
        family=family, n_layer=cfg["num_hidden_layers"], d_model=cfg["hidden_size"], n_head=cfg["num_attention_heads"],
        n_kv_head=cfg.get("num_key_value_heads"), head_dim=cfg.get("head_dim"), d_ff=cfg["intermediate_size"],
        vocab_size=cfg["vocab_size"], max_seq_len=cfg.get("max_position_embeddings", 2048),
        rope_theta=cfg.get("rope_theta", 10000.0), rms_eps=cfg.get("rms_norm_eps", 1e-6),
        qk_norm=cfg.get("model_type", "") == "qwen3", tie_embeddings=cfg.get("tie_word_embeddings", False))


def remap_hf_llama(raw: dict[str, Tensor], arch: TransformerArchConfig) -> dict[str, Tensor]:
    """HF `model.layers.N.self_attn.q_proj.weight` style keys -> internal keys (GLU family)."""
    out = {"embed.weight": raw["model.embed_tokens.weight"], "final_norm.weight": raw["model.norm.weight"]}
    if "lm_head.weight" in raw and not arch.tie_embeddings:
        out["lm_head.weight"] = raw["lm_head.weight"]
    for i in range(arch.n_layer):
        p = f"model.layers.{i}."
        out[f"layers.{i}.attn_norm.weight"] = raw[p + "input_layernorm.weight"]
        out[f"layers.{i}.mlp_norm.weight"] = raw[p + "post_attention_layernorm.weight"]
        for k in ("q", "k", "v", "o"):
            out[tf.weight_key("glu_transformer", i, k)] = raw[p + f"self_attn.{k}_proj.weight"]
        for k in ("gate", "up", "down"):
            out[tf.weight_key("glu_transformer", i, k)] = raw[p + f"mlp.{k}_proj.weight"]
        if arch.qk_norm:
            out[f"layers.{i}.q_norm.weight"] = raw[p + "self_attn.q_norm.weight"]
            out[f"layers.{i}.k_norm.weight"] = raw[p + "self_attn.k_norm.weight"]
    return out


def load_hf_snapshot(snapshot_dir: Path, dtype: torch.dtype, device) -> tuple[TransformerArchConfig, dict[str, Tensor]]:
    cfg = json.loads((Path(snapshot_dir) / "config.json").read_text())
    files = sorted(Path(snapshot_dir).glob("*.safetensors"))
    assert files, f"no safetensors files in {snapshot_dir}"
    text = cfg.get("text_config", cfg)
    if "linear_num_value_heads" in text:  # hybrid DeltaNet mixture-of-experts family
        arch = qwen35_arch_from_hf_config(cfg)
        return arch, remap_hf_qwen35(read_safetensors(files, dtype, device), arch)
    if "moe_intermediate_size" in cfg and ("num_experts" in cfg or "num_local_experts" in cfg):  # plain top-k MoE
        arch = moe_arch_from_hf_config(cfg)
        return arch, remap_hf_qwen3_moe(read_safetensors(files, dtype, device), arch)
    arch = arch_from_hf_config(cfg)
    return arch, remap_hf_llama(read_safetensors(files, dtype, device), arch)


def _cache_model_type(arch: TransformerArchConfig) -> str:
    if arch.family == "glu_transformer":
        return "LlamaSimple"
    return "GPT2Simple" if arch.norm_kind == "layer" else "LlamaSimpleMLP"


def _cache_keys(model_type: str, n_layer: int) -> dict[str, str]:
    """This package's weight key -> the pretrain checkpoint's key, per model type (the key grammars of
    param_decomp/pretrain/models.py `state_dict`: `h.{i}.attn.q_proj.weight`, `h.{i}.mlp.c_fc.weight` or
    `gate/up/down_proj`, `h.{i}.rms_1.weight` or `ln_1.{weight,bias}`, `wte.weight`, `wpe.weight`, `ln_f.*`)."""
    gpt2 = model_type == "GPT2Simple"
    fam = "glu_transformer" if model_type == "LlamaSimple" else "simple_mlp"
    n1, n2 = ("ln_1", "ln_2") if gpt2 else ("rms_1", "rms_2")
    out = {"embed.weight": "wte.weight", "final_norm.weight": "ln_f.weight"}
    if gpt2:
        out["final_norm.bias"], out["pos_embed.weight"] = "ln_f.bias", "wpe.weight"
    for i in range(n_layer):
        out[f"layers.{i}.attn_norm.weight"], out[f"layers.{i}.mlp_norm.weight"] = f"h.{i}.{n1}.weight", f"h.{i}.{n2}.weight"
        if gpt2:
            out[f"layers.{i}.attn_norm.bias"], out[f"layers.{i}.mlp_norm.bias"] = f"h.{i}.{n1}.bias", f"h.{i}.{n2}.bias"
        if fam == "simple_mlp":
            for k in tf.SIMPLE_KINDS:
                out[tf.weight_key(fam, i, k)] = tf.site_name("simple_mlp", i, k) + ".weight"
        else:
            for k in ("q", "k", "v", "o"):
                out[tf.weight_key(fam, i, k)] = f"h.{i}.attn.{k}_proj.weight"
            for k in ("gate", "up", "down"):
                out[tf.weight_key(fam, i, k)] = f"h.{i}.mlp.{k}_proj.weight"
    return out


def load_simple_mlp_cache(entry: Path, dtype: torch.dtype, device) -> tuple[TransformerArchConfig, dict[str, Tensor]]:
    """Pretrain checkpoints of the in-house dense models: `LlamaSimpleMLP` (RoPE, RMSNorm, two-matrix GELU MLP),
    `LlamaSimple` (the same with a SwiGLU MLP) and `GPT2Simple` (learned positions, LayerNorm with bias,
    two-matrix GELU MLP, tied head); `model_config.yaml` names the type."""
    mc = yaml.safe_load((entry / "model_config.yaml").read_text())
    m = mc.get("model", mc)
    model_type = m.get("model_type", "LlamaSimpleMLP")
    gpt2 = model_type == "GPT2Simple"
    arch = TransformerArchConfig(
        family="glu_transformer" if model_type == "LlamaSimple" else "simple_mlp", n_layer=m["n_layer"],
        d_model=m["n_embd"], n_head=m["n_head"], n_kv_head=None if gpt2 else m.get("n_key_value_heads"),
        d_ff=m.get("n_intermediate", 4 * m["n_embd"]), vocab_size=m["vocab_size"],
        max_seq_len=m.get("n_ctx", m.get("block_size", 512)), rope_theta=float(m.get("rotary_base", 10000)),
        rms_eps=float(m.get("layer_norm_eps", 1e-5) if gpt2 else m.get("rms_norm_eps", 1e-6)),
        tie_embeddings=bool(m.get("tie_word_embeddings", gpt2)),
        norm_kind="layer" if gpt2 else "rms", positional="learned" if gpt2 else "rope")
    raw = read_safetensors([latest_checkpoint(entry)], dtype, device)
    out = {ours: raw[theirs] for ours, theirs in _cache_keys(model_type, arch.n_layer).items()}
    if "lm_head.weight" in raw and not arch.tie_embeddings:
        out["lm_head.weight"] = raw["lm_head.weight"]
    return arch, out


def save_simple_mlp_cache(entry: Path, arch: TransformerArchConfig, weights: dict[str, Tensor], step: int) -> None:
    """Inverse of `load_simple_mlp_cache` (used by the pretrainer and by tests)."""
    from safetensors.torch import save_file

    entry.mkdir(parents=True, exist_ok=True)
    model_type = _cache_model_type(arch)
    cfg = {"model_type": model_type, "n_layer": arch.n_layer, "n_embd": arch.d_model, "n_head": arch.n_head,
           "n_intermediate": arch.d_ff, "vocab_size": arch.vocab_size, "n_ctx": arch.max_seq_len,
           "tie_word_embeddings": arch.tie_embeddings}
    if model_type == "GPT2Simple":
        cfg["layer_norm_eps"] = arch.rms_eps
    else:
        cfg.update({"n_key_value_heads": arch.n_kv_head or arch.n_head, "rotary_base": arch.rope_theta,
                    "rms_norm_eps": arch.rms_eps})
    (entry / "model_config.yaml").write_text(yaml.dump({"model": cfg}))
    raw = {theirs: weights[ours] for ours, theirs in _cache_keys(model_type, arch.n_layer).items()}
    if "lm_head.weight" in weights and not arch.tie_embeddings:
        raw["lm_head.weight"] = weights["lm_head.weight"]
    save_file({k: v.detach().cpu().contiguous() for k, v in raw.items()}, str(entry / f"model_step_{step}.safetensors"))


# ---- plain top-k mixture of experts (Qwen3-MoE style: softmax router, SwiGLU experts, no shared expert) ----


def moe_arch_from_hf_config(cfg: dict[str, Any]) -> TransformerArchConfig:
    return TransformerArchConfig(
        family="moe", n_layer=cfg["num_hidden_layers"], d_model=cfg["hidden_size"], n_head=cfg["num_attention_heads"],
        n_kv_head=cfg.get("num_key_value_heads"), head_dim=cfg.get("head_dim"), d_ff=cfg["moe_intermediate_size"],
        vocab_size=cfg["vocab_size"], max_seq_len=cfg.get("max_position_embeddings", 2048),
        rope_theta=float((cfg.get("rope_parameters") or {}).get("rope_theta", cfg.get("rope_theta", 10000.0))),
        rms_eps=cfg.get("rms_norm_eps", 1e-6), qk_norm=True, tie_embeddings=cfg.get("tie_word_embeddings", False),
        n_experts=cfg.get("num_experts", cfg.get("num_local_experts")), experts_per_token=cfg["num_experts_per_tok"],
        norm_topk_prob=cfg.get("norm_topk_prob", False))


def remap_hf_qwen3_moe(raw: dict[str, Tensor], arch: TransformerArchConfig) -> dict[str, Tensor]:
    """HF Qwen3-MoE keys -> the key grammar of `models/moe.py`; expert banks fused (`mlp.experts.gate_up_proj`,
    `mlp.experts.down_proj`) or one matrix per expert (`mlp.experts.{e}.gate_proj.weight`)."""
    out = {"embed.weight": raw["model.embed_tokens.weight"], "final_norm.weight": raw["model.norm.weight"]}
    if "lm_head.weight" in raw and not arch.tie_embeddings:
        out["lm_head.weight"] = raw["lm_head.weight"]
    for i in range(arch.n_layer):
        p = f"model.layers.{i}."
        out[f"layers.{i}.attn_norm.weight"] = raw[p + "input_layernorm.weight"]
        out[f"layers.{i}.mlp_norm.weight"] = raw[p + "post_attention_layernorm.weight"]
        for k in ("q", "k", "v", "o"):
            out[tf.weight_key("moe", i, k)] = raw[p + f"self_attn.{k}_proj.weight"]
        out[f"layers.{i}.q_norm.weight"] = raw[p + "self_attn.q_norm.weight"]
        out[f"layers.{i}.k_norm.weight"] = raw[p + "self_attn.k_norm.weight"]
        m = p + "mlp."
        out[f"layers.{i}.mlp.router.weight"] = raw[m + "gate.weight"]
        if m + "experts.gate_up_proj" in raw:
            gu = raw[m + "experts.gate_up_proj"]
            gate, up, down = gu[:, :arch.d_ff], gu[:, arch.d_ff:], raw[m + "experts.down_proj"]
        else:
            per = lambda nm: torch.stack([raw[f"{m}experts.{e}.{nm}.weight"] for e in range(arch.n_experts)])  # noqa: E731
            gate, up, down = per("gate_proj"), per("up_proj"), per("down_proj")
        for kind, w in (("experts_gate", gate), ("experts_up", up), ("experts_down", down)):
            out[tf.weight_key("moe", i, kind)] = w.contiguous()
    return out


# ---- Qwen3.5-style hybrid (gated DeltaNet + gated attention + routed experts) ------------------------


def qwen35_arch_from_hf_config(cfg: dict[str, Any]) -> TransformerArchConfig:
    """`config.json` of a Qwen3.5 / Qwen3-Next style mixture-of-experts model (the text tower's fields
    sit under `text_config` in the multimodal layout)."""
    c = cfg.get("text_config", cfg)
    rope = c.get("rope_parameters") or c.get("rope_scaling") or {}
    interval = c.get("full_attention_interval", 4)
    if c.get("layer_types"):  # the explicit per-layer list wins; it must be the periodic pattern
        kinds = list(c["layer_types"])
        interval = kinds.index("full_attention") + 1
        assert kinds == [("full_attention" if (i + 1) % interval == 0 else "linear_attention") for i in range(len(kinds))], \
            f"layer_types {kinds} is not one full-attention layer every {interval}"
    return TransformerArchConfig(
        family="qwen35_moe", n_layer=c["num_hidden_layers"], d_model=c["hidden_size"], n_head=c["num_attention_heads"],
        n_kv_head=c.get("num_key_value_heads"), head_dim=c.get("head_dim") or c["hidden_size"] // c["num_attention_heads"],
        d_ff=c["moe_intermediate_size"], vocab_size=c["vocab_size"], max_seq_len=c.get("max_position_embeddings", 4096),
        rope_theta=float(rope.get("rope_theta", c.get("rope_theta", 10000.0))), rms_eps=c.get("rms_norm_eps", 1e-6),
        n_experts=c.get("num_experts", c.get("num_local_experts")), experts_per_token=c["num_experts_per_tok"],
        norm_topk_prob=c.get("norm_topk_prob", True), full_attention_interval=interval,
        partial_rotary_factor=float(rope.get("partial_rotary_factor", c.get("partial_rotary_factor", 0.25))),
        linear_num_key_heads=c["linear_num_key_heads"], linear_key_head_dim=c["linear_key_head_dim"],
        linear_num_value_heads=c["linear_num_value_heads"], linear_value_head_dim=c["linear_value_head_dim"],
        linear_conv_kernel_dim=c.get("linear_conv_kernel_dim", 4),
        shared_expert_intermediate=c["shared_expert_intermediate_size"],
        tie_embeddings=c.get("tie_word_embeddings", cfg.get("tie_word_embeddings", False)))


def remap_hf_qwen35(raw: dict[str, Tensor], arch: TransformerArchConfig) -> dict[str, Tensor]:
    """HF keys -> the key grammar of `models/qwen35.py`.

    Accepts both text-tower prefixes (`model.language_model.` and `model.`), the fused expert banks
    (`mlp.experts.gate_up_proj [E, 2 ff, d]`, `mlp.experts.down_proj [E, d, ff]`) as well as one matrix
    per expert (`mlp.experts.{e}.gate_proj.weight`), and the fused DeltaNet input projection
    (`in_proj_qkv`, rows `[q | k | v]`, the depthwise `conv1d` over the same channel order) next to the
    Qwen3-Next form (`in_proj_qkvz` / `in_proj_ba`, grouped per key head). The gated-attention query
    projection keeps its per-head `[q | gate]` row order, which is the order the model reads."""
    from param_decomp_b200.models import qwen35 as Q

    root = "model.language_model." if any(k.startswith("model.language_model.") for k in raw) else "model."
    a = arch
    kd, vd = a.linear_num_key_heads * a.linear_key_head_dim, a.linear_num_value_heads * a.linear_value_head_dim
    out = {"embed.weight": raw[root + "embed_tokens.weight"], "final_norm.weight": raw[root + "norm.weight"]}
    out["lm_head.weight"] = raw["lm_head.weight"] if "lm_head.weight" in raw else raw[root + "embed_tokens.weight"]
    for i in range(a.n_layer):
        p = f"{root}layers.{i}."
        out[f"layers.{i}.attn_norm.weight"] = raw[p + "input_layernorm.weight"]
        out[f"layers.{i}.mlp_norm.weight"] = raw[p + "post_attention_layernorm.weight"]
        if Q.is_full_attention(a, i):
            for kind, hf in (("attn_q", "q_proj"), ("attn_k", "k_proj"), ("attn_v", "v_proj"), ("attn_o", "o_proj")):
                out[Q.site_name(i, kind) + ".weight"] = raw[p + f"self_attn.{hf}.weight"]
            out[f"layers.{i}.self_attn.q_norm.weight"] = raw[p + "self_attn.q_norm.weight"]
            out[f"layers.{i}.self_attn.k_norm.weight"] = raw[p + "self_attn.k_norm.weight"]
        else:
            la = p + "linear_attn."
            if la + "in_proj_qkv.weight" in raw:
                qkv = raw[la + "in_proj_qkv.weight"]
                q, k, v = qkv[:kd], qkv[kd:2 * kd], qkv[2 * kd:]
                z, b, al = raw[la + "in_proj_z.weight"], raw[la + "in_proj_b.weight"], raw[la + "in_proj_a.weight"]
            else:  # Qwen3-Next: rows grouped per key head as [q | k | v-heads | z-heads] and [b-heads | a-heads]
                Hk, dk, dv = a.linear_num_key_heads, a.linear_key_head_dim, a.linear_value_head_dim
                rep = a.linear_num_value_heads // Hk
                g = raw[la + "in_proj_qkvz.weight"].reshape(Hk, 2 * dk + 2 * rep * dv, -1)
                q, k = g[:, :dk].reshape(kd, -1), g[:, dk:2 * dk].reshape(kd, -1)
                v, z = g[:, 2 * dk:2 * dk + rep * dv].reshape(vd, -1), g[:, 2 * dk + rep * dv:].reshape(vd, -1)
                ba = raw[la + "in_proj_ba.weight"].reshape(Hk, 2 * rep, -1)
                b, al = ba[:, :rep].reshape(Hk * rep, -1), ba[:, rep:].reshape(Hk * rep, -1)
            for kind, w in (("gdn_q", q), ("gdn_k", k), ("gdn_v", v), ("gdn_z", z), ("gdn_b", b), ("gdn_a", al)):
                out[Q.site_name(i, kind) + ".weight"] = w.contiguous()
            out[Q.site_name(i, "gdn_out") + ".weight"] = raw[la + "out_proj.weight"]
            conv = raw[la + "conv1d.weight"].reshape(2 * kd + vd, -1)  # [channels, 1, K] -> [channels, K]
            out[f"layers.{i}.linear_attn.conv_q.weight"] = conv[:kd].contiguous()
            out[f"layers.{i}.linear_attn.conv_k.weight"] = conv[kd:2 * kd].contiguous()
            out[f"layers.{i}.linear_attn.conv_v.weight"] = conv[2 * kd:].contiguous()
            for leaf in ("A_log", "dt_bias", "norm.weight"):
                out[f"layers.{i}.linear_attn.{leaf}"] = raw[la + leaf]
        m = p + "mlp."
        out[f"layers.{i}.mlp.router.weight"] = raw[m + "gate.weight"]
        if m + "experts.gate_up_proj" in raw:
            gu = raw[m + "experts.gate_up_proj"]
            gate, up, down = gu[:, :a.d_ff], gu[:, a.d_ff:], raw[m + "experts.down_proj"]
        else:
            per = lambda nm: torch.stack([raw[f"{m}experts.{e}.{nm}.weight"] for e in range(a.n_experts)])  # noqa: E731
            gate, up, down = per("gate_proj"), per("up_proj"), per("down_proj")
        for kind, w in (("experts_gate", gate), ("experts_up", up), ("experts_down", down)):
            out[Q.site_name(i, kind) + ".weight"] = w.contiguous()
        for kind, hf in (("shared_gate", "gate_proj"), ("shared_up", "up_proj"), ("shared_down", "down_proj")):
            out[Q.site_name(i, kind) + ".weight"] = raw[m + f"shared_expert.{hf}.weight"]
        out[f"layers.{i}.mlp.shared_expert_gate.weight"] = raw[m + "shared_expert_gate.weight"].reshape(1, -1)
    return out


def load_qwen35_cache(entry: Path, dtype: torch.dtype, device) -> tuple[TransformerArchConfig, dict[str, Tensor]]:
    """Pretrain-cache entry of a hybrid model: `model_config.yaml` holds either the architecture in this
    package's field names (`model: {family: qwen35_moe, ...}`) or an HF-style config; the newest
    `model_step_<N>.safetensors` holds HF-style keys or this package's own keys."""
    mc = yaml.safe_load((entry / "model_config.yaml").read_text())
    m = mc.get("model", mc)
    arch = TransformerArchConfig.model_validate(m) if "family" in m else qwen35_arch_from_hf_config(m)
    raw = read_safetensors([latest_checkpoint(entry)], dtype, device)
    return arch, (raw if "embed.weight" in raw else remap_hf_qwen35(raw, arch))


def save_qwen35_cache(entry: Path, arch: TransformerArchConfig, weights: dict[str, Tensor], step: int) -> None:
    """Write a pretrain-cache entry in this package's own key grammar (pretrainer, tests)."""
    from safetensors.torch import save_file

    entry.mkdir(parents=True, exist_ok=True)
    (entry / "model_config.yaml").write_text(yaml.dump({"model": arch.model_dump(mode="json")}))
    save_file({k: v.detach().cpu().contiguous() for k, v in weights.items()}, str(entry / f"model_step_{step}.safetensors"))


def load_from_spec(spec: Any, data_root: Path | None, dtype: torch.dtype, device) -> tuple[TransformerArchConfig, dict]:
    if isinstance(spec, PretrainedTarget):
        assert data_root is not None, "pretrained targets resolve under --data-root"
        return load_simple_mlp_cache(pretrain_cache_dir(data_root, spec.run_path), dtype, device)
    if isinstance(spec, (HFTarget, HFWeightsInVendored)):
        assert data_root is not None
        snap = Path(data_root) / "hf_snapshots" / spec.model_name.replace("/", "--")
        assert snap.exists(), f"{snap} missing: HF snapshots must be staged offline under <data_root>/hf_snapshots/"
        return load_hf_snapshot(snap, dtype, device)
    if isinstance(spec, PretrainedQwen35MoeTarget):
        assert data_root is not None, "pretrained targets resolve under --data-root"
        return load_qwen35_cache(pretrain_cache_dir(data_root, spec.run_path), dtype, device)
    raise TypeError(type(spec).__name__)
