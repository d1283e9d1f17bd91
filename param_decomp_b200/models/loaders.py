"""Frozen-target weight sources: HuggingFace safetensors snapshots (Llama-3.1, Qwen3) and the
in-house pretrain cache (LlamaSimpleMLP / LlamaSimple / GPT2Simple checkpoints).

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


def arch_from_hf_config(cfg: dict[str, Any], family: str = "glu_transformer") -> TransformerArchConfig:
    return TransformerArchConfig(
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
    arch = arch_from_hf_config(cfg)
    files = sorted(Path(snapshot_dir).glob("*.safetensors"))
    assert files, f"no safetensors files in {snapshot_dir}"
    return arch, remap_hf_llama(read_safetensors(files, dtype, device), arch)


def load_simple_mlp_cache(entry: Path, dtype: torch.dtype, device) -> tuple[TransformerArchConfig, dict[str, Tensor]]:
    """LlamaSimpleMLP pretrain checkpoints: `h.{i}.attn.q_proj.weight`, `h.{i}.mlp.c_fc.weight`,
    `h.{i}.rms_1.weight`, `wte.weight`, `ln_f.weight`, `lm_head.weight`."""
    mc = yaml.safe_load((entry / "model_config.yaml").read_text())
    m = mc.get("model", mc)
    arch = TransformerArchConfig(
        family="simple_mlp", n_layer=m["n_layer"], d_model=m["n_embd"], n_head=m["n_head"],
        n_kv_head=m.get("n_key_value_heads"), d_ff=m["n_intermediate"], vocab_size=m["vocab_size"],
        max_seq_len=m.get("n_ctx", m.get("block_size", 512)), rope_theta=float(m.get("rotary_base", 10000)),
        rms_eps=float(m.get("rms_norm_eps", 1e-6)), tie_embeddings=bool(m.get("tie_word_embeddings", False)))
    raw = read_safetensors([latest_checkpoint(entry)], dtype, device)
    out = {"embed.weight": raw["wte.weight"], "final_norm.weight": raw["ln_f.weight"]}
    if "lm_head.weight" in raw and not arch.tie_embeddings:
        out["lm_head.weight"] = raw["lm_head.weight"]
    for i in range(arch.n_layer):
        out[f"layers.{i}.attn_norm.weight"] = raw[f"h.{i}.rms_1.weight"]
        out[f"layers.{i}.mlp_norm.weight"] = raw[f"h.{i}.rms_2.weight"]
        for k in tf.SIMPLE_KINDS:
            out[tf.weight_key("simple_mlp", i, k)] = raw[tf.site_name("simple_mlp", i, k) + ".weight"]
    return arch, out


def save_simple_mlp_cache(entry: Path, arch: TransformerArchConfig, weights: dict[str, Tensor], step: int) -> None:
    """Inverse of `load_simple_mlp_cache` (used by the pretrainer and by tests)."""
    from safetensors.torch import save_file

    entry.mkdir(parents=True, exist_ok=True)
    (entry / "model_config.yaml").write_text(yaml.dump({"model": {
        "model_type": "LlamaSimpleMLP", "n_layer": arch.n_layer, "n_embd": arch.d_model, "n_head": arch.n_head,
        "n_key_value_heads": arch.n_kv_head or arch.n_head, "n_intermediate": arch.d_ff, "vocab_size": arch.vocab_size,
        "n_ctx": arch.max_seq_len, "rotary_base": arch.rope_theta, "rms_norm_eps": arch.rms_eps,
        "tie_word_embeddings": arch.tie_embeddings}}))
    raw = {"wte.weight": weights["embed.weight"], "ln_f.weight": weights["final_norm.weight"]}
    if "lm_head.weight" in weights:
        raw["lm_head.weight"] = weights["lm_head.weight"]
    for i in range(arch.n_layer):
        raw[f"h.{i}.rms_1.weight"] = weights[f"layers.{i}.attn_norm.weight"]
        raw[f"h.{i}.rms_2.weight"] = weights[f"layers.{i}.mlp_norm.weight"]
        for k in tf.SIMPLE_KINDS:
            raw[tf.site_name("simple_mlp", i, k) + ".weight"] = weights[tf.weight_key("simple_mlp", i, k)]
    save_file({k: v.detach().cpu().contiguous() for k, v in raw.items()}, str(entry / f"model_step_{step}.safetensors"))


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
        raise NotImplementedError("the Qwen3.5 hybrid (DeltaNet) checkpoint layout is loaded by models/qwen35.py")
    raise TypeError(type(spec).__name__)
