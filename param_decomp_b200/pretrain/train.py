"""`python -m param_decomp_b200.pretrain.train <config.yaml> --data-root <dir>`

Pretrains a small decoder LM (LlamaSimpleMLP / LlamaSimple / GPT2Simple shapes expressed through
`TransformerArchConfig`) with AdamW, linear warm-up + cosine decay, gradient clipping, bf16 autocast
and data parallelism, and writes `<data_root>/pretrain_cache/<project>-<run_id>/
{model_config.yaml, model_step_<N>.safetensors}` for the decomposition runs to load.

YAML keys follow the reference's pretrain configs: `run_name, seed, dtype, global_batch,
num_iterations, warmup_iters, learning_rate, learning_rate_decay_frac, weight_decay, grad_clip,
log_every, val_every, val_steps, save_every, model: {model_type, n_layer, n_head, n_embd,
n_intermediate, vocab_size, n_ctx, rotary_base, n_key_value_heads, rms_norm_eps}, data_layout, data,
val_data, wandb` (param_decomp/pretrain/configs/*.yaml; pretrain/train.py:263-495; pretrain/models.py).
"""

from __future__ import annotations

import argparse
import math
from pathlib import Path
from typing import Any, Literal

import torch
import torch.nn.functional as F
from pydantic import Field, PositiveFloat, PositiveInt

from param_decomp_b200.config.experiments import LMDatasetRef, SyntheticZipfDataset, TransformerArchConfig
from param_decomp_b200.config.run import WandbConfig
from param_decomp_b200.core.metrics import MetricsSink, get_logger
from param_decomp_b200.formats.base import BaseConfig
from param_decomp_b200.models import transformer as tf
from param_decomp_b200.models.loaders import save_qwen35_cache, save_simple_mlp_cache


class PretrainModelConfig(BaseConfig):
    model_type: Literal["LlamaSimpleMLP", "LlamaSimple", "GPT2Simple", "Qwen35Moe"] = "LlamaSimpleMLP"
    hybrid: TransformerArchConfig | None = None
    """`Qwen35Moe` only: the full hybrid architecture (gated DeltaNet / gated attention / routed + shared experts);
    the flat fields above must agree with it where they overlap."""
    block_size: PositiveInt | None = None
    vocab_size: PositiveInt
    n_layer: PositiveInt
    n_head: PositiveInt
    n_embd: PositiveInt
    n_intermediate: PositiveInt | None = None  # GPT2Simple: 4 x n_embd
    rotary_base: PositiveFloat = 10000.0
    n_ctx: PositiveInt = 512
    n_key_value_heads: PositiveInt | None = None
    rms_norm_eps: PositiveFloat = 1e-6
    layer_norm_eps: PositiveFloat = 1e-5
    tie_word_embeddings: bool = False

    def arch(self) -> TransformerArchConfig:
        if self.model_type == "Qwen35Moe":
            assert self.hybrid is not None and self.hybrid.family == "qwen35_moe", "Qwen35Moe needs `model.hybrid`"
            h = self.hybrid
            assert (h.n_layer, h.d_model, h.vocab_size) == (self.n_layer, self.n_embd, self.vocab_size)
            return h
        family = "simple_mlp" if self.model_type in ("LlamaSimpleMLP", "GPT2Simple") else "glu_transformer"
        if self.model_type == "GPT2Simple":
            # learned absolute positions, LayerNorm with bias, plain multi-head attention, tied head
            # (param_decomp/pretrain/models.py:46-62,144-207)
            return TransformerArchConfig(family=family, n_layer=self.n_layer, d_model=self.n_embd, n_head=self.n_head,
                                         d_ff=self.n_intermediate or 4 * self.n_embd, vocab_size=self.vocab_size,
                                         max_seq_len=self.n_ctx, rms_eps=self.layer_norm_eps, tie_embeddings=True, norm_kind="layer",
                                         positional="learned")
        return TransformerArchConfig(family=family, n_layer=self.n_layer, d_model=self.n_embd, n_head=self.n_head,
                                     n_kv_head=self.n_key_value_heads, d_ff=self.n_intermediate or 4 * self.n_embd,
                                     vocab_size=self.vocab_size, max_seq_len=self.n_ctx, rope_theta=self.rotary_base,
                                     rms_eps=self.rms_norm_eps, tie_embeddings=self.tie_word_embeddings)


class PretrainConfig(BaseConfig):
    run_name: str
    seed: int = 0
    dp: PositiveInt = 1
    dtype: Literal["bfloat16", "float32"] = "bfloat16"
    attention_implementation: Literal["flash", "xla", "mosaic"] = "flash"
    global_batch: PositiveInt
    num_iterations: PositiveInt
    warmup_iters: int = 0
    learning_rate: PositiveFloat
    learning_rate_decay_frac: float = 0.1
    weight_decay: float = 0.1
    grad_clip: float | None = 1.0
    log_every: PositiveInt = 100
    val_every: PositiveInt = 1000
    val_steps: PositiveInt = 20
    save_every: PositiveInt = 1000
    model: PretrainModelConfig
    data_layout: Literal["documents", "unsegmented_tokens"] = "unsegmented_tokens"
    data: LMDatasetRef = Field(default_factory=SyntheticZipfDataset)
    val_data: LMDatasetRef = Field(default_factory=lambda: SyntheticZipfDataset(seed=1))
    wandb: WandbConfig | None = None


def lr_at(cfg: PretrainConfig, it: int) -> float:
    if it < cfg.warmup_iters:
        return cfg.learning_rate * (it + 1) / cfg.warmup_iters
    frac = (it - cfg.warmup_iters) / max(1, cfg.num_iterations - cfg.warmup_iters)
    lo = cfg.learning_rate * cfg.learning_rate_decay_frac
    return lo + 0.5 * (cfg.learning_rate - lo) * (1 + math.cos(math.pi * min(frac, 1.0)))


def pretrain(cfg: PretrainConfig, data_root: Path, run_id: str = "t-00000000", project: str = "spd",
             device: str = "cpu", max_iterations: int | None = None) -> Path:
    """Returns the cache entry directory."""
    from param_decomp_b200.data.shards import ShardServer
    from param_decomp_b200.data.synthetic import ZipfTokenSource

    log = get_logger()
    arch = cfg.model.arch()
    dtype = torch.bfloat16 if (cfg.dtype == "bfloat16" and device != "cpu") else torch.float32
    hybrid = arch.family == "qwen35_moe"
    if hybrid:
        from param_decomp_b200.models import qwen35

        init = qwen35.random_init_qwen35_weights(arch, cfg.seed, torch.float32, device)
    else:
        init = tf.random_init_weights(arch, cfg.seed, torch.float32, device)
    weights = {k: v.float().to(device).requires_grad_(True) for k, v in init.items()}
    seq = cfg.model.n_ctx

    def source(ref: Any, salt: int):
        if isinstance(ref, SyntheticZipfDataset):
            return ZipfTokenSource(arch.vocab_size, seq + 1, ref.exponent, ref.seed + salt)
        return ShardServer.open(ref, data_root, seq + 1, cfg.data_layout, seed=cfg.seed + salt)

    train_src, val_src = source(cfg.data, 0), source(cfg.val_data, 1)
    decay = [p for k, p in weights.items() if p.dim() >= 2]
    no_decay = [p for k, p in weights.items() if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": cfg.weight_decay},
                             {"params": no_decay, "weight_decay": 0.0}], lr=cfg.learning_rate, betas=(0.9, 0.95))
    entry = Path(data_root) / "pretrain_cache" / f"{project}-{run_id}"
    sink = MetricsSink.for_run(entry, 0)

    def loss_on(batch) -> torch.Tensor:
        cls = qwen35.Qwen35DecomposedModel if hybrid else tf.TransformerDecomposedModel
        model = cls(arch, {k: v.to(dtype) for k, v in weights.items()}, {}, backend="eager_torch",
                    attention="xla" if device == "cpu" else cfg.attention_implementation)
        toks = batch.tokens.to(device)
        out = model._run(tf.LMBatch(toks[:, :-1], None if batch.segment_ids is None else batch.segment_ids[:, :-1].to(device)),
                         None, None, (), want_taps=False)
        logits = model.logits(out.output).float()
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]), toks[:, 1:].reshape(-1).long())

    n_iter = min(cfg.num_iterations, max_iterations or cfg.num_iterations)
    for it in range(n_iter):
        for g in opt.param_groups:
            g["lr"] = lr_at(cfg, it)
        loss = loss_on(train_src.batch(it, cfg.global_batch))
        opt.zero_grad(set_to_none=True)
        loss.backward()
        if cfg.grad_clip:
            torch.nn.utils.clip_grad_norm_(list(weights.values()), cfg.grad_clip)
        opt.step()
        if it % cfg.log_every == 0 or it == n_iter - 1:
            sink.log(it, {"loss": loss.detach(), "lr": lr_at(cfg, it)}, prefix="pretrain/")
            log.info("pretrain it %d loss %.4f", it, float(loss))
        if (it + 1) % cfg.val_every == 0 or it == n_iter - 1:
            with torch.no_grad():
                val = sum(float(loss_on(val_src.batch(i, cfg.global_batch))) for i in range(min(cfg.val_steps, 2))) / min(cfg.val_steps, 2)
            sink.log(it, {"val_loss": val}, prefix="pretrain/")
        if (it + 1) % cfg.save_every == 0 or it == n_iter - 1:
            snap = {k: v.detach().to(torch.bfloat16 if cfg.dtype == "bfloat16" else torch.float32) for k, v in weights.items()}
            if hybrid:
                save_qwen35_cache(entry, arch, snap, it + 1)
            else:
                save_simple_mlp_cache(entry, arch, snap, it + 1)
    sink.close()
    return entry


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("config", type=Path)
    ap.add_argument("--data-root", type=Path, required=True)
    ap.add_argument("--run-id", type=str, default="t-00000000")
    ap.add_argument("--device", type=str, default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args()
    print(pretrain(PretrainConfig.from_file(args.config), args.data_root, args.run_id, device=args.device))


if __name__ == "__main__":
    main()
