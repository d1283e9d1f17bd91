"""`python -m param_decomp_b200.pretrain.train <config.yaml> --data-root <dir>`

Pretrains a small decoder LM (LlamaSimpleMLP / LlamaSimple / GPT2Simple shapes expressed through
`TransformerArchConfig`) with AdamW, linear warm-up + cosine decay, gradient clipping, bf16 autocast
and data parallelism (one process per GPU, launched with `torch.distributed.run` when `dp` is set), keeps a
resumable trainer state under `<entry>/ckpts` (newest `keep_last`), and writes `<data_root>/pretrain_cache/<project>-<run_id>/
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
import os
import re
import signal
import threading
import time
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
    """Keys of param_decomp/pretrain/config.py:40-110. `gpus_per_node` is accepted and only checked against the
    launch (one process per GPU here); `dp` is the data-parallel world the launch must have."""

    run_name: str
    run_id: str | None = None
    data_root: Path | None = None
    seed: int = 0
    dp: PositiveInt | None = None
    gpus_per_node: PositiveInt = 8
    dtype: Literal["bfloat16", "float32"] = "bfloat16"
    attention_implementation: Literal["flash", "xla", "mosaic"] = "flash"
    global_batch: PositiveInt
    num_iterations: PositiveInt
    warmup_iters: int = 0
    learning_rate: PositiveFloat
    learning_rate_decay_frac: float = 0.1
    weight_decay: float = 0.1
    grad_clip: float | None = 1.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    log_every: PositiveInt = 100
    val_every: PositiveInt = 1000
    val_steps: PositiveInt = 20
    save_every: PositiveInt = 1000
    keep_last: PositiveInt = 2
    model: PretrainModelConfig
    data_layout: Literal["documents", "unsegmented_tokens"] = "unsegmented_tokens"
    data: LMDatasetRef = Field(default_factory=SyntheticZipfDataset)
    val_data: LMDatasetRef | None = Field(default_factory=lambda: SyntheticZipfDataset(seed=1))
    """`None`: validate on the first rows of the TRAIN data (in-distribution monitoring, not validation)."""
    wandb: WandbConfig | None = None


def lr_at(cfg: PretrainConfig, it: int) -> float:
    if it < cfg.warmup_iters:
        return cfg.learning_rate * (it + 1) / cfg.warmup_iters
    frac = (it - cfg.warmup_iters) / max(1, cfg.num_iterations - cfg.warmup_iters)
    lo = cfg.learning_rate * cfg.learning_rate_decay_frac
    return lo + 0.5 * (cfg.learning_rate - lo) * (1 + math.cos(math.pi * min(frac, 1.0)))


# ---- resumable trainer state ------------------------------------------------------------------------

def _state_files(entry: Path) -> list[Path]:
    return sorted((entry / "ckpts").glob("state_step_*.pt"), key=lambda p: int(re.findall(r"\d+", p.stem)[-1]))


def _prune(files: list[Path], keep_last: int) -> None:
    for old in files[:-keep_last]:
        old.unlink(missing_ok=True)


def save_train_state(entry: Path, step: int, weights: dict[str, torch.Tensor], opt: torch.optim.Optimizer,
                     keep_last: int) -> None:
    """fp32 masters + optimizer moments after `step` iterations, written whole (temp file, then rename); only the
    newest `keep_last` are kept (param_decomp/pretrain/train.py:192-215, `LatestN`)."""
    d = entry / "ckpts"
    d.mkdir(parents=True, exist_ok=True)
    tmp = d / f".state_step_{step}.pt.tmp"
    torch.save({"step": step, "weights": {k: v.detach().cpu() for k, v in weights.items()},
                "optimizer": opt.state_dict()}, tmp)
    os.replace(tmp, d / f"state_step_{step}.pt")
    _prune(_state_files(entry), keep_last)


def restore_latest_train_state(entry: Path, weights: dict[str, torch.Tensor], opt: torch.optim.Optimizer) -> int:
    """Loads the newest readable trainer state in place and returns its step; 0 when there is none."""
    for f in reversed(_state_files(entry)):
        try:
            blob = torch.load(f, map_location="cpu", weights_only=False)
        except Exception:  # noqa: BLE001  a file cut short by a kill: fall back to the one before
            continue
        with torch.no_grad():
            for k, v in weights.items():
                v.copy_(blob["weights"][k])
        opt.load_state_dict(blob["optimizer"])
        return int(blob["step"])
    return 0


def _prune_model_snapshots(entry: Path, keep_last: int) -> None:
    files = sorted(entry.glob("model_step_*.safetensors"), key=lambda p: int(re.findall(r"\d+", p.stem)[-1]))
    _prune(files, keep_last)


class _SigtermFlag:
    """SIGTERM sets a flag for the loop to read at an iteration boundary; the previous handler comes back on exit.
    Installed only from the main thread (signal handlers cannot be set elsewhere)."""

    def __init__(self) -> None:
        self._event = threading.Event()
        self._previous: Any = None

    def __enter__(self) -> "_SigtermFlag":
        if threading.current_thread() is threading.main_thread():
            self._previous = signal.signal(signal.SIGTERM, lambda *_: self._event.set())
        return self

    def __exit__(self, *exc: Any) -> None:
        if self._previous is not None:
            signal.signal(signal.SIGTERM, self._previous)

    def is_set(self) -> bool:
        return self._event.is_set()


class _DataParallel:
    """One process per device over `torch.distributed`: every rank reads its rows of the global batch and the
    gradients are averaged in one flat all-reduce per step."""

    def __init__(self, cfg: PretrainConfig, device: str) -> None:
        import torch.distributed as dist

        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1")) if cfg.dp is not None else 1
        self.rank = 0
        if cfg.dp is not None:
            assert self.world == cfg.dp, f"config says dp={cfg.dp}, the launch has WORLD_SIZE={self.world}"
        if self.world > 1:
            if not dist.is_initialized():
                dist.init_process_group("nccl" if device.startswith("cuda") else "gloo")
            self.rank = dist.get_rank()
        assert cfg.global_batch % self.world == 0, (cfg.global_batch, self.world)

    def average_gradients(self, params: list[torch.Tensor]) -> None:
        if self.world == 1:
            return
        flat = torch.cat([p.grad.reshape(-1) for p in params])
        self.dist.all_reduce(flat)
        flat.div_(self.world)
        off = 0
        for p in params:
            n = p.numel()
            p.grad.copy_(flat[off:off + n].view_as(p))
            off += n

    def mean(self, value: float, device: str) -> float:
        if self.world == 1:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=device if device.startswith("cuda") else "cpu")
        self.dist.all_reduce(t)
        return float(t) / self.world

    def barrier(self) -> None:
        if self.world > 1:
            self.dist.barrier()


def pretrain(cfg: PretrainConfig, data_root: Path | None = None, run_id: str | None = None, project: str = "spd",
             device: str = "cpu", max_iterations: int | None = None) -> Path:
    """Trains (or resumes: the newest trainer state under `<entry>/ckpts` is picked up) and returns the cache
    entry directory. SIGTERM saves the trainer state at the next iteration boundary and returns.
    Parity: param_decomp/pretrain/train.py:263-495."""
    from param_decomp_b200.data.shards import ShardServer
    from param_decomp_b200.data.synthetic import ZipfTokenSource

    data_root = data_root if data_root is not None else cfg.data_root
    assert data_root is not None, "data_root: give it in the config or at entry"
    run_id = run_id or cfg.run_id or "t-00000000"
    dp = _DataParallel(cfg, device)
    log = get_logger(dp.rank)
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

    train_src = source(cfg.data, 0)
    val_src = source(cfg.val_data, 1) if cfg.val_data is not None else source(cfg.data, 0)
    params = list(weights.values())
    decay = [p for p in params if p.dim() >= 2]
    no_decay = [p for p in params if p.dim() < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": cfg.weight_decay},
                             {"params": no_decay, "weight_decay": 0.0}], lr=cfg.learning_rate,
                            betas=(cfg.adam_beta1, cfg.adam_beta2))
    entry = Path(data_root) / "pretrain_cache" / f"{project}-{run_id}"
    start = restore_latest_train_state(entry, weights, opt)
    if start:
        log.info("pretrain resumed from iteration %d", start)
    sink = MetricsSink.for_run(entry, dp.rank, cfg.wandb, cfg.run_name, cfg.model_dump(mode="json"))

    def loss_on(batch) -> torch.Tensor:
        cls = qwen35.Qwen35DecomposedModel if hybrid else tf.TransformerDecomposedModel
        model = cls(arch, {k: v.to(dtype) for k, v in weights.items()}, {}, backend="eager_torch",
                    attention="xla" if device == "cpu" else cfg.attention_implementation)
        toks = batch.tokens.to(device)
        out = model._run(tf.LMBatch(toks[:, :-1], None if batch.segment_ids is None else batch.segment_ids[:, :-1].to(device)),
                         None, None, (), want_taps=False)
        logits = model.logits(out.output).float()
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]), toks[:, 1:].reshape(-1).long())

    def snapshot(step: int) -> None:
        if dp.rank == 0:
            snap = {k: v.detach().to(torch.bfloat16 if cfg.dtype == "bfloat16" else torch.float32) for k, v in weights.items()}
            (save_qwen35_cache if hybrid else save_simple_mlp_cache)(entry, arch, snap, step)
            _prune_model_snapshots(entry, 1)  # the cache entry holds exactly one hand-off snapshot, as its readers expect
            save_train_state(entry, step, weights, opt, cfg.keep_last)
        dp.barrier()

    n_iter = min(cfg.num_iterations, max_iterations or cfg.num_iterations)
    last_log = (start, time.perf_counter())
    with _SigtermFlag() as preempt:
        for it in range(start, n_iter):
            for g in opt.param_groups:
                g["lr"] = lr_at(cfg, it)
            loss = loss_on(train_src.batch(it, cfg.global_batch, dp.rank, dp.world))
            opt.zero_grad(set_to_none=True)
            loss.backward()
            dp.average_gradients(params)
            if cfg.grad_clip:
                torch.nn.utils.clip_grad_norm_(params, cfg.grad_clip)
            opt.step()
            last = it == n_iter - 1
            if it % cfg.log_every == 0 or last:
                mean_loss = dp.mean(float(loss.detach()), device)
                now = time.perf_counter()
                step_time = (now - last_log[1]) / max(1, it - last_log[0]) if it > last_log[0] else 0.0
                last_log = (it, now)
                sink.log(it, {"loss": mean_loss, "lr": lr_at(cfg, it), "step_time_s": step_time}, prefix="pretrain/")
                log.info("pretrain it %d loss %.4f", it, mean_loss)
            if (it + 1) % cfg.val_every == 0 or last:
                with torch.no_grad():  # the fixed evaluation set: the first `val_steps` batches, the same at every eval
                    val = sum(float(loss_on(val_src.batch(i, cfg.global_batch, dp.rank, dp.world)))
                              for i in range(cfg.val_steps)) / cfg.val_steps
                sink.log(it, {"val_loss": dp.mean(val, device)}, prefix="pretrain/")
            stop = preempt.is_set()
            if dp.world > 1:  # every rank takes the same branch
                flag = torch.tensor([int(stop)], device=device if device.startswith("cuda") else "cpu")
                dp.dist.all_reduce(flag, op=dp.dist.ReduceOp.MAX)
                stop = bool(flag.item())
            if (it + 1) % cfg.save_every == 0 or last or stop:
                snapshot(it + 1)
            if stop:
                log.info("pretrain preempted after iteration %d; state saved", it + 1)
                break
    sink.close()
    return entry


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("config", type=Path)
    ap.add_argument("--data-root", "--data_root", type=Path, default=None)
    ap.add_argument("--run-id", "--run_id", type=str, default=None)
    ap.add_argument("--device", type=str, default=None)
    args = ap.parse_args()
    device = args.device
    if device is None:
        device = f"cuda:{os.environ.get('LOCAL_RANK', '0')}" if torch.cuda.is_available() else "cpu"
    if device.startswith("cuda"):
        torch.cuda.set_device(device)
    print(pretrain(PretrainConfig.from_file(args.config), args.data_root, args.run_id, device=device))


if __name__ == "__main__":
    main()
