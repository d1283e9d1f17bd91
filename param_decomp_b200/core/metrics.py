"""`metrics.jsonl` sink, W&B mirror, step timing and run-directory files.

Every log call appends one line `{"step": s, "train/...": v, ...}` to `<run_dir>/metrics.jsonl`.
Train-step scalars are prefixed `train/`, evaluation scalars `eval/`; performance keys are
`train/perf/step_time_s`, `train/perf/elapsed_s`, `train/perf/eta_s`, `train/perf/tokens_per_s`,
`train/perf/mfu`, and CUDA memory stats. W&B failures never abort a run.

Parity: param_decomp/core/run.py:430-442 (`_METRIC_KEYS`), :480-663 (`MetricsSink`), :382-403
(safe W&B logging); core/training_performance.py:16-162; experiments/config.py:66-116 (run id,
`launch_config.yaml` pinning); core/log.py (rank-0 logger).
"""

from __future__ import annotations

import json
import logging
import math
import re
import secrets
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

import torch

LAUNCH_CONFIG_FILENAME = "launch_config.yaml"
METRICS_FILENAME = "metrics.jsonl"
NO_REENTRY_MARKER = "NO_CHECKPOINT_RUN_STARTED"
_RUN_ID = re.compile(r"^p-[0-9a-f]{8}$")


def get_logger(rank: int = 0) -> logging.Logger:
    log = logging.getLogger(f"param_decomp_b200.rank{rank}")
    if not log.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter(f"[%(asctime)s r{rank}] %(message)s", "%H:%M:%S"))
        log.addHandler(h)
        log.setLevel(logging.INFO if rank == 0 else logging.WARNING)
        log.propagate = False
    return log


def mint_run_id() -> str:
    return "p-" + secrets.token_hex(4)


def run_dir_for(data_root: Path, run_id: str) -> Path:
    assert _RUN_ID.match(run_id), f"run_id must be p-<8hex>, got {run_id!r}"
    return Path(data_root) / "runs" / run_id


def pin_launch_config(run_dir: Path, resolved_yaml: str) -> None:
    """First entry writes the resolved config; re-entry must present byte-identical text."""
    run_dir.mkdir(parents=True, exist_ok=True)
    pinned = run_dir / LAUNCH_CONFIG_FILENAME
    if pinned.exists():
        assert pinned.read_text() == resolved_yaml, (
            f"{pinned} differs from the invoked config: refusing to resume with a changed config"
        )
    else:
        pinned.write_text(resolved_yaml)


def to_float(v: Any) -> float:
    if isinstance(v, torch.Tensor):
        return float(v.detach().float().cpu())
    return float(v)


@dataclass
class MetricsSink:
    run_dir: Path
    rank: int = 0
    wandb_run: Any = None
    _fh: Any = None
    names: Any = None  # infra.metric_names.MetricNames: local keys -> the names the W&B mirror logs

    @classmethod
    def for_run(cls, run_dir: Path, rank: int = 0, wandb_cfg: Any = None, run_name: str = "",
                config_dict: dict | None = None) -> "MetricsSink":
        sink = cls(Path(run_dir), rank)
        if rank == 0:
            sink.run_dir.mkdir(parents=True, exist_ok=True)
            reentry = (sink.run_dir / METRICS_FILENAME).exists()
            sink._fh = open(sink.run_dir / METRICS_FILENAME, "a", buffering=1)
            if wandb_cfg is not None:
                from param_decomp_b200.infra.metric_names import MetricNames, validate_resume_schema

                pinned = sink.run_dir / LAUNCH_CONFIG_FILENAME
                if reentry and pinned.exists():  # a resumed run keeps the names it was started with
                    import yaml

                    validate_resume_schema(yaml.safe_load(pinned.read_text()) or {}, wandb_cfg.metric_schema)
                sink.names = MetricNames(wandb_cfg.metric_schema)
                sink.wandb_run = try_wandb_init(wandb_cfg, run_name, sink.run_dir, config_dict)
        return sink

    def log(self, step: int, scalars: dict[str, Any], prefix: str = "train/") -> dict[str, float]:
        """Writes one record and returns it as written. The file and the `legacy` W&B mirror use the reference's
        key spellings (`infra/reference_keys.py`); the `grouped` names are derived from the internal keys."""
        flat = {prefix + k: to_float(v) for k, v in scalars.items()}
        written = public_record(flat)
        if self.rank == 0 and self._fh is not None:
            self._fh.write(json.dumps({"step": step, **written}) + "\n")
            if self.wandb_run is not None:
                try:
                    grouped = self.names is not None and self.names.schema != "legacy"
                    self.wandb_run.log(self.names.record(flat) if grouped else written, step=step)
                except Exception as err:  # W&B trouble is never fatal
                    get_logger().warning("wandb.log failed: %s", err)
        return written

    def close(self) -> None:
        if self._fh is not None:
            self._fh.close()
            self._fh = None
        if self.wandb_run is not None:
            try:
                self.wandb_run.finish()
            except Exception:
                pass


def public_record(flat: dict[str, float]) -> dict[str, float]:
    """Internal keys -> the keys that are written (also what a run without a sink reports as its last metrics)."""
    from param_decomp_b200.infra.reference_keys import reference_keys

    return reference_keys(flat)


def try_wandb_init(cfg: Any, run_name: str, run_dir: Path, config_dict: dict | None) -> Any:
    try:
        import os

        import wandb

        if os.environ.get("WANDB_MODE", "") == "disabled":
            return None
        return wandb.init(project=cfg.project, entity=cfg.entity, group=cfg.group, tags=list(cfg.tags),
                          name=run_name, dir=str(run_dir), config=config_dict or {},
                          mode=os.environ.get("WANDB_MODE", "offline"))
    except Exception as err:
        get_logger().warning("wandb init failed (continuing without): %s", err)
        return None


def assert_all_finite(step: int, scalars: dict[str, float]) -> None:
    bad = {k: v for k, v in scalars.items() if isinstance(v, float) and not math.isfinite(v)
           and not k.endswith("eta_s")}
    if bad:
        raise FloatingPointError(f"non-finite training scalars at step {step}: {bad}")


@dataclass
class PerformanceTracker:
    """Wall/device step time, throughput and MFU between consecutive log calls."""

    total_steps: int
    units_per_step: int  # tokens (LM) or samples (toys) in the global batch
    flops_per_step: float = 0.0
    peak_flops: float = 0.0
    optimizer_flops_per_step: float = 0.0  # contraction FLOPs of the optimizers (Newton-Schulz), counted apart
    t_start: float = field(default_factory=time.perf_counter)
    t_last: float = field(default_factory=time.perf_counter)
    step_last: int = 0

    def tick(self, step: int) -> dict[str, float]:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        now = time.perf_counter()
        n = max(step - self.step_last, 1)
        dt = (now - self.t_last) / n
        self.t_last, self.step_last = now, step
        out = {
            "perf/step_time_s": dt,
            "perf/elapsed_s": now - self.t_start,
            "perf/runtime_s": now - self.t_start,
            "perf/n_completed_steps": float(step),
            "perf/eta_s": dt * max(self.total_steps - step, 0),
            "perf/tokens_per_s": self.units_per_step / dt if dt > 0 else 0.0,
        }
        if self.flops_per_step:
            out["perf/useful_model_flops"] = self.flops_per_step
            out["perf/useful_optimizer_flops"] = self.optimizer_flops_per_step
        if self.flops_per_step and self.peak_flops:
            out["perf/mfu"] = self.flops_per_step / dt / self.peak_flops
            out["perf/mfu_with_optimizer"] = (self.flops_per_step + self.optimizer_flops_per_step) / dt / self.peak_flops
        if torch.cuda.is_available():
            out["perf/cuda_mem_allocated_gb"] = torch.cuda.memory_allocated() / 2**30
            out["perf/cuda_mem_peak_gb"] = torch.cuda.max_memory_allocated() / 2**30
            out["mem/peak_gb_per_rank"] = torch.cuda.max_memory_allocated() / 1e9  # decimal GB, as the reference logs it
        return out


DEVICE_PEAK_BF16 = {"B200": 2.25e15, "H100": 989.4e12, "H200": 989.4e12}


def device_peak_flops() -> float:
    """Dense bf16 peak of the current device (datasheet), 0 if unknown."""
    if not torch.cuda.is_available():
        return 0.0
    name = torch.cuda.get_device_name()
    for key, val in DEVICE_PEAK_BF16.items():
        if key in name:
            return val
    return 0.0
