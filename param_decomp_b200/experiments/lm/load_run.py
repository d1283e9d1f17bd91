"""Open a finished LM decomposition for read-only analysis.

`run_metadata` reads what can be known without a checkpoint (the pinned launch config: target
structure, sites, CI function, data, seed). `open_run` rebuilds the target on the device the CALLER
names, restores the component weights and the CI function of one checkpoint step, and returns them
with no optimizer or training state. `open_target_and_components` skips the CI function for consumers
that substitute component activations themselves.
Parity: param_decomp/experiments/lm/load_run.py:88-183,265-285,434-..., deliverable.py.
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any

import torch
import yaml
from torch import nn

from param_decomp_b200.config.experiments import LMExperimentConfig, LMTargetedExperimentConfig
from param_decomp_b200.core import checkpoint
from param_decomp_b200.core.components import ComponentStacks, ComputeWeights, prepare_compute_weights


@dataclass
class RunMetadata:
    run_dir: Path
    config: LMExperimentConfig | LMTargetedExperimentConfig
    steps_saved: list[int]
    sites: dict[str, int]  # per-kind component counts as authored


@dataclass
class LoadedRun:
    config: Any
    model: Any
    components: ComponentStacks
    ci_fn: nn.Module | None
    step: int

    def compute_weights(self) -> ComputeWeights:
        return prepare_compute_weights(self.components, self.model.compute_dtype).detached()


def load_config(run_dir: Path) -> LMExperimentConfig | LMTargetedExperimentConfig:
    raw = yaml.safe_load((Path(run_dir) / "launch_config.yaml").read_text())
    cls = LMTargetedExperimentConfig if "nontarget" in raw else LMExperimentConfig
    return cls.model_validate(raw)


def run_metadata(run_dir: Path) -> RunMetadata:
    cfg = load_config(run_dir)
    return RunMetadata(Path(run_dir), cfg, checkpoint.list_steps(Path(run_dir)), dict(cfg.decomposition.sites.cs))


def _step(run_dir: Path, step: int | None) -> int:
    steps = checkpoint.list_steps(run_dir)
    assert steps, f"{run_dir} holds no checkpoint"
    if step is None:
        return steps[-1]
    assert step in steps, f"step {step} was not saved (have {steps})"
    return step


def open_target_and_components(run_dir: Path, data_root: Path | None = None, step: int | None = None,
                               device: str | torch.device = "cpu", backend: str = "eager_torch") -> LoadedRun:
    from param_decomp_b200.experiments.lm.build import build_lm_run

    run_dir = Path(run_dir)
    cfg = load_config(run_dir)
    cfg = cfg.model_copy(update={"runtime": cfg.runtime.model_copy(update={"backend": backend})})
    run = build_lm_run(cfg, data_root, device)
    comps = ComponentStacks(run.model.sites).to(device)
    s = _step(run_dir, step)
    checkpoint.restore_components(run_dir, s, comps)
    return LoadedRun(cfg, run.model, comps, None, s)


def open_run(run_dir: Path, data_root: Path | None = None, step: int | None = None,
             device: str | torch.device = "cpu", backend: str = "eager_torch") -> LoadedRun:
    from param_decomp_b200.experiments.lm.build import build_lm_run

    run_dir = Path(run_dir)
    cfg = load_config(run_dir)
    cfg = cfg.model_copy(update={"runtime": cfg.runtime.model_copy(update={"backend": backend})})
    run = build_lm_run(cfg, data_root, device)
    comps = ComponentStacks(run.model.sites).to(device)
    ci_fn = run.ci_fn.to(device)
    s = _step(run_dir, step)
    checkpoint.restore_decomposition(run_dir, s, comps, ci_fn)
    for p in list(comps.parameters()) + list(ci_fn.parameters()):
        p.requires_grad_(False)
    return LoadedRun(cfg, run.model, comps, ci_fn, s)
