"""Open a finished LM decomposition for read-only analysis.

`run_metadata` reads what can be known without a checkpoint (the pinned launch config: target
structure, sites, CI function, data, seed). `open_run` rebuilds the target on the device the CALLER
names, restores the component weights and the CI function of one checkpoint step, and returns them
with no optimizer or training state. `open_target_and_components` skips the CI function for consumers
that substitute component activations themselves.
`load_deliverable` resolves target structure, CI definition, datasets and seed without touching a checkpoint.
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


@dataclass(frozen=True)
class ResolvedLMData:
    train_dir: Path | None  # None: a synthetic source (no files)
    eval_dir: Path | None
    layout: str
    seq_len: int


@dataclass(frozen=True)
class ResolvedDeliverable:
    """What a finished run fixed, for offline consumers that never restore its checkpoint: the target's
    architecture, the decomposed sites with their dimensions and component counts, the CI function's definition
    (as authored, plus the widths of the taps it reads), the datasets and the seed."""

    arch: Any
    sites: tuple
    ci_fn: Any
    ci_tap_widths: dict[str, int]
    data: ResolvedLMData
    seed: int


def load_deliverable(run_dir: Path, data_root: Path | None = None) -> ResolvedDeliverable:
    """Resolve the stable facts of a run from its pinned launch config alone (stored configs are migrated to the
    current schema first). No tensor of the target is materialised for `random_init` targets (their weights are
    shaped on the meta device); pretrained / snapshot targets read their architecture from the cache entry.
    Parity: param_decomp/experiments/lm/deliverable.py:36-90."""
    from param_decomp_b200.config import experiments as X
    from param_decomp_b200.core.ci_fn.resolve import tap_widths_for
    from param_decomp_b200.experiments.lm.build import build_lm_run
    from param_decomp_b200.formats.dataset_store import DatasetDir, NamedDataset, resolve_dataset_ref

    cfg = load_config(Path(run_dir))
    cfg = cfg.model_copy(update={"runtime": cfg.runtime.model_copy(update={"backend": "eager_torch"})})
    meta = isinstance(cfg.target.spec, X.RandomInitTarget)
    if meta:
        with torch.device("meta"):
            run = build_lm_run(cfg, data_root, "meta")
    else:
        run = build_lm_run(cfg, data_root, "cpu")
    model = run.model
    sites = tuple(getattr(model, "global_sites", model.sites))
    ci_cfg = cfg.decomposition.ci
    widths: dict[str, int] = {}
    sel = getattr(ci_cfg, "input_tap", None)
    if sel is not None and hasattr(model, "layer_of_site"):
        layers = sorted({model.layer_of_site(s.name) for s in sites})
        widths = tap_widths_for(model, layers, sel)
    else:  # per-site CI functions read each site's own input
        widths = {s.name: s.d_in for s in sites}

    def resolved(ref) -> Path | None:
        if isinstance(ref, (NamedDataset, DatasetDir)):
            assert data_root is not None, "dataset references resolve under --data-root"
            return resolve_dataset_ref(ref, Path(data_root))
        return None

    data = ResolvedLMData(resolved(cfg.data.train), resolved(cfg.data.eval), cfg.data.layout, cfg.data.seq_len)
    return ResolvedDeliverable(run.arch, sites, ci_cfg, widths, data, cfg.pd.seed)


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
