"""`python -m param_decomp_b200.experiments.lm.profile_config base.yaml out.yaml --layers 2 --batch-size 16
--replicate 1 --fsdp 2 --tp 1 --steps 12 --profile-steps 3 --sharding owner`

Derives a profiling run from one full LM config, so profiled shapes stay a function of the config people
actually train: the first `layers` blocks' sites, a smaller batch, another mesh and placement, a handful of steps
and `runtime.profiling: ad_hoc`. Hidden-activation reconstruction auxiliaries are re-pointed at the residual
boundaries that still exist. Both the base and the derived config must validate; an existing output is never
overwritten. `--profiling nsight_systems` brackets the captured steps for an external profiler instead.

Parity: param_decomp/experiments/lm/profile_config.py:1-125.
"""

from __future__ import annotations

import argparse
import copy
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import yaml

from param_decomp_b200.config.experiments import LMExperimentConfig


@dataclass(frozen=True)
class ProfileShape:
    layers: int
    batch_size: int
    replicate: int
    fsdp: int
    tp: int
    steps: int
    profile_steps: int
    sharding: str
    profiling: str = "ad_hoc"

    def __post_init__(self) -> None:
        for name in ("layers", "batch_size", "replicate", "fsdp", "tp", "steps", "profile_steps"):
            v = getattr(self, name)
            assert isinstance(v, int) and v > 0, (name, v)
        assert self.profile_steps <= self.steps, (self.profile_steps, self.steps)
        assert self.sharding in ("owner", "zero1", "ddp"), self.sharding
        assert self.profiling in ("ad_hoc", "nsight_systems"), self.profiling

    @property
    def run_name(self) -> str:
        return (f"profile-{self.layers}l-b{self.batch_size}-r{self.replicate}-f{self.fsdp}-t{self.tp}-"
                f"semantic-{self.sharding}")


def _mapping(value: object, where: str) -> dict[str, Any]:
    assert isinstance(value, dict), f"{where} must be a mapping"
    return value


def derive_profile(raw: dict[str, Any], shape: ProfileShape) -> dict[str, Any]:
    LMExperimentConfig.model_validate(raw)
    out = copy.deepcopy(raw)
    sites = _mapping(_mapping(out["decomposition"], "decomposition")["sites"], "decomposition.sites")
    layers = sites.get("layers", {"kind": "all"})
    kind = _mapping(layers, "decomposition.sites.layers").get("kind")
    if kind == "range":
        assert layers.get("start") == 0, "profile derivation needs all layers or a zero-based range"
        assert shape.layers <= layers["end"], "a profile cannot extend the base layer range"
    else:
        assert kind == "all", "profile derivation needs all layers or a zero-based range"
    sites["layers"] = {"kind": "range", "start": 0, "end": shape.layers}

    pd = _mapping(out["pd"], "pd")
    pd["batch_size"] = shape.batch_size
    pd["steps"] = shape.steps
    for loss in pd["loss_metrics"]:
        for aux in _mapping(loss, "pd.loss_metrics[]").get("auxiliaries", []):
            if _mapping(aux, "auxiliaries[]")["name"] == "hidden_acts_reconstruction":
                aux["comparisons"] = [{"capture": f"resid.{i}", "distance": "relative_squared_error"}
                                      for i in range(1, shape.layers + 1)]

    runtime = _mapping(out["runtime"], "runtime")
    runtime["mesh"] = {"replicate": shape.replicate, "fsdp": shape.fsdp, "tp": shape.tp}
    runtime["sharding"] = shape.sharding
    if shape.profiling == "ad_hoc":
        runtime["profiling"] = {"kind": "ad_hoc", "steps": shape.profile_steps}
    else:
        runtime["profiling"] = {"kind": "nsight_systems", "version": "2026.4.1",
                                "warmup_steps": shape.steps - shape.profile_steps, "capture_steps": shape.profile_steps}
    out["run_name"] = shape.run_name
    LMExperimentConfig.model_validate(out)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[1])
    ap.add_argument("base", type=Path)
    ap.add_argument("output", type=Path)
    for name in ("layers", "batch-size", "replicate", "fsdp", "tp", "steps", "profile-steps"):
        ap.add_argument(f"--{name}", type=int, required=True)
    ap.add_argument("--sharding", choices=("owner", "zero1", "ddp"), required=True)
    ap.add_argument("--profiling", choices=("ad_hoc", "nsight_systems"), default="ad_hoc")
    a = ap.parse_args()
    assert not a.output.exists(), f"refusing to overwrite {a.output}"
    shape = ProfileShape(a.layers, a.batch_size, a.replicate, a.fsdp, a.tp, a.steps, a.profile_steps, a.sharding,
                         a.profiling)
    derived = derive_profile(_mapping(yaml.safe_load(a.base.read_text()), str(a.base)), shape)
    a.output.write_text(yaml.safe_dump(derived, sort_keys=False))


if __name__ == "__main__":
    main()
