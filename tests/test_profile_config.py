"""Profiling runs derived from a full config, the `runtime.profiling` keys of the reference, and the step profiler's
bracketing of the captured steps."""
import subprocess
import sys

import pytest
import yaml

from param_decomp_b200.config.experiments import LMExperimentConfig, RuntimeConfig
from param_decomp_b200.core.run import StepProfiler
from param_decomp_b200.experiments.lm.profile_config import ProfileShape, derive_profile

BASE = "param_decomp_b200/experiments/configs/lm_llama4l_c4096.yaml"


def test_derived_profile_validates_and_is_cut_down():
    raw = yaml.safe_load(open(BASE).read())
    shape = ProfileShape(layers=2, batch_size=16, replicate=1, fsdp=2, tp=1, steps=12, profile_steps=3, sharding="zero1")
    out = derive_profile(raw, shape)
    cfg = LMExperimentConfig.model_validate(out)
    assert cfg.decomposition.sites.layers.model_dump() == {"kind": "range", "start": 0, "end": 2}
    assert (cfg.pd.batch_size, cfg.pd.steps, cfg.runtime.sharding) == (16, 12, "zero1")
    assert cfg.runtime.profiling.kind == "ad_hoc" and cfg.runtime.profiling.steps == 3
    assert cfg.run_name == "profile-2l-b16-r1-f2-t1-semantic-zero1"
    assert raw["pd"]["batch_size"] != 16, "the base mapping must not be edited"
    with pytest.raises(AssertionError):
        ProfileShape(layers=2, batch_size=16, replicate=1, fsdp=2, tp=1, steps=2, profile_steps=3, sharding="owner")
    raw["decomposition"]["sites"]["layers"] = {"kind": "range", "start": 0, "end": 1}
    with pytest.raises(AssertionError, match="extend"):
        derive_profile(raw, shape)


def test_cli_refuses_to_overwrite(tmp_path):
    out = tmp_path / "p.yaml"
    cmd = [sys.executable, "-m", "param_decomp_b200.experiments.lm.profile_config", BASE, str(out), "--layers", "1",
           "--batch-size", "8", "--replicate", "1", "--fsdp", "1", "--tp", "1", "--steps", "8", "--profile-steps", "2",
           "--sharding", "ddp", "--profiling", "nsight_systems"]
    assert subprocess.run(cmd, capture_output=True).returncode == 0
    cfg = LMExperimentConfig.from_file(out)
    assert (cfg.runtime.profiling.kind, cfg.runtime.profiling.warmup_steps, cfg.runtime.profiling.capture_steps) == (
        "nsight_systems", 6, 2)
    assert subprocess.run(cmd, capture_output=True).returncode != 0


def test_profiling_keys_of_the_reference_parse():
    base = {"mesh": {"replicate": 1, "fsdp": 1, "tp": 1}, "sharding": "ddp"}
    assert RuntimeConfig.model_validate({**base, "profiling": {"kind": "ad_hoc", "steps": 4}}).profiling.steps == 4
    assert RuntimeConfig.model_validate({**base, "profiling": {"kind": "ad_hoc", "n_steps": 2}}).profiling.steps == 2
    ns = RuntimeConfig.model_validate({**base, "profiling": {"kind": "nsight_systems", "version": "2026.4.1",
                                                             "warmup_steps": 7, "capture_steps": 2}}).profiling
    assert (ns.warmup_steps, ns.capture_steps) == (7, 2)
    with pytest.raises(Exception):
        RuntimeConfig.model_validate({**base, "profiling": {"kind": "ad_hoc", "steps": 0}})


def test_step_profiler_brackets_exactly_the_captured_steps(tmp_path):
    prof = StepProfiler("trace", warmup=2, n_steps=3, run_dir=tmp_path)
    stops = []
    for step in range(10):
        prof.before_step(step)
        if prof.after_step(step):
            stops.append(step)
            break
    assert stops == [4] and prof.captured == [2, 3, 4]
    assert (tmp_path / "profile" / "trace.json").stat().st_size > 0
    ranged = StepProfiler("cuda_profiler_range", warmup=1, n_steps=1, run_dir=None)  # no device: only the bookkeeping
    ranged.before_step(0)
    assert not ranged.after_step(0)
    ranged.before_step(1)
    assert ranged.after_step(1) and ranged.captured == [1]


def test_ad_hoc_profiling_run_traces_and_leaves(tmp_path):
    """`runtime.profiling: {kind: ad_hoc, steps: 2}` through the LM root: warm-up, two traced steps, exit."""
    import copy

    import __graft_entry__ as ge
    from param_decomp_b200.experiments.lm.training import train_lm

    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"].update(backend="eager_torch", sharding="ddp", profiling={"kind": "ad_hoc", "steps": 2})
    c["target"].update(weights_dtype="float32", attention_implementation="xla")
    c["data"]["seq_len"] = 8
    c["pd"].update(batch_size=4, steps=50)
    c["eval"] = None
    res = train_lm(LMExperimentConfig.model_validate(c), tmp_path, device="cpu")
    assert (res.run_dir / "profile" / "trace.json").stat().st_size > 0
    assert res.final_step == 4  # two warm-up steps (nothing is recorded on this backend) and the two traced ones


def test_profiled_run_leaves_a_memory_ledger_with_phase_marks(tmp_path):
    import copy
    import subprocess
    import sys

    import __graft_entry__ as ge
    from param_decomp_b200.core.debug.memory_ledger import Ledger
    from param_decomp_b200.experiments.lm.training import train_lm

    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"].update(backend="eager_torch", sharding="ddp", profiling={"kind": "ad_hoc", "steps": 1})
    c["target"].update(weights_dtype="float32", attention_implementation="xla")
    c["data"]["seq_len"] = 8
    c["pd"].update(batch_size=4, steps=50)
    c["eval"] = None
    res = train_lm(LMExperimentConfig.model_validate(c), tmp_path, device="cpu")
    led = Ledger.load(res.run_dir / "profile" / "memory_ledger.json")
    names = [m.name for m in led.marks]
    assert names[0] == "step_begin" and names[-1] == "step_end" and {"ci_fn", "losses", "optimizer"} <= set(names)
    assert all(m.allocated > 0 and m.top_tensors for m in led.marks)
    out = subprocess.run([sys.executable, "-m", "param_decomp_b200.core.debug.memory_ledger", str(res.run_dir), "--top", "3"],
                         capture_output=True, text=True)
    assert out.returncode == 0 and "peak" in out.stdout and "largest live tensors" in out.stdout
    import json

    counted = json.loads((res.run_dir / "profile" / "census.json").read_text())
    assert set(counted) == {"native_launches", "native", "collectives", "collective_bytes"}
