import glob

import pytest
import yaml

from param_decomp_b200.config import (LMExperimentConfig, ResidMLPExperimentConfig, ScheduleConfig,
                                      TMSExperimentConfig, get_scheduled_value)
from param_decomp_b200.config.run import flatten_typed_lists
from param_decomp_b200.formats import ComponentKey
from pathlib import Path

OURS = Path(__file__).resolve().parents[1] / "param_decomp_b200" / "experiments" / "configs"


def test_reference_yamls_parse(reference_configs):
    n = 0
    for sub, cls in (("tms", TMSExperimentConfig), ("resid_mlp", ResidMLPExperimentConfig), ("lm", LMExperimentConfig)):
        for f in sorted(glob.glob(str(reference_configs / sub / "configs" / "*.yaml"))):
            cls.from_file(f)
            n += 1
    assert n >= 10


def test_shipped_yamls_parse_and_roundtrip(tmp_path):
    for f in sorted(OURS.glob("*.yaml")):
        cls = {"tms": TMSExperimentConfig, "res": ResidMLPExperimentConfig}.get(f.name[:3], LMExperimentConfig)
        cfg = cls.from_file(f)
        cfg.to_file(tmp_path / f.name)
        assert cls.from_file(tmp_path / f.name) == cfg


def test_extra_keys_forbidden():
    with pytest.raises(Exception):
        ScheduleConfig.model_validate({"max_val": 1.0, "points": [{"at": 0, "frac": 1}, {"at": 1, "frac": 1}], "x": 1})


def test_schedule_knots():
    s = ScheduleConfig.model_validate({"max_val": 2.0, "points": [
        {"at": 0.0, "frac": 0.0}, {"at": 0.5, "frac": 1.0}, {"at": 1.0, "frac": 0.5, "interp": "cosine"}]})
    assert get_scheduled_value(0, 101, s) == 0.0
    assert get_scheduled_value(25, 101, s) == pytest.approx(1.0)
    assert get_scheduled_value(50, 101, s) == pytest.approx(2.0)
    assert get_scheduled_value(75, 101, s) == pytest.approx(2.0 * 0.75)
    assert get_scheduled_value(100, 101, s) == pytest.approx(1.0)
    assert get_scheduled_value(101, 101, s) == pytest.approx(1.0)  # one past the end holds
    hold = ScheduleConfig.model_validate({"max_val": 1.0, "points": [
        {"at": 0.0, "frac": 1.0}, {"at": 0.5, "frac": 0.1, "interp": "hold"}, {"at": 1.0, "frac": 0.1}]})
    assert get_scheduled_value(49, 101, hold) == 1.0 and get_scheduled_value(50, 101, hold) == pytest.approx(0.1)
    const = ScheduleConfig.model_validate("1e-4")
    assert const.is_constant and get_scheduled_value(3, 10, const) == pytest.approx(1e-4)


def test_schedule_validation():
    for bad in ([{"at": 0.1, "frac": 1}, {"at": 1, "frac": 1}], [{"at": 0, "frac": 0.5}, {"at": 1, "frac": 0.5}]):
        with pytest.raises(Exception):
            ScheduleConfig.model_validate({"max_val": 1.0, "points": bad})


def test_loss_list_rules():
    base = yaml.safe_load((OURS / "tms_5-2.yaml").read_text())
    base["pd"]["loss_metrics"] = [m for m in base["pd"]["loss_metrics"] if m["type"] != "FaithfulnessLoss"]
    with pytest.raises(Exception):
        TMSExperimentConfig.model_validate(base)


def test_component_key():
    k = ComponentKey("h.0.attn.q_proj", 17)
    assert ComponentKey.decode(k.encoded()) == k
    for bad in ("x:01", "nocolon", ":3", "a b:1"):
        with pytest.raises(ValueError):
            ComponentKey.decode(bad)


def test_flatten_typed_lists():
    out = flatten_typed_lists({"pd": {"loss_metrics": [{"type": "FaithfulnessLoss", "coeff": 2.0}], "seed": 1}})
    assert out["pd.loss_metrics.Faith.coeff"] == 2.0 and "loss_metrics" not in out["pd"]


def test_sequence_parallel_is_accepted_for_dense_targets_and_refused_for_expert_splits():
    """`runtime.sequence_sharding: sequence_parallel` parses; dense transformer targets run it (position-sharded
    residual of the masked passes over the tp group, `tests/test_tp_engine_cpu.py`), mixture-of-experts targets,
    whose tp axis splits experts, refuse it at start-up instead of ignoring it."""
    import copy

    import pytest

    import __graft_entry__ as ge
    from param_decomp_b200.config.experiments import LMExperimentConfig
    from param_decomp_b200.experiments.lm.training import check_runtime_supported

    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"]["sequence_sharding"] = "sequence_parallel"
    check_runtime_supported(LMExperimentConfig.model_validate(c))
    m = copy.deepcopy(c)
    m["target"]["spec"]["arch"] = {"family": "moe", "n_layer": 2, "d_model": 32, "n_head": 2, "d_ff": 16,
                                   "vocab_size": 100, "n_experts": 4, "experts_per_token": 2}
    m["decomposition"]["sites"] = {"kind": "moe", "layers": {"kind": "all"},
                                   "cs": {"q": 8, "experts_gate": 16, "experts_up": 16, "experts_down": 16}}
    with pytest.raises(NotImplementedError):
        check_runtime_supported(LMExperimentConfig.model_validate(m))
    c["runtime"]["sequence_sharding"] = "replicate"
    check_runtime_supported(LMExperimentConfig.model_validate(c))
