"""Every LM config shipped with the package passes the deviceless gate."""
from pathlib import Path

import pytest

from param_decomp_b200.config.experiments import LMExperimentConfig
from param_decomp_b200.experiments.lm import trace_check

CONFIGS = sorted(Path("param_decomp_b200/experiments/configs").glob("lm_*.yaml"))


@pytest.mark.parametrize("path", CONFIGS, ids=lambda p: p.stem)
def test_repo_lm_configs_trace(path):
    cfg = LMExperimentConfig.from_file(path)
    notes = trace_check.static_checks(cfg, 8)
    assert any("memory estimate" in n for n in notes)
    losses = trace_check.replica_step(cfg)
    assert "loss/total" in losses


def test_gate_refuses_a_mesh_that_does_not_match_the_launch():
    cfg = LMExperimentConfig.from_file(CONFIGS[0])
    with pytest.raises(AssertionError):
        trace_check.static_checks(cfg, 4)
