"""The YAML run-config schema (pydantic, torch-free apart from `schedule.as_tensor`)."""

from param_decomp_b200.config.evals import EvalConfig
from param_decomp_b200.config.experiments import (
    LMExperimentConfig,
    LMTargetedExperimentConfig,
    ResidMLPExperimentConfig,
    TMSExperimentConfig,
)
from param_decomp_b200.config.run import Cadence, PDConfig, TargetedPDConfig
from param_decomp_b200.config.schedule import ScheduleConfig, get_scheduled_value

__all__ = [
    "Cadence", "EvalConfig", "LMExperimentConfig", "LMTargetedExperimentConfig", "PDConfig",
    "ResidMLPExperimentConfig", "ScheduleConfig", "TMSExperimentConfig", "TargetedPDConfig",
    "get_scheduled_value",
]
