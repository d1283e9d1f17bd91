"""Knot schedules: `value(step) = max_val * frac(t)`, `t = step / (total_steps - 1)`.

Parity: param_decomp/core/schedule.py:18-102 (knots `{at, frac, interp}`, interp linear | cosine |
hold, a bare float is the constant schedule, `at=1.0` lands on the last step). One evaluator serves
host code and tensors: `fraction_at` takes a Python float or a 0-d tensor.
"""

from __future__ import annotations

import math
from typing import Literal, Self

import torch
from pydantic import PositiveFloat, model_validator

from param_decomp_b200.formats.base import BaseConfig, Probability

Interp = Literal["linear", "cosine", "hold"]


class Knot(BaseConfig):
    at: Probability
    frac: Probability
    interp: Interp = "linear"  # how the curve travels from the previous knot to this one


class ScheduleConfig(BaseConfig):
    max_val: PositiveFloat
    points: tuple[Knot, ...]

    @model_validator(mode="before")
    @classmethod
    def _bare_number(cls, data: object) -> object:
        if isinstance(data, str):
            data = float(data)  # YAML reads `1e-4` (no dot) as a string
        if isinstance(data, (int, float)) and not isinstance(data, bool):
            return {"max_val": data, "points": ({"at": 0.0, "frac": 1.0}, {"at": 1.0, "frac": 1.0})}
        return data

    @model_validator(mode="after")
    def _check(self) -> Self:
        ats = [k.at for k in self.points]
        assert len(ats) >= 2, f"a schedule needs >= 2 knots: {ats}"
        assert ats[0] == 0.0 and ats[-1] == 1.0, f"knots must span at=0..1, got {ats}"
        assert all(a < b for a, b in zip(ats, ats[1:])), f"knot positions must increase: {ats}"
        assert any(k.frac == 1.0 for k in self.points), "some knot must attain frac=1.0"
        return self

    @classmethod
    def constant(cls, value: float) -> "ScheduleConfig":
        return cls.model_validate(value)

    @property
    def is_constant(self) -> bool:
        return all(k.frac == 1.0 for k in self.points)


def run_fraction(step: int, total_steps: int) -> float:
    return min(step / (total_steps - 1), 1.0) if total_steps > 1 else 0.0


def fraction_at(cfg: ScheduleConfig, t: float) -> float:
    """Shape of the curve at normalized time `t` in [0, 1]. A knot owns the instant it names."""
    pts = cfg.points
    for i in range(1, len(pts)):
        prev, knot = pts[i - 1], pts[i]
        if t < knot.at or i == len(pts) - 1:
            u = (t - prev.at) / (knot.at - prev.at)
            if knot.interp == "linear":
                return prev.frac + (knot.frac - prev.frac) * u
            if knot.interp == "cosine":
                return prev.frac + (knot.frac - prev.frac) * 0.5 * (1.0 - math.cos(math.pi * u))
            return knot.frac if u >= 1.0 else prev.frac
    raise AssertionError("unreachable")


def get_scheduled_value(step: int, total_steps: int, cfg: ScheduleConfig) -> float:
    assert 0 <= step <= total_steps and total_steps > 0, (step, total_steps)
    return cfg.max_val * fraction_at(cfg, run_fraction(step, total_steps))


def scheduled_or_constant(value: "float | ScheduleConfig", step: int, total_steps: int) -> float:
    """Loss coefficients may be a bare float (0.0 allowed) or a schedule."""
    if isinstance(value, ScheduleConfig):
        return get_scheduled_value(step, total_steps, value)
    return float(value)


def as_tensor(value: float, device: torch.device | str = "cpu") -> torch.Tensor:
    return torch.tensor(value, dtype=torch.float32, device=device)
