"""Artifact-level schemas shared by trainers and analysis readers; imports nothing above it."""

from param_decomp_b200.formats.base import BaseConfig, Probability
from param_decomp_b200.formats.keys import ComponentKey, SiteId

__all__ = ["BaseConfig", "Probability", "ComponentKey", "SiteId"]
