"""Causal-importance functions: networks mapping clean activations to per-component importances."""

from param_decomp_b200.core.ci_fn.interface import CI, CIFn, TapSpec, squash
from param_decomp_b200.core.ci_fn.mlp import GlobalMLPCIFn, LayerwiseMLPCIFn, SiteMLP

__all__ = ["CI", "CIFn", "TapSpec", "squash", "GlobalMLPCIFn", "LayerwiseMLPCIFn", "SiteMLP"]
