"""Eval-metric configs (`eval.metrics` of a run YAML) and the eval cadence.

Parity: param_decomp/core/configs.py:283-345,496-573; experiments/eval_config.py:89-129;
experiments/lm/eval_config.py. Each metric carries its tier (`slow`) as a ClassVar so YAML cannot
author it.
"""

from __future__ import annotations

from itertools import pairwise
from typing import Annotated, ClassVar, Literal, Self

from pydantic import ConfigDict, Discriminator, Field, NonNegativeInt, PositiveFloat, PositiveInt, model_validator

from param_decomp_b200.config.losses import PGDConfig, ReconstructionAuxiliariesMixin
from param_decomp_b200.formats.base import BaseConfig, Probability


class CIHistogramsConfig(BaseConfig):
    slow: ClassVar[bool] = True
    type: Literal["CIHistograms"] = "CIHistograms"
    n_batches_accum: PositiveInt | None
    density_heatmap_n_bins: PositiveInt | None = None


class CI_L0Config(BaseConfig):
    slow: ClassVar[bool] = False
    type: Literal["CI_L0"] = "CI_L0"
    groups: dict[str, list[str]] | None
    ci_alive_threshold: Probability = 0.0


class CIMeanPerComponentConfig(BaseConfig):
    slow: ClassVar[bool] = True
    type: Literal["CIMeanPerComponent"] = "CIMeanPerComponent"


class ComponentActivationDensityConfig(BaseConfig):
    slow: ClassVar[bool] = True
    type: Literal["ComponentActivationDensity"] = "ComponentActivationDensity"
    ci_alive_threshold: Probability = 0.0


class IdentityCITargetSpec(BaseConfig):
    layer_pattern: str
    n_features: PositiveInt


class DenseCITargetSpec(BaseConfig):
    layer_pattern: str
    k: PositiveInt


class IdentityCIErrorConfig(BaseConfig):
    slow: ClassVar[bool] = True
    type: Literal["IdentityCIError"] = "IdentityCIError"
    identity_ci: list[IdentityCITargetSpec] | None
    dense_ci: list[DenseCITargetSpec] | None


class _PermutationPlots(BaseConfig):
    identity_patterns: list[str] | None
    dense_patterns: list[str] | None


class PermutedCIPlotsConfig(_PermutationPlots):
    slow: ClassVar[bool] = True
    type: Literal["PermutedCIPlots"] = "PermutedCIPlots"


class UVPlotsConfig(_PermutationPlots):
    slow: ClassVar[bool] = True
    type: Literal["UVPlots"] = "UVPlots"


class EvalPGDConfig(PGDConfig):
    init: Literal["random"]
    source_shape: Literal["c"]


class EvalPGDReconLossConfig(EvalPGDConfig):
    slow: ClassVar[bool] = False
    type: Literal["PGDReconLoss"] = "PGDReconLoss"
    n_steps: NonNegativeInt

    @property
    def read_out_steps(self) -> tuple[int, ...]:
        return (self.n_steps,)


class SlowPGDReconLossConfig(EvalPGDConfig):
    slow: ClassVar[bool] = True
    type: Literal["SlowPGDReconLoss"] = "SlowPGDReconLoss"
    read_out_steps: tuple[NonNegativeInt, ...] = Field(min_length=1)

    @model_validator(mode="after")
    def _ascending(self) -> Self:
        assert all(a < b for a, b in pairwise(self.read_out_steps)), (
            f"read_out_steps must strictly ascend, got {self.read_out_steps}"
        )
        return self


# ---- LM-only metrics -------------------------------------------------------------------------


class CEandKLLossesConfig(BaseConfig):
    slow: ClassVar[bool] = False
    type: Literal["CEandKLLosses"] = "CEandKLLosses"
    rounding_threshold: Probability = 0.0


class CIActiveCountsPerPositionConfig(BaseConfig):
    slow: ClassVar[bool] = True
    type: Literal["CIActiveCountsPerPosition"] = "CIActiveCountsPerPosition"


class CIMaskedAttnPatternsReconLossConfig(BaseConfig):
    slow: ClassVar[bool] = True
    type: Literal["CIMaskedAttnPatternsReconLoss"] = "CIMaskedAttnPatternsReconLoss"


class StochasticAttnPatternsReconLossConfig(BaseConfig):
    slow: ClassVar[bool] = True
    type: Literal["StochasticAttnPatternsReconLoss"] = "StochasticAttnPatternsReconLoss"


class CIMaskedStrategy(BaseConfig):
    """Masks = the CI lower values; no weight-delta correction."""

    kind: Literal["ci_masked"] = "ci_masked"


class StochasticStrategy(BaseConfig):
    """One draw of `ci + (1 - ci) U[0,1]` with random weight-delta masks."""

    kind: Literal["stochastic"] = "stochastic"


class FreshPGDStrategy(BaseConfig):
    """Fresh sign-PGD sources (random init, one source per component shared by every token) ascended `n_steps`
    times against the output KL, composed with the CI."""

    kind: Literal["fresh_pgd"] = "fresh_pgd"
    n_steps: NonNegativeInt
    step_size: PositiveFloat


class PersistentStrategy(BaseConfig):
    """The run's persistent-PGD adversary sources, composed with the CI. `state_key` is the instance key of the
    persistent training term whose sources are read; per-row (`bc` / `bsc`) sources index training rows, so every
    evaluation sequence draws one of them."""

    kind: Literal["persistent"] = "persistent"
    state_key: str


RouterDivergenceStrategy = Annotated[
    CIMaskedStrategy | StochasticStrategy | FreshPGDStrategy | PersistentStrategy, Field(discriminator="kind")]


class RouterDivergenceConfig(BaseConfig):
    """Per MoE layer, how far the masked model's expert router drifts from the target's, under each masking
    strategy (logged under the strategy's kind, so each kind appears once).
    Parity: param_decomp/experiments/lm/eval_config.py:55-112."""

    slow: ClassVar[bool] = True
    type: Literal["RouterDivergence"] = "RouterDivergence"
    strategies: tuple[RouterDivergenceStrategy, ...]

    @model_validator(mode="after")
    def _kinds(self) -> Self:
        kinds = [s.kind for s in self.strategies]
        assert kinds and len(kinds) == len(set(kinds)), f"strategies must be non-empty, unique kinds: {kinds}"
        return self


class WellTemperednessConfig(BaseConfig):
    """Whether higher CI pre-activations mean greater ablation effects: components ablated one at a time at sampled
    token positions, `n_locations * n_components_per_region` ablations per pre-activation region; `groups` maps names
    to fnmatch patterns of site names. `ablations_per_forward` is accepted for schema parity (ablations run one per
    forward here). Parity: param_decomp/experiments/lm/eval_config.py:141-156."""

    model_config = ConfigDict(extra="allow", frozen=True)
    slow: ClassVar[bool] = True
    type: Literal["WellTemperedness"] = "WellTemperedness"
    groups: dict[str, list[str]] | None = None
    n_locations: PositiveInt = 4
    n_components_per_region: PositiveInt = 16
    ablations_per_forward: PositiveInt = 1


class ArithmeticCEKLConfig(BaseConfig):
    rounding_threshold: Probability = 0.0


class ArithmeticCIL0Config(BaseConfig):
    ci_alive_threshold: Probability = 0.0
    groups: dict[str, list[str]] | None = None


class ArithmeticFreshPGDConfig(BaseConfig):
    n_steps: NonNegativeInt
    step_size: PositiveFloat


class ArithmeticProbeMetrics(BaseConfig):
    """Scalar operations evaluated on the arithmetic grid rather than on corpus batches."""

    ce_kl: ArithmeticCEKLConfig = Field(default_factory=ArithmeticCEKLConfig)
    ci_l0: ArithmeticCIL0Config = Field(default_factory=ArithmeticCIL0Config)
    fresh_pgd: ArithmeticFreshPGDConfig | None = None


class ArithmeticCIGridConfig(BaseConfig):
    """Per-component causal-importance heat maps over an arithmetic operand grid, plus the probe metrics on it.
    Parity: param_decomp/experiments/lm/eval_config.py:158-192."""

    model_config = ConfigDict(extra="allow", frozen=True)
    slow: ClassVar[bool] = True
    type: Literal["ArithmeticCIGrid"] = "ArithmeticCIGrid"
    probe_metrics: ArithmeticProbeMetrics | None = None
    operation: Literal["add", "sub", "mul"] = "add"
    a_range: tuple[int, int] = (1, 100)
    b_range: tuple[int, int] = (1, 100)
    thresholds: tuple[Probability, ...] = (0.1,)
    top_k: PositiveInt = 24


AnyEvalMetricConfig = Annotated[
    ArithmeticCIGridConfig
    | CEandKLLossesConfig
    | CIActiveCountsPerPositionConfig
    | CIHistogramsConfig
    | CI_L0Config
    | CIMaskedAttnPatternsReconLossConfig
    | CIMeanPerComponentConfig
    | ComponentActivationDensityConfig
    | IdentityCIErrorConfig
    | PermutedCIPlotsConfig
    | EvalPGDReconLossConfig
    | RouterDivergenceConfig
    | SlowPGDReconLossConfig
    | StochasticAttnPatternsReconLossConfig
    | UVPlotsConfig
    | WellTemperednessConfig,
    Discriminator("type"),
]


class EvalConfig(BaseConfig):
    """`every` drives the fast tier, `slow_every` (a multiple of it) the slow tier."""

    batch_size: PositiveInt
    n_steps: PositiveInt
    every: PositiveInt
    slow_every: PositiveInt
    slow_on_first_step: bool = True
    metrics: list[AnyEvalMetricConfig] = Field(default_factory=list)

    @model_validator(mode="after")
    def _check(self) -> Self:
        types = [m.type for m in self.metrics]
        assert len(types) == len(set(types)), f"eval.metrics lists a metric type twice: {types}"
        for m in self.metrics:
            if isinstance(m, ReconstructionAuxiliariesMixin):
                for aux in m.auxiliaries:
                    assert isinstance(aux.coeff, float), f"{m.type}: {aux.name}.coeff must be a constant"
        assert self.slow_every % self.every == 0, (
            f"slow_every ({self.slow_every}) must be a multiple of every ({self.every})"
        )
        return self

    def is_due(self, metric: BaseConfig, step: int) -> bool:
        if getattr(metric, "slow"):
            if step == 0:
                return self.slow_on_first_step
            return step % self.slow_every == 0
        return step % self.every == 0
