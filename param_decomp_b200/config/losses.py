"""Loss-metric configs: the `pd.loss_metrics` vocabulary of a run YAML.

Parity: param_decomp/core/configs.py:45-481,640-736 — same `type` tags and field names so the
reference's YAML files load unchanged. One addition: `LpImportanceMinimalityLoss`, the paper's
`(ci+eps)^p` penalty with a linear p-anneal (nano_param_decomp/run.py:408-429).
"""

from __future__ import annotations

from collections.abc import Sequence
from typing import Annotated, Literal, Self

from pydantic import (
    AliasChoices,
    Discriminator,
    Field,
    NonNegativeFloat,
    NonNegativeInt,
    PositiveFloat,
    PositiveInt,
    model_validator,
)

from param_decomp_b200.config.schedule import ScheduleConfig
from param_decomp_b200.formats.base import BaseConfig, Probability
from param_decomp_b200.formats.nonlinearity import NonlinearityUnitKind

# ---- routing ---------------------------------------------------------------------------------


class UniformKSubsetRoutingConfig(BaseConfig):
    type: Literal["uniform_k_subset"] = "uniform_k_subset"


class StaticProbabilityRoutingConfig(BaseConfig):
    type: Literal["static_probability"] = "static_probability"
    p: Probability


class AllRoutingConfig(BaseConfig):
    type: Literal["all"] = "all"


SubsetRoutingType = UniformKSubsetRoutingConfig | StaticProbabilityRoutingConfig | AllRoutingConfig
_Routing = Annotated[SubsetRoutingType, Field(discriminator="type")]

LossCoeff = float | ScheduleConfig

# ---- common bases ----------------------------------------------------------------------------


class TrainingLossConfig(BaseConfig):
    name: str | None = None  # logged identity; defaults to `type`
    coeff: LossCoeff

    @property
    def instance_key(self) -> str:
        return self.name if self.name is not None else getattr(self, "type")


class CaptureReconstruction(BaseConfig):
    capture: str = Field(min_length=1)
    distance: Literal["relative_squared_error", "categorical_kl_from_logits", "attention_pattern_kl"]


class AuxiliaryReconstructionConfig(BaseConfig):
    name: str = Field(min_length=1, pattern=r"^[^/]+$")
    coeff: NonNegativeFloat | ScheduleConfig
    comparisons: tuple[CaptureReconstruction, ...] = Field(min_length=1)

    @model_validator(mode="after")
    def _check(self) -> Self:
        assert self.name != "e2e", "e2e names the model-output comparison"
        caps = [c.capture for c in self.comparisons]
        assert len(set(caps)) == len(caps), f"duplicate comparison captures: {caps}"
        return self


class ReconstructionAuxiliariesMixin(BaseConfig):
    auxiliaries: tuple[AuxiliaryReconstructionConfig, ...] = ()

    @model_validator(mode="after")
    def _unique_aux(self) -> Self:
        names = [a.name for a in self.auxiliaries]
        assert len(set(names)) == len(names), f"duplicate auxiliary names: {names}"
        return self


# ---- non-recon terms -------------------------------------------------------------------------


class FaithfulnessLossConfig(TrainingLossConfig):
    type: Literal["FaithfulnessLoss"] = "FaithfulnessLoss"


class FrequencyMinimalityConfig(BaseConfig):
    coeff: NonNegativeFloat | ScheduleConfig
    reference_datapoint_count: PositiveInt = Field(
        validation_alias=AliasChoices("reference_datapoint_count", "reference_token_count")
    )
    ema_halflife_steps: PositiveFloat | None = Field(default=None, allow_inf_nan=False, le=1e6)


class ImportanceMinimalityLossConfig(TrainingLossConfig):
    """Smooth-L0 `c^2/(c^2+gamma^2)` on upper-leaky CI, plus an optional frequency penalty."""

    type: Literal["ImportanceMinimalityLoss"] = "ImportanceMinimalityLoss"
    gamma: ScheduleConfig
    frequency: FrequencyMinimalityConfig | None = None
    normalize_at_one: bool = False


class LpImportanceMinimalityLossConfig(TrainingLossConfig):
    """`(ci_upper + eps)^p` per component mean, plus `beta * mean * log2(1 + sum)`; p annealed."""

    type: Literal["LpImportanceMinimalityLoss"] = "LpImportanceMinimalityLoss"
    p_start: PositiveFloat = 2.0
    p_end: PositiveFloat = 0.4
    eps: NonNegativeFloat = 1e-12
    beta: NonNegativeFloat = 0.0


class NonlinearityLocalityLossConfig(TrainingLossConfig):
    type: Literal["NonlinearityLocalityLoss"] = "NonlinearityLocalityLoss"
    coeff: NonNegativeFloat | ScheduleConfig
    relative_threshold: ScheduleConfig
    unit_kind_coefficients: dict[NonlinearityUnitKind, PositiveFloat | None]
    normalize_at_one: bool = False

    @model_validator(mode="after")
    def _check(self) -> Self:
        assert all(k.frac > 0.0 for k in self.relative_threshold.points), (
            "relative_threshold knots must all keep frac > 0"
        )
        assert any(w is not None for w in self.unit_kind_coefficients.values()), (
            "unit_kind_coefficients must train at least one unit kind"
        )
        return self


# ---- recon terms -----------------------------------------------------------------------------


class CIMaskedReconLossConfig(TrainingLossConfig, ReconstructionAuxiliariesMixin):
    type: Literal["CIMaskedReconLoss"] = "CIMaskedReconLoss"


class CIMaskedReconSubsetLossConfig(TrainingLossConfig, ReconstructionAuxiliariesMixin):
    type: Literal["CIMaskedReconSubsetLoss"] = "CIMaskedReconSubsetLoss"
    routing: _Routing = UniformKSubsetRoutingConfig()


class StochasticReconLossConfig(TrainingLossConfig, ReconstructionAuxiliariesMixin):
    type: Literal["StochasticReconLoss"] = "StochasticReconLoss"
    n_samples: PositiveInt = 1
    """Independent mask draws averaged into the term (the reference spells extra draws as extra
    named terms; one field keeps the YAML short)."""


class StochasticReconSubsetLossConfig(TrainingLossConfig, ReconstructionAuxiliariesMixin):
    type: Literal["StochasticReconSubsetLoss"] = "StochasticReconSubsetLoss"
    routing: _Routing = UniformKSubsetRoutingConfig()
    n_samples: PositiveInt = 1


class UnmaskedReconLossConfig(TrainingLossConfig, ReconstructionAuxiliariesMixin):
    type: Literal["UnmaskedReconLoss"] = "UnmaskedReconLoss"


class UnmaskedNoDeltaReconLossConfig(TrainingLossConfig):
    type: Literal["UnmaskedNoDeltaReconLoss"] = "UnmaskedNoDeltaReconLoss"


PGDInitStrategy = Literal["random", "ones", "zeroes"]
BatchSourceShape = Literal["bc", "bsc"]
SourceShape = Literal["c", "bc", "bsc"]


class PGDConfig(ReconstructionAuxiliariesMixin):
    step_size: PositiveFloat


class TrainingPGDConfig(PGDConfig, TrainingLossConfig):
    n_steps: NonNegativeInt
    init: PGDInitStrategy
    source_shape: BatchSourceShape


class PGDReconLossConfig(TrainingPGDConfig):
    type: Literal["PGDReconLoss"] = "PGDReconLoss"


class PGDReconSubsetLossConfig(TrainingPGDConfig):
    type: Literal["PGDReconSubsetLoss"] = "PGDReconSubsetLoss"
    routing: _Routing = UniformKSubsetRoutingConfig()


class AdamPGDConfig(BaseConfig):
    type: Literal["adam"] = "adam"
    beta1: Probability = 0.9
    beta2: Probability = 0.999
    eps: NonNegativeFloat = 1e-8
    lr_schedule: ScheduleConfig


class SgdPGDConfig(BaseConfig):
    type: Literal["sgd"] = "sgd"
    lr_schedule: ScheduleConfig


class MomentumSgdPGDConfig(BaseConfig):
    type: Literal["momentum_sgd"] = "momentum_sgd"
    momentum: Probability
    lr_schedule: ScheduleConfig


AdversaryOptimizerConfig = Annotated[
    AdamPGDConfig | SgdPGDConfig | MomentumSgdPGDConfig, Field(discriminator="type")
]


class PersistentAdversaryLossConfig(TrainingLossConfig, ReconstructionAuxiliariesMixin):
    optimizer: AdversaryOptimizerConfig
    source_dtype: Literal["float32", "bfloat16", "uint16"] = "float32"
    n_warmup_steps: NonNegativeInt = 0
    adversary_objective: Literal["term", "e2e"] = "e2e"

    @model_validator(mode="after")
    def _storage(self) -> Self:
        if self.source_dtype == "uint16" and isinstance(self.optimizer, AdamPGDConfig):
            raise ValueError("uint16 fixed-point sources pair with sgd/momentum_sgd, not adam")
        return self


class PersistentPGDLossConfig(PersistentAdversaryLossConfig):
    source_shape: BatchSourceShape


class PersistentPGDReconLossConfig(PersistentPGDLossConfig):
    type: Literal["PersistentPGDReconLoss"] = "PersistentPGDReconLoss"


class SourcePoolConfig(BaseConfig):
    size_per_batch_element: PositiveInt


def _adv_fraction_ok(s: ScheduleConfig) -> None:
    if s.max_val > 1.0:
        raise ValueError(f"adv_fraction must stay within [0, 1]: {s}")


class MergedStochasticSubsetPooledPPGDReconLossConfig(PersistentAdversaryLossConfig):
    type: Literal["MergedStochasticSubsetPooledPPGDReconLoss"] = "MergedStochasticSubsetPooledPPGDReconLoss"
    pool: SourcePoolConfig
    adv_fraction: ScheduleConfig
    routing: _Routing = Field(default_factory=UniformKSubsetRoutingConfig)

    @model_validator(mode="after")
    def _frac(self) -> Self:
        _adv_fraction_ok(self.adv_fraction)
        return self


class MergedStochasticSubsetPPGDReconLossConfig(PersistentPGDLossConfig):
    type: Literal["MergedStochasticSubsetPPGDReconLoss"] = "MergedStochasticSubsetPPGDReconLoss"
    adv_fraction: ScheduleConfig
    routing: _Routing = Field(default_factory=UniformKSubsetRoutingConfig)

    @model_validator(mode="after")
    def _frac(self) -> Self:
        _adv_fraction_ok(self.adv_fraction)
        return self


AnyReconLossMetricConfig = (
    CIMaskedReconLossConfig
    | CIMaskedReconSubsetLossConfig
    | MergedStochasticSubsetPooledPPGDReconLossConfig
    | MergedStochasticSubsetPPGDReconLossConfig
    | PersistentPGDReconLossConfig
    | PGDReconLossConfig
    | PGDReconSubsetLossConfig
    | StochasticReconLossConfig
    | StochasticReconSubsetLossConfig
    | UnmaskedReconLossConfig
)
AnyImpMinConfig = ImportanceMinimalityLossConfig | LpImportanceMinimalityLossConfig

AnyLossMetricConfig = Annotated[
    AnyReconLossMetricConfig | FaithfulnessLossConfig | AnyImpMinConfig | NonlinearityLocalityLossConfig,
    Discriminator("type"),
]
TargetedLossMetricConfig = Annotated[AnyReconLossMetricConfig | AnyImpMinConfig, Discriminator("type")]

NontargetReconLossMetricConfig = (
    CIMaskedReconLossConfig
    | CIMaskedReconSubsetLossConfig
    | StochasticReconLossConfig
    | StochasticReconSubsetLossConfig
    | UnmaskedNoDeltaReconLossConfig
)

_NON_RECON = (FaithfulnessLossConfig, ImportanceMinimalityLossConfig, LpImportanceMinimalityLossConfig,
              NonlinearityLocalityLossConfig)


def is_recon_term(cfg: object) -> bool:
    return not isinstance(cfg, _NON_RECON)


def validate_training_losses(loss_metrics: Sequence[BaseConfig]) -> None:
    """Unique identities, exactly one imp-min term, >= 1 recon term, <= 1 nonlinearity term."""
    seen: set[str] = set()
    for cfg in loss_metrics:
        if isinstance(cfg, ReconstructionAuxiliariesMixin):
            for aux in cfg.auxiliaries:
                if isinstance(aux.coeff, float):
                    assert aux.coeff > 0.0, f"auxiliary {aux.name}: training coeff must be positive"
        key = cfg.instance_key  # type: ignore[attr-defined]
        assert key not in seen, f"duplicate loss instance_key {key!r}"
        seen.add(key)
    n_imp = sum(isinstance(c, (ImportanceMinimalityLossConfig, LpImportanceMinimalityLossConfig)) for c in loss_metrics)
    assert n_imp == 1, f"need exactly one importance-minimality term, got {n_imp}"
    assert any(is_recon_term(c) for c in loss_metrics), "need at least one recon loss term"
    n_nl = sum(isinstance(c, NonlinearityLocalityLossConfig) for c in loss_metrics)
    assert n_nl <= 1, f"need at most one nonlinearity-locality term, got {n_nl}"
