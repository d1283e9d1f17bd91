"""Top-level algorithm and run configs: optimizers, `PDConfig`, cadence, W&B, resume lineage,
mesh shapes and placement-table schema.

Parity: param_decomp/core/configs.py:581-645 (optimizers), :738-887 (placement table + meshes),
:890-990 (PDConfig / TargetedPDConfig), :1026-1148 (cadence, checkpointing, wandb, provenance),
:1155-1221 (wandb.config flattening).
"""

from __future__ import annotations

import copy
from pathlib import Path
from typing import Annotated, Any, Literal, Self

from pydantic import (
    BeforeValidator,
    Discriminator,
    Field,
    NonNegativeFloat,
    NonNegativeInt,
    PositiveFloat,
    PositiveInt,
    model_validator,
)

from param_decomp_b200.config.losses import (
    AnyLossMetricConfig,
    FaithfulnessLossConfig,
    NontargetReconLossMetricConfig,
    TargetedLossMetricConfig,
    UnmaskedNoDeltaReconLossConfig,
    validate_training_losses,
)
from param_decomp_b200.config.schedule import ScheduleConfig
from param_decomp_b200.formats.base import BaseConfig, Probability

# ---- explicit (toy) site spec --------------------------------------------------------------


class ExplicitSite(BaseConfig):
    name: str
    C: PositiveInt


class ExplicitCSpec(BaseConfig):
    kind: Literal["explicit"] = "explicit"
    sites: list[ExplicitSite] = Field(..., min_length=1)


# ---- optimizers ------------------------------------------------------------------------------


class AdamWOptimizerConfig(BaseConfig):
    type: Literal["adamw"] = "adamw"
    lr_schedule: ScheduleConfig
    weight_decay: NonNegativeFloat = 0.0
    betas: tuple[Probability, Probability] = (0.9, 0.999)
    grad_clip_norm: PositiveFloat | None = None


class MuonOptimizerConfig(BaseConfig):
    type: Literal["muon"]
    lr_schedule: ScheduleConfig
    beta: Probability = 0.95
    consistent_rms: PositiveFloat | None = 0.2
    weight_decay: NonNegativeFloat = 0.0
    grad_clip_norm: PositiveFloat | None = None
    ns_steps: PositiveInt = 5
    ns_dtype: Literal["float32", "bfloat16"] = "bfloat16"


def _default_adamw(data: object) -> object:
    if isinstance(data, dict) and "type" not in data:
        return {**data, "type": "adamw"}
    return data


AnyOptimizerConfig = Annotated[
    AdamWOptimizerConfig | MuonOptimizerConfig, Discriminator("type"), BeforeValidator(_default_adamw)
]

# ---- algorithm sections ----------------------------------------------------------------------


class PDConfigBase(BaseConfig):
    seed: int = 0
    components_optimizer: AnyOptimizerConfig
    ci_fn_optimizer: AnyOptimizerConfig
    steps: PositiveInt
    batch_size: PositiveInt


class PDConfig(PDConfigBase):
    type: Literal["faithful"] = "faithful"
    loss_metrics: list[AnyLossMetricConfig] = Field(..., min_length=1)
    faithfulness_warmup_steps: NonNegativeInt = 0
    faithfulness_warmup_lr: PositiveFloat = 0.001
    faithfulness_warmup_weight_decay: NonNegativeFloat = 0.0

    @model_validator(mode="after")
    def _check(self) -> Self:
        validate_training_losses(self.loss_metrics)
        n_faith = sum(isinstance(c, FaithfulnessLossConfig) for c in self.loss_metrics)
        assert n_faith == 1, f"need exactly one FaithfulnessLoss, got {n_faith}"
        return self


class TargetedPDConfig(PDConfigBase):
    loss_metrics: list[TargetedLossMetricConfig] = Field(..., min_length=1)
    ci_scaled_weight_decay: PositiveFloat | None = None

    @model_validator(mode="after")
    def _check(self) -> Self:
        validate_training_losses(self.loss_metrics)
        return self


class NontargetConfig(BaseConfig):
    batch_size: PositiveInt
    impmin_coeff: NonNegativeFloat | ScheduleConfig
    recon: list[Annotated[NontargetReconLossMetricConfig, Discriminator("type")]] = Field(..., min_length=1)

    @model_validator(mode="after")
    def _check(self) -> Self:
        seen: set[str] = set()
        for cfg in self.recon:
            assert cfg.instance_key not in seen, f"duplicate non-target loss {cfg.instance_key!r}"
            seen.add(cfg.instance_key)
            if not isinstance(cfg, UnmaskedNoDeltaReconLossConfig):
                assert not cfg.auxiliaries, f"nontarget.recon {cfg.type!r}: auxiliaries are target-pass-only"
        return self


AnyPDConfig = PDConfig | TargetedPDConfig

# ---- cadence / checkpointing -----------------------------------------------------------------


class DenseLogPhase(BaseConfig):
    every: PositiveInt
    until_step: PositiveInt


class KeepLastNCheckpoints(BaseConfig):
    kind: Literal["keep_last"] = "keep_last"
    n: PositiveInt


class KeepAllCheckpoints(BaseConfig):
    kind: Literal["keep_all"] = "keep_all"


CheckpointRetention = Annotated[KeepLastNCheckpoints | KeepAllCheckpoints, Discriminator("kind")]


class PeriodicCheckpointing(BaseConfig):
    kind: Literal["periodic"] = "periodic"
    save_every: PositiveInt
    retention: CheckpointRetention


class NoCheckpointing(BaseConfig):
    kind: Literal["none"] = "none"


Checkpointing = Annotated[PeriodicCheckpointing | NoCheckpointing, Discriminator("kind")]


class Cadence(BaseConfig):
    train_log_every: PositiveInt = 20
    checkpointing: Checkpointing
    dense_log_phase: DenseLogPhase | None = None

    def should_log_train(self, step: int) -> bool:
        if self.dense_log_phase is not None and step < self.dense_log_phase.until_step:
            return step % self.dense_log_phase.every == 0
        return step % self.train_log_every == 0


class WandbConfig(BaseConfig):
    project: str
    metric_schema: Literal["legacy", "grouped", "v2"] = "legacy"
    """`grouped`: W&B receives two-level `<group>/<chart>` names (`infra/metric_names.py`); `metrics.jsonl` always
    keeps the local keys. `v2` is the older spelling of `grouped`."""
    entity: str | None = None
    group: str | None = None
    tags: list[str] = Field(default_factory=list)


class ResumeProvenance(BaseConfig):
    parent_run_dir: Path
    parent_step: int


# ---- mesh + placement schema -----------------------------------------------------------------

MeshAxis = Literal["replicate", "fsdp", "tp", "data"]
SemanticAxis = Literal[
    "stack", "d_in", "d_out", "C", "expert", "C_block", "d_model", "q_head", "kv_head", "ffn_hidden",
    "input", "depth", "site", "selected_c", "batch", "position", "feature", "head_dim", "layer",
    "vocab", "rope_frequency",
]  # fmt: skip
RuleConfig = dict[SemanticAxis, MeshAxis | list[MeshAxis] | None]


class ComponentsPlacementConfig(BaseConfig):
    optimizer_state: RuleConfig
    compute_weights: RuleConfig
    faithfulness_weights: RuleConfig
    faithfulness_deltas: RuleConfig
    operands: RuleConfig
    ns_compute: RuleConfig


class ActivationsPlacementConfig(BaseConfig):
    external: RuleConfig
    component: RuleConfig


TargetActivationRef = Literal["external", "intermediate"]


class TargetLinearPlacementConfig(BaseConfig):
    persist: RuleConfig
    operand: RuleConfig
    input: TargetActivationRef
    output: TargetActivationRef


class TargetComponentLinearPlacementConfig(BaseConfig):
    input: TargetActivationRef
    output: TargetActivationRef


class TargetWeightPlacementConfig(BaseConfig):
    persist: RuleConfig
    operand: RuleConfig


class TargetPlacementConfig(BaseConfig):
    embedding: TargetWeightPlacementConfig
    normalization: RuleConfig
    position_encoding: RuleConfig
    column: TargetLinearPlacementConfig
    row: TargetLinearPlacementConfig
    output: TargetWeightPlacementConfig
    intermediate: RuleConfig
    component: TargetComponentLinearPlacementConfig


PlacementPresetName = Literal[
    "owner",
    "zero1",
    "zero1-replicated-resident",
    "owner-replicated-resident",
    "zero1-replicated-resident-moe",
    "owner-replicated-resident-moe",
    "zero1-replicated-resident-moe-replicated-ns",
    "ddp",
]


class PlacementTableConfig(BaseConfig):
    components: ComponentsPlacementConfig
    ci_fn: PlacementPresetName
    activations: ActivationsPlacementConfig
    target: TargetPlacementConfig


PlacementSpec = PlacementPresetName | PlacementTableConfig
SequenceSharding = Literal["replicate", "sequence_parallel"]


class HsdpMeshShape(BaseConfig):
    replicate: PositiveInt
    fsdp: PositiveInt
    tp: PositiveInt

    @property
    def world_size(self) -> int:
        return self.replicate * self.fsdp * self.tp

    @property
    def axes(self) -> dict[str, int]:
        return {"replicate": self.replicate, "fsdp": self.fsdp, "tp": self.tp}


class ResidentMeshShape(BaseConfig):
    data: PositiveInt
    tp: PositiveInt

    @property
    def world_size(self) -> int:
        return self.data * self.tp

    @property
    def axes(self) -> dict[str, int]:
        return {"data": self.data, "tp": self.tp}


MeshShape = HsdpMeshShape | ResidentMeshShape

# ---- wandb.config shaping ----------------------------------------------------------------------

METRIC_SHORT_NAMES: dict[str, str] = {
    "CIMaskedReconLoss": "CIMaskRecon", "CIMaskedReconSubsetLoss": "CIMaskReconSub",
    "FaithfulnessLoss": "Faith", "ImportanceMinimalityLoss": "ImpMin",
    "LpImportanceMinimalityLoss": "LpImpMin", "NonlinearityLocalityLoss": "Nonlinearity",
    "PersistentPGDReconLoss": "PersistPGDRecon", "PGDReconLoss": "PGDRecon",
    "PGDReconSubsetLoss": "PGDReconSub", "StochasticReconLoss": "StochRecon",
    "StochasticReconSubsetLoss": "StochReconSub", "UnmaskedReconLoss": "UnmaskedRecon",
    "ArithmeticCIGrid": "ArithCIGrid", "CEandKLLosses": "CEandKL", "CIHistograms": "CIHist",
    "CI_L0": "CI_L0", "CIMaskedAttnPatternsReconLoss": "CIAttnRecon",
    "CIMeanPerComponent": "CIMeanPerComp", "ComponentActivationDensity": "CompActDens",
    "IdentityCIError": "IdCIErr", "PermutedCIPlots": "PermCIPlots",
    "StochasticAttnPatternsReconLoss": "StochAttnRecon", "UVPlots": "UVPlots",
}  # fmt: skip


def flatten_typed_lists(config_dict: dict[str, Any]) -> dict[str, Any]:
    """Turn lists of `{type: ...}` dicts into `path.<ShortName>.<field>` keys (for `wandb.config`)."""
    flat: dict[str, Any] = {}

    def typed(obj: Any) -> bool:
        return isinstance(obj, list) and len(obj) > 0 and all(isinstance(x, dict) and "type" in x for x in obj)

    def visit(node: Any, path: str) -> None:
        if isinstance(node, dict):
            for key in list(node):
                child, child_path = node[key], (f"{path}.{key}" if path else key)
                if typed(child):
                    for entry in child:
                        short = METRIC_SHORT_NAMES.get(entry["type"], entry["type"])
                        flat.update({f"{child_path}.{short}.{k}": v for k, v in entry.items() if k != "type"})
                    del node[key]
                else:
                    visit(child, child_path)
        elif isinstance(node, list):
            for i, item in enumerate(node):
                visit(item, f"{path}.{i}")

    out = copy.deepcopy(config_dict)
    visit(out, "")
    out.update(flat)
    return out
