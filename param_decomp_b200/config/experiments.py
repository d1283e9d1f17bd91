"""Experiment-level YAML schema: the TMS / ResidualMLP toys and the LM run shapes.

Parity: param_decomp/experiments/config.py:25-51, toy_config.py, tms/config.py, resid_mlp/config.py,
lm/config.py:134-768 (target specs, output edge, C-specs, CI-fn configs, `LMExperimentConfig`,
`LMTargetedExperimentConfig`), lm/runtime.py:149-497 (`RuntimeConfig`, `LaunchEnv`, profiling),
lm/run_data.py (`LMDataConfig`). Field names and `kind`/`type` tags are the reference's, so its YAML
files load here. Additions (marked below): a `random_init` target spec and a `synthetic_zipf`
data source, so runs need neither a checkpoint store nor a tokenised corpus; and
`runtime.backend`, which picks the eager-torch or the fused sm_100a execution path.

The reference's XLA knobs (`compiler_options`, `compilation_cache_dir`, `launch_env.xla_*`) parse and
are carried, but have no effect here: there is no tracing compiler in this framework.
"""

from __future__ import annotations

from enum import Enum
from pathlib import Path
from typing import Annotated, Literal, Self

from pydantic import (
    Discriminator,
    Field,
    NonNegativeInt,
    PositiveFloat,
    PositiveInt,
    Tag,
    field_validator,
    model_validator,
)

from param_decomp_b200.config.evals import EvalConfig
from param_decomp_b200.config.run import (
    Cadence,
    ExplicitCSpec,
    NontargetConfig,
    PDConfig,
    PlacementSpec,
    HsdpMeshShape,
    ResidentMeshShape,
    ResumeProvenance,
    SequenceSharding,
    TargetedPDConfig,
    WandbConfig,
)
from param_decomp_b200.formats.base import BaseConfig, Probability
from param_decomp_b200.formats.dataset_store import DataLayout, DatasetRef

# =============================================================================================
# shared bases
# =============================================================================================


class ExperimentConfigBase(BaseConfig):
    run_name: str
    cadence: Cadence
    wandb: WandbConfig | None = None

    @classmethod
    def from_file(cls, path: Path | str, data_root: Path | None = None):  # type: ignore[override]
        """Stored-config boundary: a file written under an older schema is migrated in memory
        (`infra/migrations.py`; the identity on current files) before validation, so pinned launch configs of
        old runs still load, resume and serve as fine-tune parents."""
        import json

        import yaml

        from param_decomp_b200.infra.migrations import migrate_raw

        path = Path(path)
        raw = json.loads(path.read_text()) if path.suffix == ".json" else yaml.safe_load(path.read_text())
        try:
            return cls.model_validate(migrate_raw(raw, data_root) if isinstance(raw, dict) else raw)
        except Exception as err:
            err.add_note(f"while validating {cls.__name__} from {path.as_posix()}")
            raise


class ExperimentConfig(ExperimentConfigBase):
    pd: PDConfig


# =============================================================================================
# toys
# =============================================================================================


class LayerwiseMlpCIFnConfig(BaseConfig):
    type: Literal["layerwise_mlp"] = "layerwise_mlp"
    hidden_dims: list[PositiveInt] = Field(..., min_length=1)


class ToyGlobalMlpCIFnConfig(BaseConfig):
    type: Literal["global_mlp"] = "global_mlp"
    hidden_dims: list[PositiveInt] = Field(..., min_length=1)


class ToyDecompositionConfig(BaseConfig):
    sites: ExplicitCSpec
    ci: Annotated[LayerwiseMlpCIFnConfig | ToyGlobalMlpCIFnConfig, Field(discriminator="type")]


class ToyExperimentConfig(ExperimentConfig):
    eval: EvalConfig | None = None


TMSGenerationType = Literal["exactly_one_active", "exactly_two_active", "exactly_three_active",
                            "exactly_four_active", "exactly_five_active", "at_least_zero_active"]


class TMSPretrainConfig(BaseConfig):
    steps: PositiveInt
    batch_size: PositiveInt
    lr: float
    seed: int = 0


class TMSTargetConfig(BaseConfig):
    n_features: PositiveInt
    n_hidden: PositiveInt
    n_hidden_layers: NonNegativeInt = 0
    hidden_layer_init: Literal["identity", "random"] = "identity"
    init_bias_to_zero: bool = True
    pretrain: TMSPretrainConfig


class TMSDataConfig(BaseConfig):
    feature_probability: Probability
    data_generation_type: TMSGenerationType = "at_least_zero_active"


class TMSExperimentConfig(ToyExperimentConfig):
    target: TMSTargetConfig
    decomposition: ToyDecompositionConfig
    data: TMSDataConfig


class ResidMLPPretrainConfig(BaseConfig):
    steps: PositiveInt
    batch_size: PositiveInt
    lr: float
    seed: int = 0
    label_type: Literal["act_plus_resid", "abs"] = "act_plus_resid"
    loss_type: Literal["readoff", "resid"] = "readoff"
    use_trivial_label_coeffs: bool = True
    importance_val: float = 1.0

    @model_validator(mode="after")
    def _space(self) -> Self:
        assert self.loss_type == "readoff" or self.importance_val == 1.0, (
            "importance_val only applies in feature space"
        )
        return self


class ResidMLPTargetConfig(BaseConfig):
    n_features: PositiveInt
    d_embed: PositiveInt
    d_mlp: PositiveInt
    n_layers: PositiveInt
    act_fn_name: Literal["gelu", "relu"]
    in_bias: bool = False
    out_bias: bool = False
    fixed_identity_embedding: bool = False
    pretrain: ResidMLPPretrainConfig

    @model_validator(mode="after")
    def _identity(self) -> Self:
        if self.fixed_identity_embedding:
            assert self.n_features == self.d_embed, "identity embedding needs n_features == d_embed"
        return self


class ResidMLPDataConfig(BaseConfig):
    feature_probability: Probability
    data_generation_type: Literal["exactly_one_active", "exactly_two_active", "at_least_zero_active"] = (
        "at_least_zero_active"
    )


class ResidMLPExperimentConfig(ToyExperimentConfig):
    target: ResidMLPTargetConfig
    decomposition: ToyDecompositionConfig
    data: ResidMLPDataConfig


# =============================================================================================
# LM: target
# =============================================================================================

AttentionImplementation = Literal["flash", "mosaic", "xla"]
ExpertImplementation = Literal["dense_masked", "ragged_dot", "tokamax_split_vjp", "all_to_all"]
WeightsDtype = Literal["bfloat16", "float32"]


class HFTarget(BaseConfig):
    kind: Literal["hf"] = "hf"
    model_class: str
    model_name: str


class PretrainedTarget(BaseConfig):
    kind: Literal["pretrained"] = "pretrained"
    model_class: str
    run_path: str


class HFWeightsInVendored(BaseConfig):
    kind: Literal["hf_weights_in_vendored"] = "hf_weights_in_vendored"
    model_class: str
    model_name: str


class PretrainedQwen35MoeTarget(BaseConfig):
    kind: Literal["pretrained_qwen35_moe"] = "pretrained_qwen35_moe"
    run_path: str


class Llama3RopeScalingConfig(BaseConfig):
    """Llama-3.1 long-context rescaling of the RoPE frequencies (`rope_scaling` with `rope_type: llama3` in a
    HuggingFace `config.json`)."""

    factor: PositiveFloat = 8.0
    low_freq_factor: PositiveFloat = 1.0
    high_freq_factor: PositiveFloat = 4.0
    original_max_position_embeddings: PositiveInt = 8192


class TransformerArchConfig(BaseConfig):
    """Inline architecture of a decoder-only LM (addition: the reference always derives this from a
    checkpoint). Covers Llama / Qwen3 / LlamaSimpleMLP shapes and the plain top-k MoE."""

    family: Literal["glu_transformer", "simple_mlp", "moe", "qwen35_moe"] = "glu_transformer"
    n_layer: PositiveInt
    d_model: PositiveInt
    n_head: PositiveInt
    n_kv_head: PositiveInt | None = None
    head_dim: PositiveInt | None = None
    d_ff: PositiveInt
    vocab_size: PositiveInt
    max_seq_len: PositiveInt = 2048
    rope_theta: PositiveFloat = 10000.0
    rope_scaling: Llama3RopeScalingConfig | None = None
    rms_eps: PositiveFloat = 1e-6
    qk_norm: bool = False
    tie_embeddings: bool = False
    # GPT-2-style variants of the dense families (the pretrainer's `GPT2Simple`): LayerNorm with bias instead of
    # RMSNorm (`norm_eps` = `rms_eps`), learned absolute position embeddings instead of RoPE
    norm_kind: Literal["rms", "layer"] = "rms"
    positional: Literal["rope", "learned"] = "rope"
    # MoE only
    n_experts: PositiveInt | None = None
    experts_per_token: PositiveInt | None = None
    norm_topk_prob: bool = True
    # qwen35_moe only (hybrid decoder: gated-DeltaNet layers, every `interval`-th layer gated full
    # attention, top-k MoE + shared expert in every layer; `d_ff` = per-expert hidden width)
    full_attention_interval: PositiveInt | None = None
    partial_rotary_factor: PositiveFloat = 1.0
    linear_num_key_heads: PositiveInt | None = None
    linear_key_head_dim: PositiveInt | None = None
    linear_num_value_heads: PositiveInt | None = None
    linear_value_head_dim: PositiveInt | None = None
    linear_conv_kernel_dim: PositiveInt = 4
    shared_expert_intermediate: PositiveInt | None = None
    delta_rule_kernel: Literal["sequential", "chunkwise", "cuda"] = "chunkwise"

    @model_validator(mode="after")
    def _check(self) -> Self:
        kv = self.n_kv_head or self.n_head
        assert self.n_head % kv == 0, "n_head must be a multiple of n_kv_head"
        if self.family in ("moe", "qwen35_moe"):
            assert self.n_experts and self.experts_per_token, "moe needs n_experts and experts_per_token"
        if self.family == "qwen35_moe":
            iv = self.full_attention_interval
            assert iv and iv >= 2 and self.n_layer % iv == 0, "n_layer must be a multiple of full_attention_interval >= 2"
            for f in ("linear_num_key_heads", "linear_key_head_dim", "linear_num_value_heads", "linear_value_head_dim",
                      "shared_expert_intermediate", "head_dim"):
                assert getattr(self, f), f"qwen35_moe needs {f}"
            assert self.linear_num_value_heads % self.linear_num_key_heads == 0
            rot = self.head_dim * self.partial_rotary_factor
            assert rot == int(rot) and int(rot) % 2 == 0, "rotary width must be an even integer"
        return self


class RandomInitTarget(BaseConfig):
    """Addition: seeded random weights of a stated architecture (benchmarks, tests, smoke runs)."""

    kind: Literal["random_init"] = "random_init"
    arch: TransformerArchConfig
    seed: int = 0


LMTargetSpec = Annotated[
    HFTarget | PretrainedTarget | HFWeightsInVendored | PretrainedQwen35MoeTarget | RandomInitTarget,
    Discriminator("kind"),
]


class MaterializedOutputEdgeConfig(BaseConfig):
    kind: Literal["materialized"] = "materialized"


class StreamedOutputEdgeConfig(BaseConfig):
    kind: Literal["streamed"] = "streamed"
    n_vocab_chunks: PositiveInt


LMOutputEdgeConfig = Annotated[MaterializedOutputEdgeConfig | StreamedOutputEdgeConfig, Discriminator("kind")]


class LMTargetConfig(BaseConfig):
    spec: LMTargetSpec
    expert_implementation: ExpertImplementation = "tokamax_split_vjp"
    attention_implementation: AttentionImplementation
    output_edge: LMOutputEdgeConfig
    weights_dtype: WeightsDtype

    @model_validator(mode="after")
    def _attn_dtype(self) -> Self:
        if self.attention_implementation in ("flash", "mosaic") and self.weights_dtype == "float32":
            raise ValueError("flash attention requires bfloat16 target weights")
        return self


# =============================================================================================
# LM: decomposition
# =============================================================================================


class AllLayers(BaseConfig):
    kind: Literal["all"] = "all"


class LayerRange(BaseConfig):
    kind: Literal["range"] = "range"
    start: NonNegativeInt
    end: PositiveInt

    @model_validator(mode="after")
    def _nonempty(self) -> Self:
        assert self.start < self.end, (self.start, self.end)
        return self


class LayerList(BaseConfig):
    kind: Literal["list"] = "list"
    indices: list[NonNegativeInt] = Field(..., min_length=1)

    @model_validator(mode="after")
    def _sorted(self) -> Self:
        assert self.indices == sorted(set(self.indices)), self.indices
        return self


LayerSelection = Annotated[AllLayers | LayerRange | LayerList, Field(discriminator="kind")]


def select_layers(sel: AllLayers | LayerRange | LayerList, n_layer: int) -> tuple[int, ...]:
    if isinstance(sel, AllLayers):
        return tuple(range(n_layer))
    if isinstance(sel, LayerRange):
        assert sel.end <= n_layer, f"layer range end {sel.end} exceeds n_layer {n_layer}"
        return tuple(range(sel.start, sel.end))
    assert sel.indices[-1] < n_layer, f"layer {sel.indices[-1]} exceeds n_layer {n_layer}"
    return tuple(sel.indices)


GluMatrix = Literal["q", "k", "v", "o", "gate", "up", "down"]
SimpleMlpMatrix = Literal["q_proj", "k_proj", "v_proj", "o_proj", "c_fc", "down_proj"]
Qwen36MoeMatrix = Literal[
    "gdn_q", "gdn_k", "gdn_v", "gdn_z", "gdn_b", "gdn_a", "gdn_out", "attn_q", "attn_k", "attn_v",
    "attn_o", "experts_gate", "experts_up", "experts_down", "shared_gate", "shared_up", "shared_down",
]  # fmt: skip
Initialization = Literal["random", "nonlinearity_aligned"]


class GluTransformerCSpec(BaseConfig):
    kind: Literal["glu_transformer"] = "glu_transformer"
    layers: LayerSelection
    cs: dict[GluMatrix, PositiveInt] = Field(..., min_length=1)
    initialization: Initialization = "random"

    @field_validator("cs", mode="before")
    @classmethod
    def _short_names(cls, v: object) -> object:
        # `q_proj` and `q` name the same matrix; the short form is canonical.
        if isinstance(v, dict):
            return {(k[:-5] if isinstance(k, str) and k.endswith("_proj") else k): c for k, c in v.items()}
        return v


class SimpleMlpCSpec(BaseConfig):
    kind: Literal["simple_mlp"] = "simple_mlp"
    layers: LayerSelection
    cs: dict[SimpleMlpMatrix, PositiveInt] = Field(..., min_length=1)
    initialization: Initialization = "random"


class Qwen36MoeCSpec(BaseConfig):
    kind: Literal["qwen36_moe"] = "qwen36_moe"
    layers: LayerSelection
    cs: dict[Qwen36MoeMatrix, PositiveInt] = Field(..., min_length=1)
    initialization: Initialization = "random"


class MoeCSpec(BaseConfig):
    """Addition: the plain top-k MoE LM (attention q/k/v/o plus per-expert gate/up/down)."""

    kind: Literal["moe"] = "moe"
    layers: LayerSelection
    cs: dict[Literal["q", "k", "v", "o", "experts_gate", "experts_up", "experts_down"],
             PositiveInt] = Field(..., min_length=1)
    initialization: Initialization = "random"

    @field_validator("cs", mode="before")
    @classmethod
    def _short_names(cls, v: object) -> object:
        if isinstance(v, dict):
            return {(k[:-5] if isinstance(k, str) and k.endswith("_proj") else k): c for k, c in v.items()}
        return v


class ResidualBoundaryTapSelection(BaseConfig):
    kind: Literal["residual_boundaries"] = "residual_boundaries"
    offsets: tuple[NonNegativeInt, ...] = Field(min_length=1)

    @model_validator(mode="after")
    def _sorted(self) -> Self:
        assert self.offsets == tuple(sorted(set(self.offsets))), self.offsets
        return self


CIFnInputTapSelection = (
    Literal["first_block_resid", "all_block_resids", "all_block_taps"] | ResidualBoundaryTapSelection
)


class QueryKeyNormalization(str, Enum):
    NONE = "none"
    RMS = "rms"


class AttentionSink(str, Enum):
    NONE = "none"
    LEARNED = "learned"


class FinalNormalization(str, Enum):
    NONE = "none"
    RMS = "rms"


CIFnAttentionMask = Literal["causal", "bidirectional"]


def _coerce_qk_norm(v: object) -> object:
    if v is True:
        return "rms"
    if v is False:
        return "none"
    return v


class _CIFnAttentionBase(BaseConfig):
    n_heads: PositiveInt
    implementation: AttentionImplementation
    mask: CIFnAttentionMask
    qk_norm: QueryKeyNormalization = QueryKeyNormalization.NONE
    logit_softcap: PositiveFloat | None = None
    sink: AttentionSink = AttentionSink.NONE

    @field_validator("qk_norm", mode="before")
    @classmethod
    def _qk(cls, v: object) -> object:
        return _coerce_qk_norm(v)


class MHACIFnAttentionConfig(_CIFnAttentionBase):
    kind: Literal["mha"] = "mha"


class GQACIFnAttentionConfig(_CIFnAttentionBase):
    kind: Literal["gqa"] = "gqa"
    n_kv_heads: PositiveInt

    @model_validator(mode="after")
    def _group(self) -> Self:
        assert self.n_heads % self.n_kv_heads == 0 and self.n_kv_heads < self.n_heads
        return self


class GeluCIFnFfnConfig(BaseConfig):
    kind: Literal["gelu"] = "gelu"
    hidden: PositiveInt


class SwigluCIFnFfnConfig(BaseConfig):
    kind: Literal["swiglu"] = "swiglu"
    hidden: PositiveInt


CIFnFfnConfig = Annotated[GeluCIFnFfnConfig | SwigluCIFnFfnConfig, Field(discriminator="kind")]
CIFnAttentionConfig = Annotated[MHACIFnAttentionConfig | GQACIFnAttentionConfig, Field(discriminator="kind")]


class InputScaleCalibrationConfig(BaseConfig):
    min_n_tokens: PositiveInt


class AffineClippedComponentActivationConfig(BaseConfig):
    kind: Literal["affine_clipped_component_activation"]
    output_scale_init: float = Field(allow_inf_nan=False)
    calibration: InputScaleCalibrationConfig


class TransformerCIFnConfig(BaseConfig):
    d_model: PositiveInt
    n_blocks: PositiveInt
    attention: CIFnAttentionConfig
    learned_norm_scale: bool = False

    @model_validator(mode="after")
    def _head_dim(self) -> Self:
        h = self.attention.n_heads
        assert self.d_model % h == 0 and (self.d_model // h) % 2 == 0, "head_dim must be even for RoPE"
        return self


class ChunkwiseTransformerCIFnConfig(TransformerCIFnConfig):
    type: Literal["chunkwise_transformer"] = "chunkwise_transformer"
    blocks_per_chunk: PositiveInt
    input_tap: CIFnInputTapSelection = "first_block_resid"
    ffn: CIFnFfnConfig


class GlobalTransformerCIFnConfig(TransformerCIFnConfig):
    type: Literal["global_transformer"] = "global_transformer"
    input_tap: CIFnInputTapSelection
    ffn: CIFnFfnConfig
    final_norm: FinalNormalization = FinalNormalization.NONE
    component_conditioning: AffineClippedComponentActivationConfig | None = None


class MoEChunkwiseTransformerCIFnConfig(TransformerCIFnConfig):
    type: Literal["moe_chunkwise_transformer"] = "moe_chunkwise_transformer"
    blocks_per_chunk: PositiveInt
    input_tap: CIFnInputTapSelection = "first_block_resid"
    expert_ffn_hidden: PositiveInt
    shared_ffn_hidden: PositiveInt
    expert_implementation: ExpertImplementation


class LMGlobalMlpCIFnConfig(BaseConfig):
    type: Literal["global_mlp"] = "global_mlp"
    hidden_dims: tuple[PositiveInt, ...] = Field(..., min_length=1)
    input_tap: CIFnInputTapSelection


class LMLayerwiseMlpCIFnConfig(BaseConfig):
    """Addition: one MLP per site reading that site's own input (the SPD paper's CI function)."""

    type: Literal["layerwise_mlp"] = "layerwise_mlp"
    hidden_dims: tuple[PositiveInt, ...] = Field(..., min_length=1)


LMCIFnConfig = Annotated[
    ChunkwiseTransformerCIFnConfig
    | GlobalTransformerCIFnConfig
    | MoEChunkwiseTransformerCIFnConfig
    | LMGlobalMlpCIFnConfig
    | LMLayerwiseMlpCIFnConfig,
    Field(discriminator="type"),
]


class LMDecompositionConfig(BaseConfig):
    sites: Annotated[GluTransformerCSpec | SimpleMlpCSpec | Qwen36MoeCSpec | MoeCSpec, Discriminator("kind")]
    ci: LMCIFnConfig


# =============================================================================================
# LM: data + runtime
# =============================================================================================


class SyntheticZipfDataset(BaseConfig):
    """Addition: seeded Zipf(exponent) token ids over the target vocabulary, generated on the fly.
    Row `i` of step `s` is a pure function of `(seed, s, i)`, like the parquet batch schedule."""

    kind: Literal["synthetic_zipf"] = "synthetic_zipf"
    exponent: PositiveFloat = 1.1
    seed: int = 0


LMDatasetRef = Annotated[DatasetRef.__origin__ | SyntheticZipfDataset, Discriminator("kind")]  # type: ignore[attr-defined]


class LMDataConfig(BaseConfig):
    train: LMDatasetRef
    eval: LMDatasetRef
    layout: DataLayout
    seq_len: PositiveInt


class ProfilingDisabled(BaseConfig):
    kind: Literal["disabled"] = "disabled"


class AdHocProfiling(BaseConfig):
    """An in-process `torch.profiler` run: after a warm-up (long enough for the step to have been recorded into
    its CUDA graph, where it is) the trainer traces `steps` steps into `<run_dir>/profile/trace.json` and exits:
    a measurement, not a trajectory. Parity: param_decomp/experiments/lm/runtime.py:247-254."""

    kind: Literal["ad_hoc"] = "ad_hoc"
    steps: PositiveInt = 3

    @model_validator(mode="before")
    @classmethod
    def _old_key(cls, data: object) -> object:
        if isinstance(data, dict) and "n_steps" in data and "steps" not in data:
            data = {**data, "steps": data["n_steps"]}
            data.pop("n_steps")
        return data


class NsightSystemsProfiling(BaseConfig):
    """For a run launched under an external `nsys profile --capture-range=cudaProfilerApi`: the trainer brackets
    `capture_steps` steps after `warmup_steps` with the CUDA profiler start / stop calls (one NVTX range per
    step) and exits. Without an attached profiler the calls do nothing.
    Parity: param_decomp/experiments/lm/runtime.py:257-262."""

    kind: Literal["nsight_systems"] = "nsight_systems"
    version: str = "2026.4.1"
    warmup_steps: NonNegativeInt = 5
    capture_steps: PositiveInt = 3


ProfilingConfig = Annotated[ProfilingDisabled | AdHocProfiling | NsightSystemsProfiling, Discriminator("kind")]


class LaunchEnv(BaseConfig):
    """Process environment exported before CUDA initialises. The `xla_*` fields are inert here."""

    xla_python_client_mem_fraction: PositiveFloat = 0.92
    xla_flags: str = ""
    xla_python_client_allocator: str | None = None
    xla_pjrt_gpu_host_memory_limit_gb: PositiveInt = 1024
    nccl_debug: str = "WARN"
    malloc_arena_max: PositiveInt = 2
    env: dict[str, str] = Field(default_factory=dict)

    def rendered(self) -> dict[str, str]:
        out = {"NCCL_DEBUG": self.nccl_debug, "MALLOC_ARENA_MAX": str(self.malloc_arena_max)}
        out.update(self.env)
        return out


class RuntimeConfig(BaseConfig):
    mesh: HsdpMeshShape | ResidentMeshShape
    sharding: PlacementSpec
    sequence_sharding: SequenceSharding = "replicate"
    remat_recon_forwards: bool = False
    remat_ci_fn: bool = False
    compiler_options: str | dict[str, bool | int | str] = "bare"
    compilation_cache_dir: Path = Path("~/.cache/param-decomp")
    launch_env: LaunchEnv = Field(default_factory=LaunchEnv)
    profiling: ProfilingConfig = Field(default_factory=ProfilingDisabled)
    backend: Literal["eager_torch", "fused_sm100"] = "fused_sm100"
    """Addition. `fused_sm100`: the hand-written sm_100a kernels (GPU only, fails loudly without
    them). `eager_torch`: plain PyTorch ops, the CPU oracle and the correctness reference."""
    step_recording: Literal["cuda_graph", "off"] = "cuda_graph"
    """Addition. `cuda_graph`: on the fused backend the train step is recorded into a CUDA graph after a few
    eager steps and replayed (per-step scalars live in a device table); runs whose step keeps per-step state
    on the host (persistent adversaries, frequency EMA, Muon, ...) stay eager and say so in the log."""
    peer_wait_limit_s: float = 30.0
    """Addition. How long a kernel that exchanges data with peer GPUs waits for a peer before it gives up and
    reports through the device status word (the engine then stops every rank before the next log line,
    evaluation or checkpoint)."""
    step_watchdog_s: PositiveFloat | None = None
    """Addition. When set, a host thread watches the training loop: an iteration (its evaluation and save
    included) that takes longer than this many seconds is treated as a preemption (all ranks save and exit at
    the next step boundary); if no boundary is reached within the same time again, the process exits without
    a checkpoint. Host-side only."""

    @model_validator(mode="before")
    @classmethod
    def _nested_mesh(cls, data: object) -> object:
        if isinstance(data, dict):
            flat = [k for k in ("replicate", "fsdp", "data", "tp") if k in data]
            if flat:
                raise ValueError(f"mesh axes are nested under `runtime.mesh:`; got flat keys {flat}")
        return data


class InlinePromptsConfig(BaseConfig):
    """Addition: target-stream prompts given literally, or drawn from rows of a tokenised dataset. Literal prompts
    shorter than `seq_len` are left-padded with their first token."""

    kind: Literal["inline"] = "inline"
    prompts: tuple[str, ...] | None = None
    dataset: LMDatasetRef | None = None
    seq_len: PositiveInt | None = None


class ArithmeticGridPromptsConfig(BaseConfig):
    """The `[a_range] x [b_range]` grid (both ends included) of `"<a><op><b>="` prompts as a training pool: the
    same construction as the `ArithmeticCIGrid` eval probe. Every prompt must tokenise to one length.
    Parity: param_decomp/experiments/lm/targeted_data.py:20-34."""

    kind: Literal["arithmetic_grid"] = "arithmetic_grid"
    operation: Literal["add", "sub", "mul"]
    a_range: tuple[int, int]
    b_range: tuple[int, int]


class PromptsFileConfig(BaseConfig):
    """One prompt per non-empty line of a text file; every line must tokenise to one length.
    Parity: param_decomp/experiments/lm/targeted_data.py:37-42."""

    kind: Literal["prompts_file"] = "prompts_file"
    path: Path


def _prompt_pool_kind(v: object) -> str:
    if isinstance(v, dict):
        return v.get("kind", "inline")
    return getattr(v, "kind", "inline")


LMPromptPoolConfig = Annotated[
    Annotated[InlinePromptsConfig, Tag("inline")]
    | Annotated[ArithmeticGridPromptsConfig, Tag("arithmetic_grid")]
    | Annotated[PromptsFileConfig, Tag("prompts_file")],
    Discriminator(_prompt_pool_kind),
]


class LMExperimentConfig(ExperimentConfig):
    runtime: RuntimeConfig
    eval: EvalConfig | None = None
    resume_provenance: ResumeProvenance | None = None
    target: LMTargetConfig
    decomposition: LMDecompositionConfig
    data: LMDataConfig


class LMTargetedExperimentConfig(ExperimentConfigBase):
    pd: TargetedPDConfig
    runtime: RuntimeConfig
    eval: EvalConfig | None = None
    target: LMTargetConfig
    decomposition: LMDecompositionConfig
    data: LMDataConfig
    prompts: LMPromptPoolConfig
    nontarget: NontargetConfig
