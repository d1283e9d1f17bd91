"""Resolve an `LMExperimentConfig` into runtime objects: target, sites, CI function, data sources.

Parity: param_decomp/experiments/lm/load_run.py:88-183 (`load_target`, `build_target`),
experiments/lm/config.py:262-327 (C-spec -> site tree), :454-696 (CI-fn resolution),
experiments/lm/training.py:197-301 (`_train` wiring).
"""

from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

import torch
from torch import nn

from param_decomp_b200.config import experiments as X
from param_decomp_b200.core.ci_fn.mlp import LayerwiseMLPCIFn
from param_decomp_b200.core.components import SiteSpec
from param_decomp_b200.data.synthetic import ZipfTokenSource
from param_decomp_b200.models import transformer as tf


@dataclass
class LMRun:
    model: Any
    ci_fn: nn.Module
    sample_train: Callable[[int], Any]
    sample_eval: Callable[[int], Any]
    arch: X.TransformerArchConfig
    tokens_per_step: int
    init_components: Callable | None = None
    ep: Any = None  # parallel.ep.ExpertParallel when the experts are split over the mesh's tp axis


def _dtype(name: str) -> torch.dtype:
    return torch.bfloat16 if name == "bfloat16" else torch.float32


def resolve_site_cs(sites: Any, arch: X.TransformerArchConfig) -> dict[str, int]:
    """Tile the per-matrix-type `cs` over the selected layers, in canonical within-block order."""
    layers = X.select_layers(sites.layers, arch.n_layer)
    if isinstance(sites, X.GluTransformerCSpec):
        assert arch.family == "glu_transformer", f"c-spec family glu_transformer != target family {arch.family}"
        kinds = [k for k in tf.GLU_KINDS if k in sites.cs]
    elif isinstance(sites, X.SimpleMlpCSpec):
        assert arch.family == "simple_mlp", f"c-spec family simple_mlp != target family {arch.family}"
        kinds = [k for k in tf.SIMPLE_KINDS if k in sites.cs]
    else:
        raise NotImplementedError(f"site spec {sites.kind!r} is resolved by its own target module")
    return {tf.site_name(arch.family, i, k): sites.cs[k] for i in layers for k in kinds}


def load_target_weights(cfg: X.LMTargetConfig, data_root: Path | None, device) -> tuple[X.TransformerArchConfig, dict]:
    spec = cfg.spec
    dtype = _dtype(cfg.weights_dtype)
    if isinstance(spec, X.RandomInitTarget):
        if spec.arch.family == "qwen35_moe":
            from param_decomp_b200.models.qwen35 import random_init_qwen35_weights

            return spec.arch, random_init_qwen35_weights(spec.arch, spec.seed, dtype, device)
        if spec.arch.family == "moe":
            from param_decomp_b200.models.moe import random_init_moe_weights

            return spec.arch, random_init_moe_weights(spec.arch, spec.seed, dtype, device)
        return spec.arch, tf.random_init_weights(spec.arch, spec.seed, dtype, device)
    from param_decomp_b200.models import loaders

    return loaders.load_from_spec(spec, data_root, dtype, device)


def build_ci_fn(cfg: Any, model: Any, seed: int) -> nn.Module:
    g = torch.Generator().manual_seed(seed + 1)
    sites: tuple[SiteSpec, ...] = getattr(model, "global_sites", model.sites)
    if isinstance(cfg, X.LMLayerwiseMlpCIFnConfig):
        blocked = {s.name: (model.layer_of_site(s.name), s.n_blocks, s.C_block) for s in sites if s.blocked}
        shapes = {s.name: (model.arch.d_model if s.blocked else s.d_in, s.C) for s in sites}
        return LayerwiseMLPCIFn(shapes, {s.name: model.tap_for_site(s.name) for s in sites},
                                tuple(cfg.hidden_dims), g, blocked=blocked)
    from param_decomp_b200.core.ci_fn import resolve

    return resolve.build_lm_ci_fn(cfg, model, g)


def build_lm_run(cfg: X.LMExperimentConfig | X.LMTargetedExperimentConfig, data_root: Path | None,
                 device: torch.device | str, rank: int = 0, world: int = 1, expert_group: Any = None,
                 expert_mode: str = "allreduce") -> LMRun:
    """`rank`/`world` index the batch axes (data shards). `expert_group`: the process group of the mesh's
    `tp` axis, whose ranks see the same tokens; on a mixture-of-experts target they split the experts (and
    their component blocks, param_decomp/routed/experts.py:28-40), on a dense target every site's component
    axis (param_decomp/core/placement.py:1040-1048)."""
    arch, weights = load_target_weights(cfg.target, data_root, device)
    ep = None
    if expert_group is not None and arch.family in ("moe", "qwen35_moe"):
        from param_decomp_b200.parallel.ep import ExpertParallel

        on_gpu = torch.device(device).type == "cuda" and cfg.runtime.backend == "fused_sm100"
        # `all_to_all`: the batch is sharded over the group too and jobs travel to their expert's owner (by
        # direct peer stores on GPUs); `allreduce`: the reference's scheme, tokens replicated over the group
        ep = ExpertParallel(expert_group, arch.n_experts, mode=expert_mode,
                            transport="p2p" if (expert_mode == "all_to_all" and on_gpu) else "collective")
    sites_cfg = cfg.decomposition.sites
    edge = cfg.target.output_edge
    n_chunks = edge.n_vocab_chunks if isinstance(edge, X.StreamedOutputEdgeConfig) else None
    backend = cfg.runtime.backend if torch.device(device).type == "cuda" else "eager_torch"
    if arch.family == "qwen35_moe":
        from param_decomp_b200.models import qwen35

        model = qwen35.build_qwen35_model(arch, weights, sites_cfg, cfg.target, backend, ep=ep)
    elif arch.family == "moe" or isinstance(sites_cfg, (X.MoeCSpec, X.Qwen36MoeCSpec)):
        from param_decomp_b200.models import moe

        model = moe.build_moe_model(arch, weights, sites_cfg, cfg.target, backend, rank, world, ep=ep)
    else:
        site_cs = resolve_site_cs(sites_cfg, arch)
        model = tf.TransformerDecomposedModel(arch, weights, site_cs, backend=backend,
                                              attention=cfg.target.attention_implementation, n_vocab_chunks=n_chunks)
    if expert_group is not None and ep is None:
        assert expert_mode != "all_to_all", "all_to_all dispatch applies to mixture-of-experts targets"
        model.split_components(expert_group)  # dense target: the tp axis divides every site's component axis
    ci_fn = build_ci_fn(cfg.decomposition.ci, model, cfg.pd.seed)
    if backend == "fused_sm100":
        from param_decomp_b200.core.ci_fn.mlp import BlockedSiteMLP, SiteMLP
        from param_decomp_b200.core.ci_fn.transformer import FusedLinear, RoutedExpertFFN

        for m in ci_fn.modules():
            if isinstance(m, (SiteMLP, BlockedSiteMLP, FusedLinear, RoutedExpertFFN)):
                m.fused = True

    seq = cfg.data.seq_len

    def source(ref: Any, salt: int):
        if isinstance(ref, X.SyntheticZipfDataset):
            return ZipfTokenSource(arch.vocab_size, seq, ref.exponent, ref.seed + salt)
        from param_decomp_b200.data.shards import ShardServer

        assert data_root is not None, "named datasets need --data-root"
        return ShardServer.open(ref, data_root, seq, cfg.data.layout, seed=cfg.pd.seed + salt)

    train_src, eval_src = source(cfg.data.train, 0), source(cfg.data.eval, 1)
    gb = cfg.pd.batch_size
    eb = cfg.eval.batch_size if cfg.eval is not None else gb
    pin = torch.device(device).type == "cuda"

    def sample_train(step: int):
        return train_src.batch(step, gb, rank, world, pin=pin).to(device, non_blocking=True)

    def sample_eval(i: int):
        return eval_src.batch(i, eb, rank, world, pin=pin).to(device, non_blocking=True)

    init = None
    if getattr(sites_cfg, "initialization", "random") == "nonlinearity_aligned":
        from param_decomp_b200.core.init_aligned import nonlinearity_aligned_init

        init = lambda comps: nonlinearity_aligned_init(comps, model, cfg.pd.seed)  # noqa: E731
    return LMRun(model, ci_fn, sample_train, sample_eval, arch, gb * seq, init, ep)
