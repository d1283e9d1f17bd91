"""Resolve an authored LM CI-fn config against a target into a concrete CI-function module.

Tap selection vocabulary (param_decomp/experiments/lm/config.py:454-696):
  first_block_resid   the residual entering the group's first block
  all_block_resids    the residual entering every block of the group
  all_block_taps      every site-input vector of every block of the group
  residual_boundaries residual boundaries at the given offsets from the group's first block
A "group" is one chunk of `blocks_per_chunk` decomposed blocks (chunkwise) or all decomposed
blocks (global).
"""

from __future__ import annotations

from typing import Any

import torch
from torch import nn

from param_decomp_b200.config import experiments as X
from param_decomp_b200.core.ci_fn.mlp import GlobalMLPCIFn
from param_decomp_b200.core.ci_fn.transformer import (
    ChunkwiseTransformerCIFn,
    GlobalTransformerCIFn,
    MoEChunkwiseTransformerCIFn,
)


def _sites(model):
    """Site specs with GLOBAL block counts (a model split by expert parallelism lists only its own blocks in `sites`)."""
    return getattr(model, "global_sites", model.sites)


def _site_layers(model: Any) -> dict[int, list]:
    by_layer: dict[int, list] = {}
    for s in _sites(model):
        by_layer.setdefault(model.layer_of_site(s.name), []).append(s)
    return dict(sorted(by_layer.items()))


def tap_widths_for(model: Any, layers: list[int], selection: Any) -> dict[str, int]:
    d = model.arch.d_model
    first = layers[0]
    if selection == "first_block_resid":
        return {f"resid.{first}": d}
    if selection == "all_block_resids":
        return {f"resid.{l}": d for l in layers}
    if selection == "all_block_taps":
        out: dict[str, int] = {}
        for l in layers:
            for name, width in model.block_tap_widths(l).items():
                out[name] = width
        return out
    assert isinstance(selection, X.ResidualBoundaryTapSelection), selection
    return {f"resid.{first + off}": d for off in selection.offsets if first + off <= model.arch.n_layer}


def _attention(cfg: Any) -> dict:
    return {
        "n_heads": cfg.n_heads,
        "n_kv_heads": getattr(cfg, "n_kv_heads", None),
        "mask": cfg.mask,
        "qk_norm": cfg.qk_norm == X.QueryKeyNormalization.RMS,
        "logit_softcap": cfg.logit_softcap,
        "sink": cfg.sink == X.AttentionSink.LEARNED,
    }


def build_lm_ci_fn(cfg: Any, model: Any, g: torch.Generator) -> nn.Module:
    by_layer = _site_layers(model)
    layers = list(by_layer)
    site_taps = {s.name: model.tap_for_site(s.name) for s in _sites(model)}
    if isinstance(cfg, X.LMGlobalMlpCIFnConfig):
        widths = tap_widths_for(model, layers, cfg.input_tap)
        return GlobalMLPCIFn(tuple(widths.items()), {s.name: s.C for s in _sites(model)}, tuple(cfg.hidden_dims), g)
    if isinstance(cfg, X.GlobalTransformerCIFnConfig):
        widths = tap_widths_for(model, layers, cfg.input_tap)
        cond = None
        if cfg.component_conditioning is not None:
            cond = {"output_scale_init": cfg.component_conditioning.output_scale_init,
                    "min_n_tokens": cfg.component_conditioning.calibration.min_n_tokens}
            for s in _sites(model):  # conditioning also reads each site's own input
                widths.setdefault(site_taps[s.name], s.d_in)
        return GlobalTransformerCIFn(widths, {s.name: s.C for s in _sites(model)}, site_taps, cfg.d_model, cfg.n_blocks,
                                     _attention(cfg.attention), {"kind": cfg.ffn.kind, "hidden": cfg.ffn.hidden},
                                     final_norm=cfg.final_norm == X.FinalNormalization.RMS,
                                     learned_norm_scale=cfg.learned_norm_scale, conditioning=cond, g=g)
    if isinstance(cfg, X.ChunkwiseTransformerCIFnConfig):
        chunks = []
        for i in range(0, len(layers), cfg.blocks_per_chunk):
            ls = layers[i:i + cfg.blocks_per_chunk]
            cs = {s.name: s.C for l in ls for s in by_layer[l]}
            chunks.append((tap_widths_for(model, ls, cfg.input_tap), cs))
        shapes = {tuple(sorted(c.values())) for _, c in chunks}
        assert len(shapes) == 1, "chunkwise CI needs structurally identical chunks"
        return ChunkwiseTransformerCIFn(chunks, cfg.d_model, cfg.n_blocks, _attention(cfg.attention),
                                        {"kind": cfg.ffn.kind, "hidden": cfg.ffn.hidden}, cfg.learned_norm_scale, g=g)
    if isinstance(cfg, X.MoEChunkwiseTransformerCIFnConfig):
        chunks = []
        for i in range(0, len(layers), cfg.blocks_per_chunk):
            ls = layers[i:i + cfg.blocks_per_chunk]
            dense, blocked = {}, {}
            for li, l in enumerate(ls):
                for s in by_layer[l]:
                    if s.blocked:
                        blocked[s.name] = (li, s.C_block)
                    else:
                        dense[s.name] = s.C
            chunks.append({"layers": ls, "tap_widths": tap_widths_for(model, ls, cfg.input_tap),
                           "dense_sites": dense, "blocked_sites": blocked})
        return MoEChunkwiseTransformerCIFn(chunks, cfg.d_model, cfg.n_blocks, _attention(cfg.attention),
                                           model.arch.n_experts, cfg.expert_ffn_hidden, cfg.shared_ffn_hidden,
                                           cfg.learned_norm_scale, g)
    raise NotImplementedError(type(cfg).__name__)
