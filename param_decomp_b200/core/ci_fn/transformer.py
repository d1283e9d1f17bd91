"""Transformer causal-importance functions: chunkwise, global, and the MoE block-selected variant.

Building blocks
  * input: each tap is RMS-normed without weights (eps = fp32 eps) and the taps are concatenated,
    then projected to `d_model`;
  * block: pre-norm RoPE self-attention (MHA or GQA; causal or bidirectional, always confined to a
    document when segment ids are given; optional per-head QK RMS-norm with learned gains, logit
    soft-cap, learned attention sink) + pre-norm FFN (GELU `Linear-GELU-Linear` or SwiGLU), biases
    everywhere, block norms weightless unless `learned_norm_scale`;
  * heads: one linear head per decomposed site mapping `d_model -> C_site`.
Architectures
  * `ChunkwiseTransformerCIFn`: the decomposed layers are cut into chunks of `blocks_per_chunk`
    consecutive target blocks; each chunk has its own transformer reading that chunk's taps and
    emitting CI for that chunk's sites (chunks are stacked modules evaluated one after another);
  * `GlobalTransformerCIFn`: one transformer over taps from all decomposed blocks, heads for every
    site, optional final RMS norm, optional component conditioning;
  * component conditioning adds `s+ * clip(a+ h + b+) + s- * clip(a- (-h) + b-) + bias` per
    component, `h = x V` of the clean site input; input scales start at `1/q` with `q` the 99.9th
    percentile of `|h|` on the calibration batch;
  * `MoEChunkwiseTransformerCIFn`: the FFN is a bank of routed experts dispatched by the target's
    captured routing, and expert-blocked sites emit narrow `SelectedCI` (values only for the
    selected experts of each token).

Parity: param_decomp/core/ci_fn/implementations/transformer/layers.py:128-543,
chunkwise/arch.py:164-517, global_transformer/arch.py:94-453,
transformer/component_conditioning.py:105-425, block_selected/arch.py:206-910 and routing.py.
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from param_decomp_b200.core.ci_fn.interface import census
from param_decomp_b200.core.components import BlockSelection, SelectedCI
from param_decomp_b200.models import ports

FP32_EPS = torch.finfo(torch.float32).eps


class FusedLinear(nn.Linear):
    """`nn.Linear` whose product runs on the hand-written tcgen05 GEMM (bf16 operands, fp32 masters and
    gradients) once the builder sets `fused` on the sm_100a backend; plain `F.linear` otherwise (CPU, the eager
    backend, widths that are not multiples of 8 elements - the TMA row pitch)."""

    fused = False

    def forward(self, x: Tensor) -> Tensor:  # type: ignore[override]
        if self.fused and x.is_cuda:
            from param_decomp_b200.ops.linear import trainable_linear, trainable_linear_supported

            if trainable_linear_supported(x, self.weight):
                return trainable_linear(x, self.weight, self.bias)
        return F.linear(x, self.weight.to(x.dtype), None if self.bias is None else self.bias.to(x.dtype))


def _norm(x: Tensor, w: Tensor | None) -> Tensor:
    """Weightless / learned-scale RMS norm with eps = fp32 eps; the bandwidth kernel on bf16 CUDA activations."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        from param_decomp_b200.ops import native

        if native.available():
            from param_decomp_b200.ops.elementwise import rms_norm

            return rms_norm(x, None if w is None else w.to(torch.bfloat16), FP32_EPS)
    return ports.rms_norm(x, w, FP32_EPS)


def _linear(d_in: int, d_out: int, g: torch.Generator | None, bias: bool = True) -> nn.Linear:
    lin = FusedLinear(d_in, d_out, bias=bias)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(d_out, d_in, generator=g) / math.sqrt(d_in))
        if bias:
            lin.bias.zero_()
    return lin


class CIAttention(nn.Module):
    def __init__(self, d_model: int, n_heads: int, n_kv_heads: int | None, mask: str, qk_norm: bool,
                 logit_softcap: float | None, sink: bool, rope_base: float, g: torch.Generator | None) -> None:
        super().__init__()
        self.n_heads, self.n_kv = n_heads, n_kv_heads or n_heads
        self.hd = d_model // n_heads
        self.causal = mask == "causal"
        self.softcap, self.rope_base = logit_softcap, rope_base
        self.wq = _linear(d_model, n_heads * self.hd, g)
        self.wk = _linear(d_model, self.n_kv * self.hd, g)
        self.wv = _linear(d_model, self.n_kv * self.hd, g)
        self.wo = _linear(n_heads * self.hd, d_model, g)
        self.q_gain = nn.Parameter(torch.ones(self.hd)) if qk_norm else None
        self.k_gain = nn.Parameter(torch.ones(self.hd)) if qk_norm else None
        self.sink = nn.Parameter(torch.zeros(n_heads)) if sink else None

    def forward(self, x: Tensor, positions: Tensor, segment_ids: Tensor | None) -> Tensor:
        B, T, _ = x.shape
        q = self.wq(x).view(B, T, self.n_heads, self.hd)
        k = self.wk(x).view(B, T, self.n_kv, self.hd)
        v = self.wv(x).view(B, T, self.n_kv, self.hd)
        if self.q_gain is not None:
            q = ports.rms_norm(q, self.q_gain, FP32_EPS)
            k = ports.rms_norm(k, self.k_gain, FP32_EPS)
        cos, sin = ports.rope_cos_sin(positions, self.hd, self.rope_base)
        q, k = ports.apply_rope(q, cos, sin), ports.apply_rope(k, cos, sin)
        if self.softcap is None and self.sink is None and x.is_cuda:
            out = ports.sdpa(q, k, v, self.causal, segment_ids, "flash")
        else:
            out = ports.sdpa_reference(q, k, v, self.causal, segment_ids, self.softcap, self.sink)
        return self.wo(out.reshape(B, T, self.n_heads * self.hd))


class CIFeedForward(nn.Module):
    def __init__(self, d_model: int, hidden: int, kind: str, g: torch.Generator | None) -> None:
        super().__init__()
        self.kind = kind
        self.w1 = _linear(d_model, hidden, g)
        self.w_gate = _linear(d_model, hidden, g) if kind == "swiglu" else None
        self.w2 = _linear(hidden, d_model, g)

    def forward(self, x: Tensor) -> Tensor:
        if self.w_gate is not None:
            return self.w2(F.silu(self.w_gate(x)) * self.w1(x))
        return self.w2(F.gelu(self.w1(x)))


class CIBlock(nn.Module):
    def __init__(self, d_model: int, attn: CIAttention, ffn: nn.Module, learned_norm_scale: bool) -> None:
        super().__init__()
        self.attn, self.ffn = attn, ffn
        self.n1 = nn.Parameter(torch.ones(d_model)) if learned_norm_scale else None
        self.n2 = nn.Parameter(torch.ones(d_model)) if learned_norm_scale else None

    def forward(self, x: Tensor, positions: Tensor, segment_ids: Tensor | None, **ffn_ctx: Any) -> Tensor:
        x = x + self.attn(_norm(x, self.n1), positions, segment_ids)
        return x + self.ffn(_norm(x, self.n2), **ffn_ctx)


def normed_concat(taps: dict[str, Tensor], keys: tuple[str, ...]) -> Tensor:
    return torch.cat([ports.rms_norm(taps[k].float(), None, FP32_EPS) for k in keys], dim=-1)


def _positions(x: Tensor, ctx: dict[str, Any]) -> Tensor:
    pos = ctx.get("positions")
    return pos if pos is not None else torch.arange(x.shape[1], device=x.device)[None]


class TransformerBackbone(nn.Module):
    """Input projection + `n_blocks` blocks over `[B, T, sum(tap widths)]`."""

    def __init__(self, tap_widths: dict[str, int], d_model: int, n_blocks: int, attention: dict, ffn: dict,
                 learned_norm_scale: bool, rope_base: float, g: torch.Generator | None) -> None:
        super().__init__()
        self.tap_keys = tuple(tap_widths)
        self.w_in = _linear(sum(tap_widths.values()), d_model, g)
        self.blocks = nn.ModuleList(
            CIBlock(d_model, CIAttention(d_model, attention["n_heads"], attention.get("n_kv_heads"), attention["mask"],
                                         attention.get("qk_norm", False), attention.get("logit_softcap"),
                                         attention.get("sink", False), rope_base, g),
                    CIFeedForward(d_model, ffn["hidden"], ffn["kind"], g), learned_norm_scale)
            for _ in range(n_blocks))

    def forward(self, taps: dict[str, Tensor], ctx: dict[str, Any], remat: bool = False) -> Tensor:
        x = self.w_in(normed_concat(taps, self.tap_keys))
        pos, seg = _positions(x, ctx), ctx.get("segment_ids")
        for blk in self.blocks:
            if remat and x.requires_grad:
                x = torch.utils.checkpoint.checkpoint(blk, x, pos, seg, use_reentrant=False)
            else:
                x = blk(x, pos, seg)
        return x


class ComponentConditioning(nn.Module):
    """Per-component affine-clipped function of the component activation `h = x V`."""

    def __init__(self, site_cs: dict[str, int], output_scale_init: float) -> None:
        super().__init__()
        self.sites = tuple(site_cs)
        mk = lambda val: nn.ParameterDict({self.key(s): nn.Parameter(torch.full((c,), val)) for s, c in site_cs.items()})  # noqa: E731
        self.s_pos, self.s_neg = mk(output_scale_init), mk(output_scale_init)
        self.a_pos, self.a_neg = mk(1.0), mk(1.0)
        self.b_pos, self.b_neg, self.bias = mk(0.0), mk(0.0), mk(0.0)
        self.calibrated = False

    @staticmethod
    def key(site: str) -> str:
        return site.replace(".", "_")

    @torch.no_grad()
    def calibrate(self, h: dict[str, Tensor], quantile: float = 0.999) -> None:
        """Input scales become `1/q`, `q` = each component's `quantile` of `|h|` over the batch."""
        for s in self.sites:
            a = h[s].float().abs().reshape(-1, h[s].shape[-1])
            k = max(1, int(math.ceil(quantile * a.shape[0])))
            q = a.kthvalue(k, dim=0).values.clamp_min(1e-12)
            self.a_pos[self.key(s)].copy_(1.0 / q)
            self.a_neg[self.key(s)].copy_(1.0 / q)
        self.calibrated = True

    def forward(self, site: str, h: Tensor) -> Tensor:
        from param_decomp_b200.core.squashing import lower_leaky_hard_sigmoid as clip

        k = self.key(site)
        h = h.float()
        pos = self.s_pos[k] * clip(self.a_pos[k] * h + self.b_pos[k])
        neg = self.s_neg[k] * clip(self.a_neg[k] * (-h) + self.b_neg[k])
        return pos + neg + self.bias[k]


class GlobalTransformerCIFn(nn.Module):
    def __init__(self, tap_widths: dict[str, int], site_cs: dict[str, int], site_taps: dict[str, str], d_model: int,
                 n_blocks: int, attention: dict, ffn: dict, final_norm: bool = False, learned_norm_scale: bool = False,
                 conditioning: dict | None = None, rope_base: float = 10000.0, g: torch.Generator | None = None) -> None:
        super().__init__()
        self.backbone = TransformerBackbone(tap_widths, d_model, n_blocks, attention, ffn, learned_norm_scale, rope_base, g)
        self.input_taps = tuple(tap_widths)
        self.site_cs, self.site_taps = dict(site_cs), dict(site_taps)
        self.final_norm = final_norm
        self.heads = nn.ModuleDict({ComponentConditioning.key(s): _linear(d_model, c, g) for s, c in site_cs.items()})
        self.conditioning = ComponentConditioning(site_cs, conditioning["output_scale_init"]) if conditioning else None
        self.calibration_min_tokens = int(conditioning.get("min_n_tokens", 1)) if conditioning else 1
        self.remat = False

    def forward(self, taps: dict[str, Tensor], **ctx: Any) -> dict[str, Tensor]:
        x = self.backbone(taps, ctx, self.remat)
        if self.final_norm:
            x = ports.rms_norm(x, None, FP32_EPS)
        out = {s: self.heads[ComponentConditioning.key(s)](x) for s in self.site_cs}
        if self.conditioning is not None:
            comps = ctx["components"]
            h = {s: comps.component_activations(s, taps[self.site_taps[s]].float()) for s in self.site_cs}
            if not self.conditioning.calibrated:
                # the first batch calibrates the input scales; it must hold enough tokens for the quantile
                # (param_decomp/experiments/lm/ci_fn_init.py:70-77 asserts the same on the global batch)
                import torch.distributed as dist

                first = next(iter(h.values()))
                n_tokens = first.numel() // first.shape[-1] * (dist.get_world_size() if dist.is_initialized() else 1)
                assert n_tokens >= self.calibration_min_tokens, (
                    f"the calibration batch holds {n_tokens} tokens, fewer than calibration.min_n_tokens "
                    f"{self.calibration_min_tokens}")
                self.conditioning.calibrate({k: v.detach() for k, v in h.items()})
            out = {s: out[s] + self.conditioning(s, h[s]) for s in self.site_cs}
        return out

    def parameter_census(self) -> dict[str, int]:
        return census(self)

    def useful_flops_per_position(self) -> int:
        return 2 * sum(p.numel() for p in self.parameters() if p.dim() >= 2)


class ChunkwiseTransformerCIFn(nn.Module):
    """`chunks[i] = (tap_widths_i, site_cs_i)`: one backbone + heads per chunk of target blocks."""

    def __init__(self, chunks: list[tuple[dict[str, int], dict[str, int]]], d_model: int, n_blocks: int, attention: dict,
                 ffn: dict, learned_norm_scale: bool = False, rope_base: float = 10000.0,
                 g: torch.Generator | None = None) -> None:
        super().__init__()
        self.chunk_fns = nn.ModuleList(
            GlobalTransformerCIFn(taps, cs, {}, d_model, n_blocks, attention, ffn, False, learned_norm_scale, None,
                                  rope_base, g) for taps, cs in chunks)
        self.input_taps = tuple(dict.fromkeys(k for taps, _ in chunks for k in taps))
        self.remat = False

    def forward(self, taps: dict[str, Tensor], **ctx: Any) -> dict[str, Tensor]:
        out: dict[str, Tensor] = {}
        for fn in self.chunk_fns:
            fn.remat = self.remat
            out.update(fn(taps, **ctx))
        return out

    def parameter_census(self) -> dict[str, int]:
        return census(self)

    def useful_flops_per_position(self) -> int:
        return sum(fn.useful_flops_per_position() for fn in self.chunk_fns)  # type: ignore[operator]


def routed_linear(rows: Tensor, W: Tensor, sel: BlockSelection, per_job: bool, fused: bool) -> Tensor:
    """`out[n, s] = in[n, s] @ W[e(n, s)]` for the experts `sel.indices [.., k]` each token selected:
    `rows` is `[N, d]` (one row per token, shared by its `k` jobs) or, with `per_job`, `[N * k, d]` (one row
    per job, token-major); `W [E, d, h]`; returns `[N * k, h]`. Never gathers per-token weight copies: on the
    fused backend the jobs are sorted by expert into padded row groups and run as ONE grouped tcgen05 product
    (`ops/grouped.py`, the layout is shared with the target's own expert products of that routing decision);
    elsewhere each expert's jobs are one dense product."""
    idx = sel.indices.reshape(-1, sel.indices.shape[-1])
    N, k = idx.shape
    E = W.shape[0]
    if fused and rows.is_cuda and W.shape[1] % 8 == 0 and W.shape[2] % 8 == 0:
        from param_decomp_b200.ops.grouped import JobLayout, grouped_linear_trainable

        layout = JobLayout.cached(sel.indices, E)
        r = rows.to(torch.bfloat16)
        padded = layout.scatter_rows(r) if per_job else layout.expand_tokens(r.contiguous(), k)
        return layout.gather_rows(grouped_linear_trainable(padded, W, None, layout))
    flat_e = idx.reshape(-1)
    order = flat_e.argsort(stable=True)
    counts = torch.bincount(flat_e, minlength=E).tolist()
    src = rows if per_job else rows.repeat_interleave(k, dim=0)
    pieces, start = [], 0
    for e, n in enumerate(counts):
        if n:
            jobs = order[start:start + n]
            pieces.append(src[jobs].to(W.dtype) @ W[e])
            start += n
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    return torch.cat(pieces)[inv]


class RoutedExpertFFN(nn.Module):
    """Concat-wide routed expert bank: for each covered target layer one bank of `E` SwiGLU experts,
    dispatched by that layer's captured routing, plus a dense shared SwiGLU expert. The last block's
    bank also carries per-expert heads that emit CI for the experts' component blocks."""

    fused = False  # set by the builder on the fused sm_100a backend

    def __init__(self, d_model: int, n_layers: int, n_experts: int, hidden: int, shared_hidden: int,
                 g: torch.Generator | None) -> None:
        super().__init__()
        self.n_layers, self.n_experts = n_layers, n_experts
        s = 1.0 / math.sqrt(d_model)
        self.w_gate = nn.Parameter(torch.randn(n_layers, n_experts, d_model, hidden, generator=g) * s)
        self.w_up = nn.Parameter(torch.randn(n_layers, n_experts, d_model, hidden, generator=g) * s)
        self.w_down = nn.Parameter(torch.randn(n_layers, n_experts, hidden, d_model, generator=g) / math.sqrt(hidden))
        self.shared = CIFeedForward(d_model, shared_hidden, "swiglu", g)

    def expert_hidden(self, x: Tensor, layer: int, sel: BlockSelection) -> Tensor:
        """`[N * k, hidden]` (token-major jobs): SwiGLU hidden of the selected experts of `layer`."""
        x2 = x.reshape(-1, x.shape[-1])
        gate = routed_linear(x2, self.w_gate[layer], sel, False, self.fused)
        up = routed_linear(x2, self.w_up[layer], sel, False, self.fused)
        return F.silu(gate) * up

    def forward(self, x: Tensor, routing: list[BlockSelection] | None = None) -> Tensor:
        out = self.shared(x)
        if routing is None:
            return out
        lead, d = x.shape[:-1], x.shape[-1]
        for layer, sel in enumerate(routing):
            k = sel.indices.shape[-1]
            h = self.expert_hidden(x, layer, sel)
            y = routed_linear(h, self.w_down[layer], sel, True, self.fused).reshape(*lead, k, d)
            out = out + (y * sel.weights.unsqueeze(-1).to(y.dtype)).sum(-2).to(out.dtype)
        return out


class MoEChunkwiseTransformerCIFn(nn.Module):
    """Chunkwise CI transformer for expert-blocked targets. Sites listed in `blocked_sites` map to
    `(layer_in_chunk, C_block)` and emit `SelectedCI`; other sites emit full-width CI."""

    def __init__(self, chunks: list[dict], d_model: int, n_blocks: int, attention: dict, n_experts: int,
                 expert_hidden: int, shared_hidden: int, learned_norm_scale: bool = False,
                 g: torch.Generator | None = None) -> None:
        super().__init__()
        self.chunks_meta = chunks
        self.n_experts = n_experts
        self.backbones = nn.ModuleList()
        self.dense_heads = nn.ModuleList()
        self.expert_heads = nn.ParameterList()
        for ch in chunks:
            widths = dict(ch["tap_widths"])
            widths.update({f"__routing.{l}": n_experts for l in ch["layers"]})
            bb = TransformerBackbone(widths, d_model, n_blocks, attention, {"kind": "swiglu", "hidden": shared_hidden},
                                     learned_norm_scale, 10000.0, g)
            for blk in bb.blocks:
                blk.ffn = RoutedExpertFFN(d_model, len(ch["layers"]), n_experts, expert_hidden, shared_hidden, g)
            self.backbones.append(bb)
            self.dense_heads.append(nn.ModuleDict({ComponentConditioning.key(s): _linear(d_model, c, g)
                                                   for s, c in ch["dense_sites"].items()}))
            # per-expert heads read the last block's expert hidden: [E, hidden, C_block] per blocked site
            for s, (layer, c_block) in ch["blocked_sites"].items():
                self.expert_heads.append(nn.Parameter(
                    torch.randn(n_experts, expert_hidden, c_block, generator=g) / math.sqrt(expert_hidden)))
        self.input_taps = tuple(dict.fromkeys(k for ch in chunks for k in ch["tap_widths"]))

    def forward(self, taps: dict[str, Tensor], aux: dict[str, Any] | None = None, **ctx: Any) -> dict[str, Any]:
        routing_all: dict[int, BlockSelection] = (aux or {}).get("routing", {})
        out: dict[str, Any] = {}
        head_i = 0
        for ci, ch in enumerate(self.chunks_meta):
            routing = [routing_all[l] for l in ch["layers"]]
            t = dict(taps)
            for l, sel in zip(ch["layers"], routing):
                dense = torch.zeros(*sel.indices.shape[:-1], self.n_experts, device=sel.indices.device)
                t[f"__routing.{l}"] = dense.scatter(-1, sel.indices, sel.weights.float())
            bb = self.backbones[ci]
            x = bb.w_in(torch.cat([ports.rms_norm(t[k].float(), None, FP32_EPS) if not k.startswith("__routing")
                                   else t[k] for k in bb.tap_keys], dim=-1))
            pos, seg = _positions(x, ctx), ctx.get("segment_ids")
            for blk in bb.blocks:
                x = blk(x, pos, seg, routing=routing)
            for s in ch["dense_sites"]:
                out[s] = self.dense_heads[ci][ComponentConditioning.key(s)](x)
            last_ffn: RoutedExpertFFN = bb.blocks[-1].ffn  # type: ignore[assignment]
            xn = _norm(x, bb.blocks[-1].n2)
            for s, (layer, c_block) in ch["blocked_sites"].items():
                sel = routing[layer]
                h = last_ffn.expert_hidden(xn, layer, sel)  # [N * k, hidden], token-major jobs
                vals = routed_linear(h, self.expert_heads[head_i], sel, True, last_ffn.fused)  # [N * k, c]
                out[s] = SelectedCI(vals.reshape(*sel.indices.shape[:-1], -1), sel, self.n_experts)
                head_i += 1
        return out

    def parameter_census(self) -> dict[str, int]:
        return census(self)

    def useful_flops_per_position(self) -> int:
        return 2 * sum(p.numel() for p in self.parameters() if p.dim() >= 2)
