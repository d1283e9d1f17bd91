"""Config-driven decoder-only transformer target (Llama / Qwen3 / LlamaSimpleMLP anatomies).

Per block:  resid -> RMSNorm -> q,k,v (RoPE on q,k; optional per-head QK RMS-norm; GQA) -> causal
attention -> o -> +resid -> RMSNorm -> gated MLP `down(silu(gate) * up)` or plain MLP
`down(gelu_tanh(c_fc))` -> +resid;  final RMSNorm -> (tied or untied) head.

Site names follow the reference's grammars: GLU family `layers.{i}.self_attn.{q,k,v,o}_proj`,
`layers.{i}.mlp.{gate,up,down}_proj`; simple-MLP family `h.{i}.attn.{q,k,v,o}_proj`,
`h.{i}.mlp.{c_fc,down_proj}`. Taps / captures: `resid.{b}` (b = 0..n_layer), `attn_in.{i}`,
`attn_out.{i}`, `post_attn.{i}`, `mlp_in.{i}`, `mlp_hidden.{i}`, `{site}.out`, `attn_scores.{i}`.

Two execution paths behind one class: `backend="eager_torch"` (plain torch ops; the oracle, any
device) and `backend="fused_sm100"` (every linear of the target and every decomposed site runs on
the tcgen05 GEMM engine, masks are drawn inside the site kernel's epilogue).

Parity: param_decomp/targets/transformer.py:182-343 (anatomy, site grammar), :622-824 (attention,
MLPs), :1759-1972 (clean / masked forward), :2134-2185 (weight deltas); targets/llama_simple_mlp.py;
targets/lm_output.py:20-88 and targets/losses.py:50-293 (materialised vs streamed output edge).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any

import torch
import torch.nn.functional as F
from torch import Tensor

from param_decomp_b200.config.experiments import TransformerArchConfig
from param_decomp_b200.core.components import ComputeWeights, SiteSpec
from param_decomp_b200.core.decomposed_linear import site_forward, site_forward_split
from param_decomp_b200.core.masking import Masks
from param_decomp_b200.core.model import ForwardResult
from param_decomp_b200.formats.nonlinearity import KVHeads, Neurons, NonlinearityAlignment, QueryHeads
from param_decomp_b200.models import ports

GLU_KINDS = ("q", "k", "v", "o", "gate", "up", "down")
SIMPLE_KINDS = ("q_proj", "k_proj", "v_proj", "o_proj", "c_fc", "down_proj")
ATTN_KINDS = {"q", "k", "v", "o", "q_proj", "k_proj", "v_proj", "o_proj"}


def site_name(family: str, layer: int, kind: str) -> str:
    if family == "simple_mlp":
        return f"h.{layer}.{'attn' if kind in ATTN_KINDS else 'mlp'}.{kind}"
    if kind.startswith(("experts_", "shared_")):
        return f"layers.{layer}.mlp.{kind}"
    return f"layers.{layer}.{'self_attn' if kind in ATTN_KINDS else 'mlp'}.{kind}_proj"


def weight_key(family: str, layer: int, kind: str) -> str:
    return site_name(family, layer, kind) + ".weight"


def _short(kind: str) -> str:
    return kind[:-5] if kind.endswith("_proj") and kind != "down_proj" else ("down" if kind == "down_proj" else kind)


@dataclass
class LMBatch:
    tokens: Tensor  # [B, T] int64/int32
    segment_ids: Tensor | None = None  # [B, T] document ids (block-diagonal causal attention)
    positions: Tensor | None = None  # [B, T] positions within documents

    def to(self, device, non_blocking: bool = False) -> "LMBatch":
        mv = lambda t: None if t is None else t.to(device, non_blocking=non_blocking)  # noqa: E731
        return LMBatch(mv(self.tokens), mv(self.segment_ids), mv(self.positions))


def random_init_weights(arch: TransformerArchConfig, seed: int, dtype: torch.dtype = torch.bfloat16,
                        device: torch.device | str = "cpu") -> dict[str, Tensor]:
    """Seeded GPT-style init: N(0, 0.02) matrices (output projections scaled by 1/sqrt(2 L)), unit norms."""
    g = torch.Generator().manual_seed(seed)
    fam = arch.family
    d, hd = arch.d_model, arch.head_dim or arch.d_model // arch.n_head
    kv = arch.n_kv_head or arch.n_head
    out: dict[str, Tensor] = {}

    def mat(rows: int, cols: int, std: float = 0.02) -> Tensor:
        return (torch.randn(rows, cols, generator=g) * std).to(dtype).to(device)

    out["embed.weight"] = mat(arch.vocab_size, d)
    if arch.positional == "learned":
        out["pos_embed.weight"] = mat(arch.max_seq_len, d)
    resid_std = 0.02 / math.sqrt(2 * arch.n_layer)
    names = (("q_proj", "k_proj", "v_proj", "o_proj") if fam == "simple_mlp" else ("q", "k", "v", "o"))
    for i in range(arch.n_layer):
        out[f"layers.{i}.attn_norm.weight"] = torch.ones(d, dtype=dtype, device=device)
        out[f"layers.{i}.mlp_norm.weight"] = torch.ones(d, dtype=dtype, device=device)
        if arch.norm_kind == "layer":
            out[f"layers.{i}.attn_norm.bias"] = torch.zeros(d, dtype=dtype, device=device)
            out[f"layers.{i}.mlp_norm.bias"] = torch.zeros(d, dtype=dtype, device=device)
        out[weight_key(fam, i, names[0])] = mat(arch.n_head * hd, d)
        out[weight_key(fam, i, names[1])] = mat(kv * hd, d)
        out[weight_key(fam, i, names[2])] = mat(kv * hd, d)
        out[weight_key(fam, i, names[3])] = mat(d, arch.n_head * hd, resid_std)
        if arch.qk_norm:
            out[f"layers.{i}.q_norm.weight"] = torch.ones(hd, dtype=dtype, device=device)
            out[f"layers.{i}.k_norm.weight"] = torch.ones(hd, dtype=dtype, device=device)
        if fam == "simple_mlp":
            out[weight_key(fam, i, "c_fc")] = mat(arch.d_ff, d)
            out[weight_key(fam, i, "down_proj")] = mat(d, arch.d_ff, resid_std)
        else:
            out[weight_key(fam, i, "gate")] = mat(arch.d_ff, d)
            out[weight_key(fam, i, "up")] = mat(arch.d_ff, d)
            out[weight_key(fam, i, "down")] = mat(d, arch.d_ff, resid_std)
    out["final_norm.weight"] = torch.ones(d, dtype=dtype, device=device)
    if arch.norm_kind == "layer":
        out["final_norm.bias"] = torch.zeros(d, dtype=dtype, device=device)
    if not arch.tie_embeddings:
        out["lm_head.weight"] = mat(arch.vocab_size, d)
    return out


def alignment_for(arch: TransformerArchConfig, kind: str) -> NonlinearityAlignment | None:
    """Which side of each matrix faces a nonlinearity, and its unit partition."""
    k = _short(kind)
    kv = arch.n_kv_head or arch.n_head
    if k == "q":
        return NonlinearityAlignment("output", QueryHeads(arch.n_head))
    if k in ("k", "v"):
        return NonlinearityAlignment("output", KVHeads(kv, arch.n_head // kv))
    if k == "o":
        return NonlinearityAlignment("input", QueryHeads(arch.n_head))
    if k in ("gate", "up", "c_fc"):
        return NonlinearityAlignment("output", Neurons())
    if k == "down":
        return NonlinearityAlignment("input", Neurons())
    return None


class TransformerDecomposedModel:
    has_position_axis = True

    def __init__(self, arch: TransformerArchConfig, weights: dict[str, Tensor], site_cs: dict[str, int],
                 backend: str = "eager_torch", attention: str = "flash", n_vocab_chunks: int | None = None,
                 kl_token_chunk: int = 8192) -> None:
        assert arch.family in ("glu_transformer", "simple_mlp", "moe"), arch.family
        self.arch = arch
        self.w = weights
        self.backend = backend
        # the eager backend means library ops end to end: torch's fused attention instead of the hand-written kernel
        self.attention_impl = "sdpa" if (backend == "eager_torch" and attention == "flash") else attention
        self.n_vocab_chunks = n_vocab_chunks
        self.kl_token_chunk = kl_token_chunk
        self.compute_dtype = weights["embed.weight"].dtype
        self.head_dim = arch.head_dim or arch.d_model // arch.n_head
        self.n_kv = arch.n_kv_head or arch.n_head
        self.kinds = SIMPLE_KINDS if arch.family == "simple_mlp" else self._family_kinds()
        specs = []
        self._site_layer_kind: dict[str, tuple[int, str]] = {}
        for i in range(arch.n_layer):
            for kind in self.kinds:
                name = site_name(arch.family, i, kind)
                if name in site_cs:
                    specs.append(self._site_spec(name, kind, site_cs[name]))
                    self._site_layer_kind[name] = (i, kind)
        unknown = set(site_cs) - set(self._site_layer_kind)
        assert not unknown, f"unknown sites {sorted(unknown)[:4]}..."
        self.sites = tuple(specs)
        self._fused_cache: dict[str, Any] = {}

    def _family_kinds(self) -> tuple[str, ...]:
        return GLU_KINDS

    def _site_spec(self, name: str, kind: str, C: int) -> SiteSpec:
        W = self.w[name + ".weight"]
        return SiteSpec(name, W.shape[1], W.shape[0], C, group=kind, alignment=alignment_for(self.arch, kind))

    # -- protocol ---------------------------------------------------------------------------------
    def batch_size(self, batch: LMBatch) -> int:
        return batch.tokens.shape[0]

    def tap_for_site(self, site: str) -> str:
        layer, kind = self._site_layer_kind[site]
        k = _short(kind)
        if k in ("q", "k", "v"):
            return f"attn_in.{layer}"
        if k == "o":
            return f"attn_out.{layer}"
        if k in ("gate", "up", "c_fc"):
            return f"mlp_in.{layer}"
        return f"mlp_hidden.{layer}"

    def target_weight(self, site: str) -> Tensor:
        return self.w[site + ".weight"]

    def layer_of_site(self, site: str) -> int:
        return self._site_layer_kind[site][0]

    def block_tap_widths(self, layer: int) -> dict[str, int]:
        """Every site-input vector the block computes (each physical vector once)."""
        a = self.arch
        return {f"attn_in.{layer}": a.d_model, f"attn_out.{layer}": a.n_head * self.head_dim,
                f"mlp_in.{layer}": a.d_model, f"mlp_hidden.{layer}": a.d_ff}

    def head_weight(self) -> Tensor:
        return self.w["embed.weight"] if self.arch.tie_embeddings else self.w["lm_head.weight"]

    # -- building blocks ----------------------------------------------------------------------------
    def _linear(self, x: Tensor, name: str, weights: ComputeWeights | None, masks: Masks | None) -> Tensor:
        W = self.w[name + ".weight"]
        decomposed = weights is not None and masks is not None and name in masks and name in weights.V
        split = getattr(self, "component_group", None) if decomposed else None
        if self.backend == "fused_sm100" and x.is_cuda:
            from param_decomp_b200.ops import linear as fused

            if decomposed and split is not None:
                return fused.site_split(x, weights, name, W, masks[name], split)  # type: ignore[index]
            if decomposed:
                return fused.site(x, weights, name, W, masks[name])  # type: ignore[index]
            return fused.linear(x, W)
        if decomposed:
            V, U = weights.site(name)  # type: ignore[union-attr]
            if split is not None:
                return site_forward_split(x, V, U, W, masks[name], split)  # type: ignore[index]
            return site_forward(x, V, U, W, masks[name])  # type: ignore[index]
        return F.linear(x, W)

    def split_components(self, group: Any) -> None:
        """Split every site's component axis over the ranks of `group` (the mesh's `tp` axis): from here on
        `sites` describes this rank's `C / W` components and `global_sites` the whole sites, which is what
        the CI function, the masks and the adversaries see (param_decomp/core/placement.py:1040-1048)."""
        import torch.distributed as dist

        world = dist.get_world_size(group)
        assert all(not s.blocked for s in self.sites), "blocked sites split by expert, not by component"
        for s in self.sites:
            assert s.C % (8 * world) == 0, f"{s.name}: C={s.C} must be a multiple of 8 x {world} ranks"
        self._global_sites = self.sites
        self.sites = tuple(SiteSpec(s.name, s.d_in, s.d_out, s.C // world, group=s.group, alignment=s.alignment)
                           for s in self.sites)
        self.component_group = group

    @property
    def global_sites(self) -> tuple[SiteSpec, ...]:
        return getattr(self, "_global_sites", self.sites)

    # the three bandwidth-bound ops of a block: hand-written kernels on the fused backend
    def _fused(self, x: Tensor) -> bool:
        return self.backend == "fused_sm100" and x.is_cuda and x.dtype == torch.bfloat16

    def _norm(self, x: Tensor, w: Tensor, b: Tensor | None = None) -> Tensor:
        if getattr(self.arch, "norm_kind", "rms") == "layer":
            # LayerNorm with bias (GPT-2 style): statistics in fp32, scale and shift in the activation dtype
            # (param_decomp/pretrain/models.py:182-188)
            xf = x.float()
            mean = xf.mean(-1, keepdim=True)
            var = (xf - mean).pow(2).mean(-1, keepdim=True)
            y = ((xf - mean) * torch.rsqrt(var + self.arch.rms_eps)).to(x.dtype) * w.to(x.dtype)
            return y + b.to(x.dtype) if b is not None else y
        if self._fused(x):
            from param_decomp_b200.ops import elementwise as ew

            return ew.rms_norm(x, w, self.arch.rms_eps)
        return ports.rms_norm(x, w, self.arch.rms_eps)

    def _rope(self, x: Tensor, cos: Tensor, sin: Tensor, shared_positions: bool) -> Tensor:
        if getattr(self.arch, "positional", "rope") == "learned":
            return x  # positions entered with the embeddings
        if self._fused(x) and shared_positions and cos.shape[-1] == x.shape[-1]:
            from param_decomp_b200.ops import elementwise as ew

            half = x.shape[-1] // 2
            return ew.rope(x, cos[0, :, :half].contiguous(), sin[0, :, :half].contiguous())
        return ports.apply_rope(x, cos, sin)

    def _swiglu(self, gate: Tensor, up: Tensor) -> Tensor:
        if self._fused(gate):
            from param_decomp_b200.ops import elementwise as ew

            return ew.swiglu(gate, up)
        return ports.swiglu(gate, up)

    def _block(self, i: int, resid: Tensor, cos: Tensor, sin: Tensor, batch: LMBatch, weights, masks,
               taps: dict[str, Tensor] | None, captures: dict[str, Tensor], want: set[str], aux: dict) -> Tensor:
        a, fam, eps = self.arch, self.arch.family, self.arch.rms_eps
        B, T, _ = resid.shape
        names = (("q_proj", "k_proj", "v_proj", "o_proj") if fam == "simple_mlp" else ("q", "k", "v", "o"))

        def lin(x: Tensor, kind: str) -> Tensor:
            name = site_name(fam, i, kind)
            y = self._linear(x, name, weights, masks)
            if name + ".out" in want:
                captures[name + ".out"] = y
            return y

        # Sequence-parallel masked pass: `resid` is this rank's `[B, T / W, d]` positions. Norms and residual adds
        # run on the shard; each sublayer gathers its normed input to the whole sequence, and takes its own
        # positions of the sublayer's (group-summed) output back.
        sp = aux.get("sequence_group")
        if sp is not None:
            from param_decomp_b200.parallel.group_ops import gather_sequence, slice_sequence

            T = T * aux["sequence_world"]
        x = self._norm(resid, self.w[f"layers.{i}.attn_norm.weight"], self.w.get(f"layers.{i}.attn_norm.bias"))
        if sp is not None:
            x = gather_sequence(x, sp)
        if taps is not None:
            taps[f"attn_in.{i}"] = x
        lanes = getattr(self, "lanes", None)
        if lanes is not None and x.is_cuda:  # independent products of one input: side by side on the device
            q, k, v = lanes.run([lambda: lin(x, names[0]), lambda: lin(x, names[1]), lambda: lin(x, names[2])])
        else:
            q, k, v = lin(x, names[0]), lin(x, names[1]), lin(x, names[2])
        q = q.view(B, T, a.n_head, self.head_dim)
        k = k.view(B, T, self.n_kv, self.head_dim)
        v = v.view(B, T, self.n_kv, self.head_dim)
        if a.qk_norm:
            q = ports.rms_norm(q, self.w[f"layers.{i}.q_norm.weight"], eps)
            k = ports.rms_norm(k, self.w[f"layers.{i}.k_norm.weight"], eps)
        shared = batch.positions is None
        q, k = self._rope(q, cos, sin, shared), self._rope(k, cos, sin, shared)
        if f"attn_scores.{i}" in want:
            from param_decomp_b200.ops.attention_kl import capture_scores

            captures[f"attn_scores.{i}"] = capture_scores(q, k, True, batch.segment_ids, self._fused(q))
        att = ports.sdpa(q, k, v, True, batch.segment_ids, self.attention_impl).reshape(B, T, a.n_head * self.head_dim)
        if taps is not None:
            taps[f"attn_out.{i}"] = att
        o = lin(att, names[3])
        resid = resid + (slice_sequence(o, sp) if sp is not None else o)
        if f"post_attn.{i}" in want:
            captures[f"post_attn.{i}"] = resid
        x = self._norm(resid, self.w[f"layers.{i}.mlp_norm.weight"], self.w.get(f"layers.{i}.mlp_norm.bias"))
        if sp is not None:
            x = gather_sequence(x, sp)
        if taps is not None:
            taps[f"mlp_in.{i}"] = x
        aux["capture_sink"] = (captures, want)  # for MLP variants that have captures of their own (router logits)
        m = self._mlp(i, x, lin, taps, weights, masks, aux)
        return resid + (slice_sequence(m, sp) if sp is not None else m)

    def _mlp(self, i: int, x: Tensor, lin, taps: dict[str, Tensor] | None, weights, masks, aux: dict) -> Tensor:
        if self.arch.family == "simple_mlp":
            h = ports.gelu_tanh(lin(x, "c_fc"))  # the tanh form, as the reference's plain MLP (targets/transformer.py:802-809)
            down = "down_proj"
        else:
            lanes = getattr(self, "lanes", None)
            if lanes is not None and x.is_cuda:
                g, u = lanes.run([lambda: lin(x, "gate"), lambda: lin(x, "up")])
            else:
                g, u = lin(x, "gate"), lin(x, "up")
            h = self._swiglu(g, u)
            down = "down"
        if taps is not None:
            taps[f"mlp_hidden.{i}"] = h
        return lin(h, down)

    def _run(self, batch: LMBatch, weights, masks, capture: tuple[str, ...], want_taps: bool,
             aux: dict | None = None) -> ForwardResult:
        a = self.arch
        aux = {} if aux is None else aux
        want = set(capture)
        tokens = batch.tokens
        B, T = tokens.shape
        resid = F.embedding(tokens.long(), self.w["embed.weight"])
        pos = batch.positions if batch.positions is not None else torch.arange(T, device=tokens.device)[None]
        if getattr(a, "positional", "rope") == "learned":
            resid = resid + F.embedding(pos.long(), self.w["pos_embed.weight"])
        cos, sin = ports.rope_cos_sin(pos, self.head_dim, a.rope_theta, a.rope_scaling)
        taps: dict[str, Tensor] | None = {} if want_taps else None
        captures: dict[str, Tensor] = {}
        sp = None
        if (masks is not None and getattr(self, "sequence_parallel", False) and not want and not want_taps
                and getattr(self, "component_group", None) is not None):
            # `runtime.sequence_sharding: sequence_parallel`: the MASKED passes carry the residual stream
            # position-sharded over the tp group between blocks; clean passes keep it whole
            # (param_decomp/core/placement.py:273-287, targets/qwen36_moe.py:3100-3120).
            import torch.distributed as dist

            from param_decomp_b200.parallel.group_ops import gather_sequence, slice_sequence

            # (a pass that captures activations keeps the whole-sequence residual: tap buffers are whole-sequence)
            sp = self.component_group
            aux["sequence_group"], aux["sequence_world"] = sp, dist.get_world_size(sp)
            resid = slice_sequence(resid, sp)
        for i in range(a.n_layer):
            if taps is not None:
                taps[f"resid.{i}"] = resid
            if f"resid.{i}" in want:
                captures[f"resid.{i}"] = resid
            resid = self._block(i, resid, cos, sin, batch, weights, masks, taps, captures, want, aux)
        if taps is not None:
            taps[f"resid.{a.n_layer}"] = resid
        if f"resid.{a.n_layer}" in want:
            captures[f"resid.{a.n_layer}"] = resid
        final = self._norm(resid, self.w["final_norm.weight"], self.w.get("final_norm.bias"))
        if sp is not None:  # the output edge sees the whole sequence: a position-sharded residual never leaves here
            final = gather_sequence(final, sp)
            aux.pop("sequence_group"), aux.pop("sequence_world")
        return ForwardResult(output=final, taps=taps or {}, captures=captures, aux=aux)

    def clean_forward(self, batch: LMBatch, capture: tuple[str, ...] = ()) -> ForwardResult:
        out = self._run(batch, None, None, capture, want_taps=True)
        # the clean side of the KL: keep what the loss needs, once per step
        out.aux["clean_stats"] = self._clean_logit_stats(out.output)
        out.aux["segment_ids"], out.aux["positions"] = batch.segment_ids, batch.positions
        return out

    def masked_forward(self, weights: ComputeWeights, batch: LMBatch, masks: Masks,
                       capture: tuple[str, ...] = (), clean: ForwardResult | None = None) -> ForwardResult:
        return self._run(batch, weights, masks, capture, want_taps=False)

    def logits(self, final_hidden: Tensor) -> Tensor:
        return F.linear(final_hidden, self.head_weight())

    # -- output edge: KL(clean || masked) over the vocabulary ---------------------------------------
    def _clean_logit_stats(self, hidden: Tensor) -> dict[str, Tensor]:
        """Fused backend: the clean logits are formed once per step and reused by every draw."""
        if self.backend == "fused_sm100" and hidden.is_cuda and self.n_vocab_chunks is None:
            from param_decomp_b200.ops import vocab_kl

            return {"logits": vocab_kl.padded_logits(hidden.reshape(-1, hidden.shape[-1]), self.head_weight())}
        return {}  # streamed output edge: no `[positions, vocab]` tensor is ever kept

    def recon_loss(self, clean: ForwardResult, masked: ForwardResult) -> Tensor:
        """Mean over positions of `KL(softmax(clean logits) || softmax(masked logits))`.
        Logits are never held for the whole batch: positions are processed in chunks and each chunk
        is recomputed in the backward pass (`ops/vocab_kl.py` is the fused kernel of this loss)."""
        hc = clean.output.reshape(-1, clean.output.shape[-1])
        hm = masked.output.reshape(-1, masked.output.shape[-1])
        if self.backend == "fused_sm100" and hm.is_cuda:
            from param_decomp_b200.ops import vocab_kl

            if self.n_vocab_chunks is not None:  # `output_edge: streamed`: chunks of positions, logits never whole
                rows = (-(-hm.shape[0] // self.n_vocab_chunks) + 127) // 128 * 128
                return vocab_kl.kl_from_hidden_streamed(hc, hm, self.head_weight(), rows)
            return vocab_kl.kl_from_hidden(clean.aux["clean_stats"]["logits"], hm, self.head_weight())
        return chunked_kl_from_hidden(hc, hm, self.head_weight(), self.kl_token_chunk)

    def ce_loss(self, out: ForwardResult, tokens: Tensor) -> Tensor:
        """Next-token cross entropy (evaluation)."""
        logits = self.logits(out.output[:, :-1]).float()
        return F.cross_entropy(logits.reshape(-1, logits.shape[-1]), tokens[:, 1:].reshape(-1).long())

    def to(self, device) -> "TransformerDecomposedModel":
        self.w = {k: v.to(device) for k, v in self.w.items()}
        return self


class _ChunkKL(torch.autograd.Function):
    """KL of one chunk of positions from final hidden states; recomputes the chunk's logits in
    backward, so at most `chunk x vocab` logits exist at a time."""

    @staticmethod
    def forward(ctx, hc: Tensor, hm: Tensor, head: Tensor) -> Tensor:  # type: ignore[override]
        lc = F.linear(hc, head).float()
        lm = F.linear(hm, head).float()
        logp_c = F.log_softmax(lc, dim=-1)
        logp_m = F.log_softmax(lm, dim=-1)
        ctx.save_for_backward(hc, hm, head)
        return (logp_c.exp() * (logp_c - logp_m)).sum()

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        hc, hm, head = ctx.saved_tensors
        p_c = torch.softmax(F.linear(hc, head).float(), dim=-1)
        p_m = torch.softmax(F.linear(hm, head).float(), dim=-1)
        dlogits = ((p_m - p_c) * g).to(hm.dtype)  # d KL / d masked logits
        return None, dlogits @ head, None


def chunked_kl_from_hidden(hc: Tensor, hm: Tensor, head: Tensor, chunk: int) -> Tensor:
    n = hc.shape[0]
    total = hm.new_zeros((), dtype=torch.float32)
    for s in range(0, n, chunk):
        total = total + _ChunkKL.apply(hc[s:s + chunk], hm[s:s + chunk], head)
    return total / n
