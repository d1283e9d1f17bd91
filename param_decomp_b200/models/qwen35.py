"""Qwen3.5 / 3.6-MoE style hybrid decoder target.

Layer `i` = `x + mixer(norm(x))`, then `x + moe(norm(x))`. The mixer is gated full attention when
`(i + 1) % full_attention_interval == 0` and a gated DeltaNet (linear attention) otherwise:

  DeltaNet   q,k,v,z,b,a projections -> causal depthwise conv + SiLU on q,k,v -> l2-normalised q,k
             (repeated to the value heads) -> gated delta rule with `g = -exp(A_log) softplus(a + dt_bias)`,
             `beta = sigmoid(b)` -> RMSNorm(core) * silu(z) -> out projection
  attention  q projection emits query|gate per head; zero-centred RMSNorm on q and k heads; RoPE on
             the first `partial_rotary_factor * head_dim` dims; causal GQA attention; `core * sigmoid(gate)`;
             o projection
  MoE        fp32 router softmax -> top-k (a masked pass is pinned to the clean pass's indices, its
             weights come from its own softmax renormalised over those indices) -> routed SwiGLU experts
             + `sigmoid(x w_sg) * shared expert`

All norms but the DeltaNet output norm store zero-centred weights (`1 + w`). Seventeen decomposable
matrix kinds in computation order; the `experts_*` kinds are blocked sites (one component block per
expert, narrow CI), everything else is dense.

Parity: param_decomp/targets/qwen36_moe.py:241-328 (config), :331-443 (site grammar), :539-569 (dims),
:1562-1693 (DeltaNet), :1712-1813 (gated attention), :2923-3046 (MoE forward); math in
param_decomp/target_ports/qwen3_5_moe.py.
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.nn.functional as F
from torch import Tensor

from param_decomp_b200.config.experiments import TransformerArchConfig
from param_decomp_b200.core.components import BlockSelection, SiteSpec
from param_decomp_b200.formats.nonlinearity import KVHeads, Neurons, NonlinearityAlignment, QueryHeads
from param_decomp_b200.models import moe, ports
from param_decomp_b200.models import transformer as tf
from param_decomp_b200.ops.grouped import repeat_rows

KIND_ORDER = ("gdn_q", "gdn_k", "gdn_v", "gdn_z", "gdn_b", "gdn_a", "gdn_out", "attn_q", "attn_k", "attn_v", "attn_o",
              "experts_gate", "experts_up", "experts_down", "shared_gate", "shared_up", "shared_down")
SITE_SUFFIX = {
    "gdn_q": "linear_attn.in_proj_qkv.q", "gdn_k": "linear_attn.in_proj_qkv.k", "gdn_v": "linear_attn.in_proj_qkv.v",
    "gdn_z": "linear_attn.in_proj_z", "gdn_b": "linear_attn.in_proj_b", "gdn_a": "linear_attn.in_proj_a",
    "gdn_out": "linear_attn.out_proj", "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj",
    "attn_v": "self_attn.v_proj", "attn_o": "self_attn.o_proj", "experts_gate": "mlp.experts.gate_proj",
    "experts_up": "mlp.experts.up_proj", "experts_down": "mlp.experts.down_proj",
    "shared_gate": "mlp.shared_expert.gate_proj", "shared_up": "mlp.shared_expert.up_proj",
    "shared_down": "mlp.shared_expert.down_proj",
}  # fmt: skip
EXPERT_KINDS = ("experts_gate", "experts_up", "experts_down")
GDN_KINDS = tuple(k for k in KIND_ORDER if k.startswith("gdn_"))
ATTN_KINDS = tuple(k for k in KIND_ORDER if k.startswith("attn_"))


def site_name(layer: int, kind: str) -> str:
    return f"layers.{layer}.{SITE_SUFFIX[kind]}"


def is_full_attention(arch: TransformerArchConfig, layer: int) -> bool:
    return (layer + 1) % arch.full_attention_interval == 0


def layers_of_kind(arch: TransformerArchConfig, kind: str) -> tuple[int, ...]:
    """Which layers carry a matrix kind is a fact of the architecture (one mixer per layer)."""
    if kind in GDN_KINDS:
        return tuple(i for i in range(arch.n_layer) if not is_full_attention(arch, i))
    if kind in ATTN_KINDS:
        return tuple(i for i in range(arch.n_layer) if is_full_attention(arch, i))
    return tuple(range(arch.n_layer))


def site_dims(a: TransformerArchConfig, kind: str) -> tuple[int, int]:
    """(d_in, d_out) of one site matrix; expert kinds give the per-expert matrix."""
    d = a.d_model
    kd, vd = a.linear_num_key_heads * a.linear_key_head_dim, a.linear_num_value_heads * a.linear_value_head_dim
    kv = a.n_kv_head or a.n_head
    return {
        "gdn_q": (d, kd), "gdn_k": (d, kd), "gdn_v": (d, vd), "gdn_z": (d, vd),
        "gdn_b": (d, a.linear_num_value_heads), "gdn_a": (d, a.linear_num_value_heads), "gdn_out": (vd, d),
        "attn_q": (d, 2 * a.n_head * a.head_dim), "attn_k": (d, kv * a.head_dim), "attn_v": (d, kv * a.head_dim),
        "attn_o": (a.n_head * a.head_dim, d), "experts_gate": (d, a.d_ff), "experts_up": (d, a.d_ff),
        "experts_down": (a.d_ff, d), "shared_gate": (d, a.shared_expert_intermediate),
        "shared_up": (d, a.shared_expert_intermediate), "shared_down": (a.shared_expert_intermediate, d),
    }[kind]  # fmt: skip


def alignment_for(a: TransformerArchConfig, kind: str) -> NonlinearityAlignment | None:
    kv = a.n_kv_head or a.n_head
    if kind == "attn_q":
        return NonlinearityAlignment("output", QueryHeads(a.n_head))
    if kind in ("attn_k", "attn_v"):
        return NonlinearityAlignment("output", KVHeads(kv, a.n_head // kv))
    if kind == "attn_o":
        return NonlinearityAlignment("input", QueryHeads(a.n_head))
    if kind in ("shared_gate", "shared_up", "experts_gate", "experts_up"):
        return NonlinearityAlignment("output", Neurons())
    if kind in ("shared_down", "experts_down"):
        return NonlinearityAlignment("input", Neurons())
    return None


def random_init_qwen35_weights(a: TransformerArchConfig, seed: int, dtype=torch.bfloat16, device="cpu") -> dict[str, Tensor]:
    g = torch.Generator().manual_seed(seed)
    d, E = a.d_model, a.n_experts
    resid_std = 0.02 / math.sqrt(2 * a.n_layer)

    def mat(*shape: int, std: float = 0.02) -> Tensor:
        return (torch.randn(*shape, generator=g) * std).to(dtype).to(device)

    w: dict[str, Tensor] = {"embed.weight": mat(a.vocab_size, d), "lm_head.weight": mat(a.vocab_size, d),
                            "final_norm.weight": torch.zeros(d, dtype=dtype, device=device)}
    Hv, K = a.linear_num_value_heads, a.linear_conv_kernel_dim
    for i in range(a.n_layer):
        w[f"layers.{i}.attn_norm.weight"] = torch.zeros(d, dtype=dtype, device=device)
        w[f"layers.{i}.mlp_norm.weight"] = torch.zeros(d, dtype=dtype, device=device)
        kinds = ATTN_KINDS if is_full_attention(a, i) else GDN_KINDS
        for kind in kinds:
            din, dout = site_dims(a, kind)
            w[site_name(i, kind) + ".weight"] = mat(dout, din, std=resid_std if kind in ("gdn_out", "attn_o") else 0.02)
        if is_full_attention(a, i):
            w[f"layers.{i}.self_attn.q_norm.weight"] = torch.zeros(a.head_dim, dtype=dtype, device=device)
            w[f"layers.{i}.self_attn.k_norm.weight"] = torch.zeros(a.head_dim, dtype=dtype, device=device)
        else:
            for nm, kind in (("q", "gdn_q"), ("k", "gdn_k"), ("v", "gdn_v")):
                w[f"layers.{i}.linear_attn.conv_{nm}.weight"] = mat(site_dims(a, kind)[1], K, std=0.5)
            w[f"layers.{i}.linear_attn.A_log"] = torch.log(torch.rand(Hv, generator=g) * 15 + 1).to(device)
            w[f"layers.{i}.linear_attn.dt_bias"] = torch.ones(Hv, device=device)
            w[f"layers.{i}.linear_attn.norm.weight"] = torch.ones(a.linear_value_head_dim, dtype=dtype, device=device)
        w[f"layers.{i}.mlp.router.weight"] = mat(E, d)
        w[site_name(i, "experts_gate") + ".weight"] = mat(E, a.d_ff, d)
        w[site_name(i, "experts_up") + ".weight"] = mat(E, a.d_ff, d)
        w[site_name(i, "experts_down") + ".weight"] = mat(E, d, a.d_ff, std=resid_std)
        for kind in ("shared_gate", "shared_up", "shared_down"):
            din, dout = site_dims(a, kind)
            w[site_name(i, kind) + ".weight"] = mat(dout, din, std=resid_std if kind == "shared_down" else 0.02)
        w[f"layers.{i}.mlp.shared_expert_gate.weight"] = mat(1, d)
    return w


class Qwen35DecomposedModel(moe.MoEDecomposedModel):
    """`DecomposedModel` of the hybrid decoder; expert banks run through the MoE model's job machinery."""

    def __init__(self, arch: TransformerArchConfig, weights: dict[str, Tensor], site_cs: dict[str, int],
                 backend: str = "eager_torch", attention: str = "flash", ep: Any = None, **kw: Any) -> None:
        assert arch.family == "qwen35_moe"
        self.ep = ep
        tf.TransformerDecomposedModel.__init__(self, self._as_moe(arch), weights, {}, backend=backend,
                                               attention=attention, **kw)
        self.arch = arch
        specs = []
        self._site_layer_kind = {}
        for i in range(arch.n_layer):
            for kind in KIND_ORDER:
                name = site_name(i, kind)
                if name in site_cs:
                    assert i in layers_of_kind(arch, kind), f"layer {i} has no {kind} matrix"
                    specs.append(self._site_spec(name, kind, site_cs[name]))
                    self._site_layer_kind[name] = (i, kind)
        unknown = set(site_cs) - set(self._site_layer_kind)
        assert not unknown, f"unknown sites {sorted(unknown)[:4]}"
        self.sites = tuple(specs)
        self.rotary_dim = int(arch.head_dim * arch.partial_rotary_factor)

    @staticmethod
    def _as_moe(arch: TransformerArchConfig) -> TransformerArchConfig:
        return arch.model_copy(update={"family": "moe"})

    def _site_spec(self, name: str, kind: str, C: int) -> SiteSpec:
        W = self.w[name + ".weight"]
        if kind in EXPERT_KINDS:
            E = W.shape[0]
            assert C % E == 0, f"{name}: C={C} must be a multiple of n_experts={E}"
            return SiteSpec(name, W.shape[2], W.shape[1], C, group=kind, n_blocks=E,
                            alignment=alignment_for(self.arch, kind), routed=True)
        return SiteSpec(name, W.shape[1], W.shape[0], C, group=kind, alignment=alignment_for(self.arch, kind))

    def tap_for_site(self, site: str) -> str:
        layer, kind = self._site_layer_kind[site]
        if kind in ("gdn_out", "attn_o"):
            return f"attn_out.{layer}"
        if kind == "shared_down":
            return f"shared_hidden.{layer}"
        if kind.startswith(("gdn_", "attn_")):
            return f"attn_in.{layer}"
        return f"mlp_in.{layer}"

    def block_tap_widths(self, layer: int) -> dict[str, int]:
        a = self.arch
        core = a.n_head * a.head_dim if is_full_attention(a, layer) else a.linear_num_value_heads * a.linear_value_head_dim
        return {f"attn_in.{layer}": a.d_model, f"attn_out.{layer}": core, f"mlp_in.{layer}": a.d_model,
                f"shared_hidden.{layer}": a.shared_expert_intermediate}

    def expert_site_names(self, layer: int) -> list[str]:
        return [site_name(layer, k) for k in EXPERT_KINDS]

    def _linear(self, x: Tensor, name: str, weights, masks) -> Tensor:
        W = self.w[name + ".weight"]
        if W.dim() == 2 and (W.shape[0] % 8 or W.shape[1] % 8) and self.backend == "fused_sm100":
            # per-head scalars (`gdn_a`, `gdn_b`): rows narrower than a 16-byte TMA pitch stay on plain ops
            decomposed = weights is not None and masks is not None and name in masks and name in weights.V
            if decomposed:
                from param_decomp_b200.core.decomposed_linear import site_forward

                V, U = weights.site(name)
                return site_forward(x, V, U, W, masks[name].materialize())
            return F.linear(x, W)
        return super()._linear(x, name, weights, masks)

    # -- building blocks --------------------------------------------------------------------------
    def _norm(self, x: Tensor, w: Tensor) -> Tensor:
        return ports.rms_norm(x, w, self.arch.rms_eps, zero_centered=True)

    def _deltanet(self, i: int, x: Tensor, lin) -> Tensor:
        a = self.arch
        B, T, _ = x.shape
        Hk, Hv, dk, dv = a.linear_num_key_heads, a.linear_num_value_heads, a.linear_key_head_dim, a.linear_value_head_dim
        pre = f"layers.{i}.linear_attn."
        q = self._conv(lin(x, "gdn_q"), self.w[pre + "conv_q.weight"]).view(B, T, Hk, dk)
        k = self._conv(lin(x, "gdn_k"), self.w[pre + "conv_k.weight"]).view(B, T, Hk, dk)
        v = self._conv(lin(x, "gdn_v"), self.w[pre + "conv_v.weight"]).view(B, T, Hv, dv)
        z = lin(x, "gdn_z").view(B, T, Hv, dv)
        beta = torch.sigmoid(lin(x, "gdn_b"))
        g = -torch.exp(self.w[pre + "A_log"].float()) * F.softplus(lin(x, "gdn_a").float() + self.w[pre + "dt_bias"].float())
        rep = Hv // Hk
        if rep > 1:
            q, k = q.repeat_interleave(rep, dim=2), k.repeat_interleave(rep, dim=2)
        kern = a.delta_rule_kernel if self._fused(x) or a.delta_rule_kernel != "cuda" else "chunkwise"
        core = ports.gated_delta_rule(q, k, v, g, beta, kern)
        core = ports.gated_rms_norm(core, z, self.w[pre + "norm.weight"], a.rms_eps)
        return core.reshape(B, T, Hv * dv)

    def _conv(self, x: Tensor, w: Tensor) -> Tensor:
        if self._fused(x):
            from param_decomp_b200.ops import delta_rule

            if delta_rule.conv_supported(x, w):
                return delta_rule.causal_conv1d_silu(x, w)
        return ports.causal_depthwise_conv1d_silu(x, w)

    def _gated_attention(self, i: int, x: Tensor, lin, batch: tf.LMBatch, cos: Tensor, sin: Tensor,
                         captures: dict[str, Tensor], want: set[str]) -> Tensor:
        a, eps = self.arch, self.arch.rms_eps
        B, T, _ = x.shape
        kv, hd = a.n_kv_head or a.n_head, a.head_dim
        qg = lin(x, "attn_q").view(B, T, a.n_head, 2 * hd)
        q, gate = qg[..., :hd], qg[..., hd:]
        q = ports.rms_norm(q, self.w[f"layers.{i}.self_attn.q_norm.weight"], eps, zero_centered=True)
        k = ports.rms_norm(lin(x, "attn_k").view(B, T, kv, hd), self.w[f"layers.{i}.self_attn.k_norm.weight"], eps,
                           zero_centered=True)
        v = lin(x, "attn_v").view(B, T, kv, hd)
        q, k = ports.apply_partial_rope(q, cos, sin), ports.apply_partial_rope(k, cos, sin)
        if f"attn_scores.{i}" in want:
            from param_decomp_b200.ops.attention_kl import capture_scores

            captures[f"attn_scores.{i}"] = capture_scores(q, k, True, batch.segment_ids, self._fused(q))
        out = ports.sdpa(q.contiguous(), k.contiguous(), v.contiguous(), True, batch.segment_ids, self.attention_impl)
        return (out.float() * torch.sigmoid(gate.float())).to(x.dtype).reshape(B, T, a.n_head * hd)

    def _block(self, i: int, resid: Tensor, cos: Tensor, sin: Tensor, batch: tf.LMBatch, weights, masks,
               taps: dict[str, Tensor] | None, captures: dict[str, Tensor], want: set[str], aux: dict) -> Tensor:
        def lin(x: Tensor, kind: str) -> Tensor:
            name = site_name(i, kind)
            y = self._linear(x, name, weights, masks)
            if name + ".out" in want:
                captures[name + ".out"] = y
            return y

        x = self._norm(resid, self.w[f"layers.{i}.attn_norm.weight"])
        if taps is not None:
            taps[f"attn_in.{i}"] = x
        if is_full_attention(self.arch, i):
            core = self._gated_attention(i, x, lin, batch, cos, sin, captures, want)
            out_kind = "attn_o"
        else:
            core = self._deltanet(i, x, lin)
            out_kind = "gdn_out"
        if taps is not None:
            taps[f"attn_out.{i}"] = core
        resid = resid + lin(core, out_kind)
        if f"post_attn.{i}" in want:
            captures[f"post_attn.{i}"] = resid
        x = self._norm(resid, self.w[f"layers.{i}.mlp_norm.weight"])
        if taps is not None:
            taps[f"mlp_in.{i}"] = x
        return resid + self._moe(i, x, lin, taps, weights, masks, aux, captures, want)

    def _moe(self, i: int, x: Tensor, lin, taps, weights, masks, aux: dict, captures: dict[str, Tensor],
             want: set[str]) -> Tensor:
        a = self.arch
        B, T, d = x.shape
        xt = x.reshape(B * T, d)
        logits = F.linear(xt.float(), self.w[f"layers.{i}.mlp.router.weight"].float())
        probs = torch.softmax(logits, dim=-1)
        if f"router_logits.{i}" in want:
            captures[f"router_logits.{i}"] = logits.view(B, T, -1)
        if f"router_probs.{i}" in want:
            captures[f"router_probs.{i}"] = probs.view(B, T, -1)
        pinned = aux.get("pinned_routing")
        idx = pinned[i].indices.reshape(B * T, -1) if pinned is not None else probs.topk(a.experts_per_token, dim=-1).indices
        sel_w = probs.gather(-1, idx)
        sel_w = sel_w / sel_w.sum(-1, keepdim=True)
        sel = BlockSelection(idx.reshape(B, T, -1), sel_w.reshape(B, T, -1))
        if pinned is None:
            aux.setdefault("routing", {})[i] = sel
        k = idx.shape[-1]
        token_of_job = torch.arange(B * T, device=x.device).repeat_interleave(k)
        slot_of_job = torch.arange(k, device=x.device).repeat(B * T)
        expert_of_job = idx.reshape(-1)
        if self.ep is None and self._fused(xt):
            routed = self.expert_tokens(i, xt, pinned[i].indices if pinned is not None else sel.indices, sel_w, weights,
                                        masks, token_of_job, slot_of_job).reshape(B, T, d)
        elif self.ep is not None and self.ep.fast_allreduce(self, xt):
            routed = self.ep.run_tokens_allreduce(self, i, xt, pinned[i].indices if pinned is not None else sel.indices,
                                                  sel_w, weights, masks, token_of_job, slot_of_job).reshape(B, T, d)
        elif self.ep is not None:
            y_jobs = self.ep.run_experts(self, i, xt, expert_of_job, token_of_job, slot_of_job, weights, masks)
        else:
            order, bounds = expert_of_job, [0]
            if not self._fused(xt):
                order = expert_of_job.argsort(stable=True)
                for n in torch.bincount(expert_of_job, minlength=a.n_experts).tolist():
                    bounds.append(bounds[-1] + n)
            y_jobs = self.expert_jobs(i, repeat_rows(xt, k), expert_of_job, order, bounds, weights, masks, token_of_job,
                                      slot_of_job, routing_indices=(pinned[i].indices if pinned is not None else sel.indices))
        if not self._fused(xt) or (self.ep is not None and not self.ep.fast_allreduce(self, xt)):
            routed = (y_jobs.reshape(B * T, k, d) * sel_w.reshape(B * T, k, 1).to(y_jobs.dtype)).sum(1).reshape(B, T, d)
        h = self._swiglu(lin(x, "shared_gate"), lin(x, "shared_up"))
        if taps is not None:
            taps[f"shared_hidden.{i}"] = h
        shared = lin(h, "shared_down")
        sg = torch.sigmoid(F.linear(x.float(), self.w[f"layers.{i}.mlp.shared_expert_gate.weight"].float()))
        return routed + (sg * shared.float()).to(x.dtype)

    def expert_tokens(self, i: int, xt: Tensor, indices: Tensor, route_w: Tensor, weights, masks,
                      token_of_job: Tensor, slot_of_job: Tensor, layout=None) -> Tensor:
        """Fused single-rank path: tokens `[N, d]` fan out to padded sorted job rows, run gate / up / down on
        the grouped kernels and come back as the routing-weighted sum per token."""
        from param_decomp_b200.ops.grouped import JobLayout

        n = lambda kind: site_name(i, kind)  # noqa: E731
        k = indices.shape[-1]
        if layout is None:  # (an expert group passes the layout of its own experts' jobs)
            layout = JobLayout.cached(indices, self.w[n("experts_gate") + ".weight"].shape[0])
        xs = layout.expand_tokens(xt, k)
        gate = self._grouped_site(n("experts_gate"), xs, layout, weights, masks, token_of_job, slot_of_job)
        up = self._grouped_site(n("experts_up"), xs, layout, weights, masks, token_of_job, slot_of_job)
        down = self._grouped_site(n("experts_down"), self._swiglu(gate, up), layout, weights, masks, token_of_job,
                                  slot_of_job)
        return layout.combine(down, route_w.reshape(-1, k))

    def expert_jobs(self, i: int, x_jobs: Tensor, expert_of_job: Tensor, order: Tensor, bounds: list[int], weights,
                    masks, token_of_job: Tensor, slot_of_job: Tensor, routing_indices: Tensor | None = None) -> Tensor:
        n = lambda kind: site_name(i, kind)  # noqa: E731
        if self._fused(x_jobs):
            from param_decomp_b200.ops.grouped import JobLayout

            n_e = self.w[n("experts_gate") + ".weight"].shape[0]
            layout = JobLayout.cached(routing_indices, n_e) if routing_indices is not None else JobLayout.build(expert_of_job, n_e)
            xs = layout.scatter_rows(x_jobs)
            gate = self._grouped_site(n("experts_gate"), xs, layout, weights, masks, token_of_job, slot_of_job)
            up = self._grouped_site(n("experts_up"), xs, layout, weights, masks, token_of_job, slot_of_job)
            h = self._swiglu(gate, up)
            return layout.gather_rows(self._grouped_site(n("experts_down"), h, layout, weights, masks, token_of_job,
                                                         slot_of_job))
        args = (expert_of_job, order, bounds, weights, masks, token_of_job, slot_of_job)
        gate = self._expert_site(n("experts_gate"), x_jobs, *args)
        up = self._expert_site(n("experts_up"), x_jobs, *args)
        return self._expert_site(n("experts_down"), self._swiglu(gate, up), *args)

    def _run(self, batch: tf.LMBatch, weights, masks, capture: tuple[str, ...], want_taps: bool,
             aux: dict | None = None):
        from param_decomp_b200.core.model import ForwardResult

        a = self.arch
        aux = {} if aux is None else aux
        want = set(capture)
        tokens = batch.tokens
        B, T = tokens.shape
        resid = F.embedding(tokens.long(), self.w["embed.weight"])
        pos = batch.positions if batch.positions is not None else torch.arange(T, device=tokens.device)[None]
        cos, sin = ports.rope_cos_sin(pos, self.rotary_dim, a.rope_theta)
        taps: dict[str, Tensor] | None = {} if want_taps else None
        captures: dict[str, Tensor] = {}
        for i in range(a.n_layer):
            if taps is not None:
                taps[f"resid.{i}"] = resid
            if f"resid.{i}" in want:
                captures[f"resid.{i}"] = resid
            resid = self._block(i, resid, cos, sin, batch, weights, masks, taps, captures, want, aux)
        if taps is not None:
            taps[f"resid.{a.n_layer}"] = resid
        if f"resid.{a.n_layer}" in want:  # the boundary that leaves the last block, as the dense transformer captures it
            captures[f"resid.{a.n_layer}"] = resid
        final = self._norm(resid, self.w["final_norm.weight"])
        return ForwardResult(output=final, taps=taps or {}, captures=captures, aux=aux)


def build_qwen35_model(arch: TransformerArchConfig, weights: dict[str, Tensor], sites_cfg: Any, target_cfg: Any,
                       backend: str, ep: Any = None) -> Qwen35DecomposedModel:
    """Tile the per-kind component counts over the selected layers that carry each kind."""
    from param_decomp_b200.config.experiments import select_layers

    layers = set(select_layers(sites_cfg.layers, arch.n_layer))

    def local_c(kind: str) -> int:
        C = sites_cfg.cs[kind]
        if ep is None or kind not in EXPERT_KINDS:
            return C
        return C // arch.n_experts * ep.e_loc

    site_cs = {site_name(i, k): local_c(k) for k in KIND_ORDER if k in sites_cfg.cs
               for i in layers_of_kind(arch, k) if i in layers}
    if ep is not None:
        from param_decomp_b200.parallel.ep import shard_expert_weights

        weights = shard_expert_weights({k.replace("mlp.experts.", "mlp.experts_"): v for k, v in weights.items()},
                                       arch.n_experts, ep.rank, ep.world)
        weights = {k.replace("mlp.experts_", "mlp.experts."): v for k, v in weights.items()}
    model = Qwen35DecomposedModel(arch, weights, site_cs, backend=backend,
                                 attention=target_cfg.attention_implementation, ep=ep)
    edge = getattr(target_cfg, "output_edge", None)
    model.n_vocab_chunks = getattr(edge, "n_vocab_chunks", None)  # streamed output edge: chunks of positions
    return model
