"""Top-k routed mixture-of-experts LM target (Qwen-MoE style) and its expert-parallel execution.

Block = the dense transformer's attention half, then per token: router logits `x W_r^T` ->
softmax -> top-k -> (optionally renormalised) weights; each selected expert is a SwiGLU MLP
`down_e(silu(gate_e x) * up_e x)`; the block output is the weighted sum.

Decomposition: attention `q,k,v,o` as dense sites; the expert banks as BLOCKED sites
`layers.{i}.mlp.experts_{gate,up,down}` with `n_blocks = n_experts`: expert `e` owns the component
block `V_e [d_in, c]`, `U_e [c, d_out]`, the site's flat component axis is block-major `C = E c`.
A (token, slot) pair routed to expert `e` is a *job*; a blocked site evaluates
`((x_j V_e) * (m_j - d)) U_e + d (x_j W_e^T)` per job, where `m_j [c]` is the job's slice of the
site mask. CI and masks of blocked sites are NARROW: `[tokens, k * c]`, slot-major in the order of the
token's selected experts (`SelectedCI`), never the `E c`-wide dense form. Masked forwards reuse the
clean forward's routing (pinned), so CI slots and jobs line up.

Expert parallelism (`ep_world > 1`): experts (their frozen weights and their component blocks) are
dealt in contiguous ranges to the ranks of the expert group, padded with never-routed experts so the
count tiles the group; tokens are data-parallel. Dispatch sends each job's activation row to the
expert's owner, combine returns the output row: an all-to-all each way (`parallel/ep.py`).

Parity: param_decomp/targets/qwen36_moe.py:473-515 (router verbs), :1562-1875 (expert paths),
:2596-2750 (dense / routed / placed), routed/experts.py:28-40,375-420,864-885 (jobs, EP by
activation slicing + all-reduce: kept as `ep_mode="allreduce"`), routed/dense.py (dense oracle).
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.nn.functional as F
from torch import Tensor

from param_decomp_b200.config.experiments import TransformerArchConfig
from param_decomp_b200.core.components import BlockSelection, ComputeWeights, SiteSpec
from param_decomp_b200.core.decomposed_linear import site_forward
from param_decomp_b200.core.masking import Masks, SiteMask
from param_decomp_b200.core.model import ForwardResult
from param_decomp_b200.models import transformer as tf
from param_decomp_b200.ops.grouped import repeat_rows

EXPERT_KINDS = ("experts_gate", "experts_up", "experts_down")


def route_topk(logits: Tensor, k: int, renormalise: bool) -> BlockSelection:
    """softmax over experts (fp32) -> top-k -> optional renormalisation of the kept weights."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = probs.topk(k, dim=-1)
    if renormalise:
        w = w / w.sum(-1, keepdim=True)
    return BlockSelection(indices=idx, weights=w)


def random_init_moe_weights(arch: TransformerArchConfig, seed: int, dtype=torch.bfloat16, device="cpu") -> dict[str, Tensor]:
    base = TransformerArchConfig.model_validate({**arch.model_dump(), "family": "glu_transformer"})
    w = tf.random_init_weights(base, seed, dtype, device)
    g = torch.Generator().manual_seed(seed + 7)
    E, d, ff = arch.n_experts, arch.d_model, arch.d_ff
    for i in range(arch.n_layer):
        for kind in ("gate", "up", "down"):
            w.pop(tf.weight_key("glu_transformer", i, kind))
        w[f"layers.{i}.mlp.router.weight"] = (torch.randn(E, d, generator=g) * 0.02).to(dtype).to(device)
        w[f"layers.{i}.mlp.experts_gate.weight"] = (torch.randn(E, ff, d, generator=g) * 0.02).to(dtype).to(device)
        w[f"layers.{i}.mlp.experts_up.weight"] = (torch.randn(E, ff, d, generator=g) * 0.02).to(dtype).to(device)
        w[f"layers.{i}.mlp.experts_down.weight"] = (
            torch.randn(E, d, ff, generator=g) * 0.02 / math.sqrt(2 * arch.n_layer)).to(dtype).to(device)
    return w


def dense_moe_oracle(x: Tensor, sel: BlockSelection, Wg: Tensor, Wu: Tensor, Wd: Tensor) -> Tensor:
    """All-experts reference: every expert evaluated on every token, unselected ones weighted 0."""
    E = Wg.shape[0]
    dense_w = torch.zeros(*sel.indices.shape[:-1], E, device=x.device, dtype=torch.float32)
    dense_w.scatter_(-1, sel.indices, sel.weights.float())
    h = F.silu(torch.einsum("nd,efd->nef", x.float(), Wg.float())) * torch.einsum("nd,efd->nef", x.float(), Wu.float())
    y = torch.einsum("nef,edf->ned", h, Wd.float())
    return (y * dense_w.unsqueeze(-1)).sum(1).to(x.dtype)


class MoEDecomposedModel(tf.TransformerDecomposedModel):
    use_row_map = True  # fused backend: mask inputs stay in token order (False = materialise per-job rows)

    def __init__(self, arch: TransformerArchConfig, weights: dict[str, Tensor], site_cs: dict[str, int],
                 backend: str = "eager_torch", attention: str = "flash", ep: Any = None, **kw: Any) -> None:
        assert arch.family == "moe"
        self.ep = ep  # parallel.ep.ExpertParallel or None
        super().__init__(arch, weights, site_cs, backend=backend, attention=attention, **kw)

    def _family_kinds(self) -> tuple[str, ...]:
        return ("q", "k", "v", "o", *EXPERT_KINDS)

    def _site_spec(self, name: str, kind: str, C: int) -> SiteSpec:
        if kind not in EXPERT_KINDS:
            return super()._site_spec(name, kind, C)
        W = self.w[name + ".weight"]  # [E, d_out, d_in]
        E = W.shape[0]
        assert C % E == 0, f"{name}: C={C} must be a multiple of n_experts={E} (components are expert-local)"
        return SiteSpec(name, W.shape[2], W.shape[1], C, group=kind, n_blocks=E, routed=True)

    def tap_for_site(self, site: str) -> str:
        layer, kind = self._site_layer_kind[site]
        if kind in EXPERT_KINDS:
            return f"mlp_in.{layer}"
        return super().tap_for_site(site)

    def block_tap_widths(self, layer: int) -> dict[str, int]:
        a = self.arch
        return {f"attn_in.{layer}": a.d_model, f"attn_out.{layer}": a.n_head * self.head_dim, f"mlp_in.{layer}": a.d_model}

    def expert_site_names(self, layer: int) -> list[str]:
        return [tf.site_name("moe", layer, k) for k in EXPERT_KINDS]

    @property
    def global_sites(self) -> tuple[SiteSpec, ...]:
        """The sites as the CI function, masks and adversaries see them. Under expert parallelism
        `sites` describes this rank's component blocks (its own experts, dummies included) while the
        importances of a token cover whichever of ALL experts it selected."""
        if self.ep is None:
            return self.sites
        E = self.ep.n_experts
        return tuple(s if not s.blocked else SiteSpec(s.name, s.d_in, s.d_out, s.C_block * E, group=s.group, n_blocks=E,
                                                      alignment=s.alignment, routed=s.routed) for s in self.sites)

    # -- expert bank --------------------------------------------------------------------------------
    def _expert_site(self, name: str, x_jobs: Tensor, expert_of_job: Tensor, order: Tensor, bounds: list[int],
                     weights: ComputeWeights | None, masks: Masks | None, token_of_job: Tensor,
                     slot_of_job: Tensor) -> Tensor:
        """One blocked site on jobs sorted by expert (`order`); `bounds[e]:bounds[e+1]` = expert e's jobs."""
        W = self.w[name + ".weight"]
        spec = next(s for s in self.sites if s.name == name) if (masks is not None and name in (masks or {})) else None
        out = x_jobs.new_empty(x_jobs.shape[0], W.shape[1])
        sm = masks[name] if spec is not None else None
        if sm is not None:
            sm = sm.materialize()
        c = spec.C_block if spec is not None else 0
        for e in range(W.shape[0]):
            lo, hi = bounds[e], bounds[e + 1]
            if lo == hi:
                continue
            rows = order[lo:hi]
            xe = x_jobs[rows]
            if spec is None or weights is None:
                out[rows] = F.linear(xe, W[e])
                continue
            V, U = weights.site(name)
            tok, slot = token_of_job[rows], slot_of_job[rows]
            m = None
            if sm.mask is not None:
                flat = sm.mask.reshape(-1, sm.mask.shape[-1])  # [tokens, k*c]
                m = flat.reshape(flat.shape[0], flat.shape[1] // c, c)[tok, slot]
            d = None if sm.delta is None else sm.delta.reshape(-1, 1)[tok]
            r = None if sm.route is None else sm.route.reshape(-1)[tok]
            out[rows] = site_forward(xe, V[e], U[e], W[e], SiteMask(mask=m, delta=d, route=r))
        return out

    def _mlp(self, i: int, x: Tensor, lin, taps, weights, masks, aux: dict) -> Tensor:
        a = self.arch
        B, T, d = x.shape
        xt = x.reshape(B * T, d)
        pinned = aux.get("pinned_routing")
        captures, want = aux.get("capture_sink", ({}, ()))
        logits = None
        if pinned is None or f"router_logits.{i}" in want:
            logits = F.linear(xt, self.w[f"layers.{i}.mlp.router.weight"])
        if f"router_logits.{i}" in want:
            # what the router WOULD decide on this pass's residual stream (the masked passes keep the clean pass's
            # choice): the quantity a router-KL auxiliary compares (param_decomp/targets/qwen36_moe.py:473-515)
            captures[f"router_logits.{i}"] = logits.float().view(B, T, -1)
        if pinned is not None:
            sel = pinned[i]
        else:
            sel = route_topk(logits, a.experts_per_token, a.norm_topk_prob)
            sel = BlockSelection(sel.indices.reshape(B, T, -1), sel.weights.reshape(B, T, -1))
            aux.setdefault("routing", {})[i] = sel
        k = sel.indices.shape[-1]
        idx = sel.indices.reshape(B * T, k)
        token_of_job = torch.arange(B * T, device=x.device).repeat_interleave(k)
        slot_of_job = torch.arange(k, device=x.device).repeat(B * T)
        expert_of_job = idx.reshape(-1)
        if self.ep is None and self._fused(xt):
            return self.expert_tokens(i, xt, sel.indices, sel.weights, weights, masks, token_of_job,
                                      slot_of_job).reshape(B, T, d)
        if self.ep is not None and self.ep.fast_allreduce(self, xt):
            return self.ep.run_tokens_allreduce(self, i, xt, sel.indices, sel.weights, weights, masks, token_of_job,
                                                slot_of_job).reshape(B, T, d)
        if self.ep is not None:
            y_jobs = self.ep.run_experts(self, i, xt, expert_of_job, token_of_job, slot_of_job, weights, masks)
        else:
            order, bounds = expert_of_job, [0]
            if not self._fused(xt):
                order = expert_of_job.argsort(stable=True)
                for n in torch.bincount(expert_of_job, minlength=a.n_experts).tolist():
                    bounds.append(bounds[-1] + n)
            y_jobs = self.expert_jobs(i, repeat_rows(xt, k), expert_of_job, order, bounds, weights, masks, token_of_job,
                                      slot_of_job, routing_indices=sel.indices)
        w = sel.weights.reshape(B * T, k, 1).to(y_jobs.dtype)
        return (y_jobs.reshape(B * T, k, d) * w).sum(1).reshape(B, T, d)

    def _grouped_site(self, name: str, xs: Tensor, layout, weights, masks, token_of_job: Tensor,
                      slot_of_job: Tensor) -> Tensor:
        """Fused path of one blocked site on padded sorted jobs (`ops/grouped.py`)."""
        from param_decomp_b200.ops import grouped

        W = self.w[name + ".weight"]
        if weights is None or masks is None or name not in masks or name not in weights.V:
            return grouped.grouped_linear(xs, W, layout)
        spec = next(s for s in self.sites if s.name == name)
        c = spec.C_block
        sm0 = masks[name]
        V, U = weights.site(name)
        J = token_of_job.numel()
        src = sm0.ci if sm0.stochastic is not None else sm0.mask
        local_ok = self.ep is None or getattr(layout, "foreign", False)
        if self.use_row_map and src is not None and local_ok and src.shape[-1] % c == 0 and c % 8 == 0:
            # mask inputs stay in token order; the kernels map job rows to them and draw the mask themselves
            from param_decomp_b200.ops import grouped as G

            kk = src.shape[-1] // c
            n_tok = src.numel() // src.shape[-1]
            if J == n_tok * kk:
                ci2 = src.reshape(n_tok, kk * c)
                ci2 = ci2 if ci2.dtype == torch.bfloat16 else ci2.to(torch.bfloat16)
                ci2 = ci2 if ci2.is_contiguous() else ci2.contiguous()
                st = sm0.stochastic
                mode, seed, stream, off = (0, st.seed64, st.stream, st.row_offset) if st is not None else (1, 0, 0, 0)
                d = None if sm0.delta is None else sm0.delta.reshape(n_tok).float().contiguous()
                r = None if sm0.route is None else sm0.route.reshape(n_tok)
                return G.grouped_site_mapped(xs, V, U, W, layout, ci2, mode, seed, stream, off, d, r, kk,
                                             weights.grad_V.get(name), weights.grad_U.get(name),
                                             need_wgrad=weights.direct_grads)
        sm = sm0.materialize()

        def per_job(t: Tensor | None, width: int) -> Tensor | None:
            if t is None:
                return None
            flat = t.reshape(-1, t.shape[-1]) if width else t.reshape(-1)
            # (explicit middle extent: a rank may receive no job at all, and -1 cannot be inferred from 0 elements)
            vals = flat.reshape(flat.shape[0], flat.shape[1] // c, c)[token_of_job, slot_of_job] if width else flat[token_of_job]
            out = vals.new_zeros(layout.n_rows, *vals.shape[1:])
            return out.index_copy(0, layout.pos, vals)

        m = per_job(sm.mask, c)
        d = per_job(None if sm.delta is None else sm.delta.reshape(-1).float(), 0)
        r = per_job(None if sm.route is None else sm.route.reshape(-1), 0)
        return grouped.grouped_site(xs, V, U, W, layout, m, d, r, weights.grad_V.get(name), weights.grad_U.get(name),
                                    need_wgrad=weights.direct_grads)

    def expert_tokens(self, i: int, xt: Tensor, indices: Tensor, route_w: Tensor, weights, masks,
                      token_of_job: Tensor, slot_of_job: Tensor, layout=None) -> Tensor:
        """Fused single-rank path: tokens `[N, d]` fan out to padded sorted job rows, run gate / up / down on
        the grouped kernels and come back as the routing-weighted sum per token."""
        from param_decomp_b200.ops.grouped import JobLayout

        n = lambda kind: tf.site_name("moe", i, kind)  # noqa: E731
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
        """gate/up/down of every job; `expert_of_job` indexes THIS rank's expert bank. `routing_indices`:
        the pinned `[.., k]` selection tensor the jobs were flattened from (keys the cached job layout)."""
        n = lambda kind: tf.site_name("moe", i, kind)  # noqa: E731
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
        h = self._swiglu(gate, up)
        return self._expert_site(n("experts_down"), h, *args)

    def masked_forward(self, weights: ComputeWeights, batch: tf.LMBatch, masks: Masks, capture: tuple[str, ...] = (),
                       clean: ForwardResult | None = None) -> ForwardResult:
        aux = {}
        if clean is not None and "routing" in clean.aux:
            aux["pinned_routing"] = clean.aux["routing"]
        return self._run(batch, weights, masks, capture, want_taps=False, aux=aux)


def build_moe_model(arch: TransformerArchConfig, weights: dict[str, Tensor], sites_cfg: Any, target_cfg: Any,
                    backend: str, rank: int = 0, world: int = 1, ep: Any = None) -> MoEDecomposedModel:
    from param_decomp_b200.config.experiments import select_layers

    layers = select_layers(sites_cfg.layers, arch.n_layer)
    kinds = [k for k in ("q", "k", "v", "o", *EXPERT_KINDS) if k in sites_cfg.cs]

    def local_c(kind: str) -> int:
        C = sites_cfg.cs[kind]
        if ep is None or kind not in EXPERT_KINDS:
            return C
        assert C % arch.n_experts == 0, f"{kind}: C={C} must be a multiple of n_experts={arch.n_experts}"
        return C // arch.n_experts * ep.e_loc  # this rank's expert blocks only

    site_cs = {tf.site_name("moe", i, k): local_c(k) for i in layers for k in kinds}
    if ep is not None:
        from param_decomp_b200.parallel.ep import shard_expert_weights

        weights = shard_expert_weights(weights, arch.n_experts, ep.rank, ep.world)
    model = MoEDecomposedModel(arch, weights, site_cs, backend=backend, attention=target_cfg.attention_implementation,
                              ep=ep)
    edge = getattr(target_cfg, "output_edge", None)
    model.n_vocab_chunks = getattr(edge, "n_vocab_chunks", None)  # streamed output edge: chunks of positions
    return model
