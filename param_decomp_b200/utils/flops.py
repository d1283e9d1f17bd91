"""Analytical useful-FLOP accounting of a decomposition step, term by term (for MFU).

Model FLOPs count contractions only (2 per multiply-add): the clean target forward, the CI function (forward
and backward; its first layer reads frozen taps, so it has a weight gradient but no input gradient), every
masked forward / backward of every reconstruction term (component path `2 C (d_in + d_out)` plus the frozen
product `2 d_in d_out` per position per site, causal attention `2 T d` per position per layer, the vocabulary
head), the extra forward / backward-to-sources passes of adversary ascents, and the faithfulness product and
its two gradients. Optimizer FLOPs are listed separately: elementwise update arithmetic (AdamW 12 per parameter,
+1 with weight decay; Muon 8 per matrix entry, 15 per vector entry), global-norm clipping (3 per parameter), and
the Newton-Schulz contractions of Muon (`X' = (aI + bA + cA^2) X` with the smaller Gram matrix `A = X X^T`,
symmetric products counted by their triangle).

`step_flops(...)` returns the breakdown; `decomposition_step_flops(...)` its model total (what `train/perf/mfu`
uses); `train/perf/mfu_with_optimizer` adds the optimizer's contractions.

Parity: param_decomp/core/flops/{types,target,ci,model,optimizer}.py, experiments/lm/model_flops.py,
core/hardware_utilization.py:19-84, core/training_performance.py:16-162.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from param_decomp_b200.config.run import AdamWOptimizerConfig, MuonOptimizerConfig
from param_decomp_b200.core.objective import build_objective


@dataclass(frozen=True)
class ForwardBackward:
    forward: float = 0.0
    backward: float = 0.0

    @property
    def total(self) -> float:
        return self.forward + self.backward

    def __add__(self, o: "ForwardBackward") -> "ForwardBackward":
        return ForwardBackward(self.forward + o.forward, self.backward + o.backward)

    def scaled(self, k: float) -> "ForwardBackward":
        return ForwardBackward(self.forward * k, self.backward * k)


@dataclass
class StepFlops:
    """`model[name]` contraction FLOPs per step of each term; `optimizer_contractions` (Newton-Schulz) and
    `optimizer_arithmetic` (elementwise updates, clipping) per optimizer group."""

    model: dict[str, ForwardBackward] = field(default_factory=dict)
    optimizer_contractions: dict[str, float] = field(default_factory=dict)
    optimizer_arithmetic: dict[str, float] = field(default_factory=dict)

    @property
    def model_total(self) -> float:
        return sum(t.total for t in self.model.values())

    @property
    def optimizer_total(self) -> float:
        return sum(self.optimizer_contractions.values())

    def scalars(self) -> dict[str, float]:
        return {"perf/useful_model_flops": self.model_total, "perf/useful_optimizer_flops": self.optimizer_total,
                "perf/useful_flops": self.model_total + self.optimizer_total}


# ---- target ----------------------------------------------------------------------------------------------

def masked_forward_count(pd: Any) -> tuple[int, int]:
    """(forward+backward passes with parameter grads, extra forward+backward passes for ascents)."""
    obj = build_objective(pd)
    main = sum(t.n_samples for t in obj.recon)
    extra = 0
    for t in obj.recon:
        if t.is_persistent:
            extra += t.cfg.n_warmup_steps  # type: ignore[attr-defined]
        if t.strategy == "fresh_pgd":
            extra += t.cfg.n_steps  # type: ignore[attr-defined]
    return main, extra


def site_flops_per_position(model: Any) -> tuple[float, float]:
    comp = sum(2.0 * s.C * (s.d_in + s.d_out) / max(s.n_blocks, 1) for s in model.sites)
    dense = sum(2.0 * s.d_in * s.d_out for s in model.sites)
    return comp, dense


def target_flops_per_position(model: Any, seq_len: int) -> float:
    arch = getattr(model, "arch", None)
    if arch is None:
        return sum(2.0 * s.d_in * s.d_out for s in model.sites)
    hd = arch.head_dim or arch.d_model // arch.n_head
    kv = arch.n_kv_head or arch.n_head
    attn_proj = 2.0 * arch.d_model * hd * (2 * arch.n_head + 2 * kv)
    attn_core = 4.0 * seq_len * arch.n_head * hd / 2  # causal: half the square, QK^T and PV
    n_mlp = 2 if arch.family == "simple_mlp" else 3
    k = (arch.experts_per_token or 1) if arch.family in ("moe", "qwen35_moe") else 1
    mlp = 2.0 * arch.d_model * arch.d_ff * n_mlp * k
    head = 2.0 * arch.d_model * arch.vocab_size
    return arch.n_layer * (attn_proj + attn_core + mlp) + head


# ---- CI function -----------------------------------------------------------------------------------------

def ci_fn_flops_per_position(ci_fn: Any, seq_len: int) -> ForwardBackward:
    """Matrix products of the CI function (2 per parameter of every matrix) plus, for transformer CI functions,
    the attention core of each block; the backward costs twice the forward except for the first projection,
    whose input (frozen taps) needs no gradient."""
    if ci_fn is None:
        return ForwardBackward()
    mat = float(getattr(ci_fn, "useful_flops_per_position", lambda: 0)())
    attn = 0.0
    first = 0.0
    for m in getattr(ci_fn, "modules", lambda: [])():
        cls = type(m).__name__
        if cls == "CIAttention":
            causal = 0.5 if getattr(m, "causal", False) else 1.0
            attn += 4.0 * seq_len * m.n_heads * m.hd * causal
        elif cls == "TransformerBackbone":
            first += 2.0 * m.w_in.weight.numel()
    fwd = mat + attn
    return ForwardBackward(fwd, 2.0 * fwd - first)


# ---- optimizer -------------------------------------------------------------------------------------------

def newton_schulz_flops(n_rows: int, n_cols: int, n_matrices: int, n_steps: int) -> float:
    r, c = sorted((n_rows, n_cols))
    tri = r * (r + 1) // 2
    per_step = 2.0 * tri * c + 2.0 * tri * r + 2.0 * r * r * c
    return n_matrices * n_steps * per_step


def optimizer_flops(name: str, cfg: Any, params: list[Any]) -> tuple[float, float]:
    """`(contraction FLOPs, elementwise arithmetic)` of one optimizer group per step."""
    n = sum(p.numel() for p in params)
    decay = int(getattr(cfg, "weight_decay", 0.0) != 0)
    contractions = 0.0
    if isinstance(cfg, MuonOptimizerConfig):
        mats = [p for p in params if p.dim() >= 2 and min(p.shape[-2:]) > 1]
        n_mat = sum(p.numel() for p in mats)
        arithmetic = n_mat * (8 + decay) + 15.0 * (n - n_mat)
        for p in mats:
            stack = p.numel() // (p.shape[-1] * p.shape[-2])
            contractions += newton_schulz_flops(p.shape[-2], p.shape[-1], stack, cfg.ns_steps)
            arithmetic += stack * (3.0 * p.shape[-1] * p.shape[-2] + 1)  # Frobenius normalisation
    else:
        assert isinstance(cfg, AdamWOptimizerConfig), type(cfg)
        arithmetic = n * (12.0 + decay)
    if getattr(cfg, "grad_clip_norm", None) is not None and n:
        arithmetic += 3.0 * n + 2
    return contractions, arithmetic


# ---- the step --------------------------------------------------------------------------------------------

def step_flops(model: Any, ci_fn: Any, pd: Any, seq_len: int | None, components: Any = None) -> StepFlops:
    T = seq_len or 1
    positions = float(pd.batch_size * T)
    obj = build_objective(pd)
    comp, _dense = site_flops_per_position(model)
    target = target_flops_per_position(model, T)
    masked = target + comp  # the frozen product rides along for the delta path (already in `target`)
    out = StepFlops()
    out.model["clean_forward"] = ForwardBackward(target * positions, 0.0)
    out.model["ci_fn"] = ci_fn_flops_per_position(ci_fn, T).scaled(positions)
    for t in obj.recon:
        out.model[f"recon/{t.name}"] = ForwardBackward(masked, 2.0 * masked).scaled(positions * t.n_samples)
        ascents = (t.cfg.n_warmup_steps if t.is_persistent else 0) + (t.cfg.n_steps if t.strategy == "fresh_pgd" else 0)  # type: ignore[attr-defined]
        if ascents:  # forward + backward to the sources (no weight gradients: one backward product per forward one)
            out.model[f"ascent/{t.name}"] = ForwardBackward(masked, masked).scaled(positions * ascents)
    if obj.faith is not None:
        f = sum(2.0 * s.d_in * s.d_out * s.C / max(s.n_blocks, 1) for s in model.sites)
        out.model["faithfulness"] = ForwardBackward(f, 2.0 * f)
    comp_params = list(components.parameters()) if components is not None else []
    ci_params = list(ci_fn.parameters()) if ci_fn is not None and hasattr(ci_fn, "parameters") else []
    for name, cfg, params in (("components", pd.components_optimizer, comp_params), ("ci_fn", pd.ci_fn_optimizer, ci_params)):
        if params:
            out.optimizer_contractions[name], out.optimizer_arithmetic[name] = optimizer_flops(name, cfg, params)
    return out


def decomposition_step_flops(model: Any, ci_fn: Any, pd: Any, seq_len: int | None) -> float:
    return step_flops(model, ci_fn, pd, seq_len).model_total
