"""Analytical useful-FLOP accounting for a decomposition step (for MFU).

Counts matmul FLOPs only (2 per multiply-add), forward + backward, for: the clean target forward,
every masked forward/backward (component path `2 C (d_in + d_out)` plus the frozen product
`2 d_in d_out` per position per site, attention `4 T d` per position per layer, the vocabulary head),
the CI function, and the faithfulness product `2 d_in d_out C` per site.

Parity: param_decomp/core/flops/*.py, experiments/lm/model_flops.py, core/hardware_utilization.py.
"""

from __future__ import annotations

from typing import Any

from param_decomp_b200.core.objective import build_objective


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
    attn_core = 4.0 * seq_len * arch.n_head * hd / 2  # causal: half the square
    n_mlp = 2 if arch.family == "simple_mlp" else 3
    k = (arch.experts_per_token or 1) if arch.family == "moe" else 1
    mlp = 2.0 * arch.d_model * arch.d_ff * n_mlp * k
    head = 2.0 * arch.d_model * arch.vocab_size
    return arch.n_layer * (attn_proj + attn_core + mlp) + head


def decomposition_step_flops(model: Any, ci_fn: Any, pd: Any, seq_len: int | None) -> float:
    positions = pd.batch_size * (seq_len or 1)
    main, extra = masked_forward_count(pd)
    comp, dense = site_flops_per_position(model)
    target = target_flops_per_position(model, seq_len or 1)
    masked_fwd = target + comp  # dense product rides along for the delta path (already in `target`)
    ci = getattr(ci_fn, "useful_flops_per_position", lambda: 0)()
    per_position = target + 3.0 * (main + extra) * masked_fwd + 3.0 * ci
    faith = sum(3.0 * 2.0 * s.d_in * s.d_out * s.C / max(s.n_blocks, 1) for s in model.sites)
    return per_position * positions + faith
