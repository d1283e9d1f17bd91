"""Permutation metrics: how close a matrix of causal importances (rows = probes or features, columns =
components) is to an identity or to a dense pattern, after the best reordering of its columns; and the
figures that show CI, `V` and `U` in that order.

Parity: param_decomp/core/slow_eval.py:494-551 (`permute_to_identity` by Hungarian assignment on `-ci` over the
`min(shape)` square block with the unassigned columns appended in order; `permute_to_dense` by total mass;
the discrete `identity_ci_error` and `dense_ci_error` distances), :553-632 (metric specs resolved against the
run's sites by fnmatch patterns), :801-911 (permuted CI heat maps, `V` / `U` matrices in the CI order).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from fnmatch import fnmatch

import numpy as np

from param_decomp_b200.utils import figures


def permute_to_identity(ci: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """`(permuted [rows, C], perm [C])`: columns assigned to rows by maximum total CI, the rest in order."""
    from scipy.optimize import linear_sum_assignment

    assert ci.ndim == 2, ci.shape
    rows, C = ci.shape
    size = min(rows, C)
    _, cols = linear_sum_assignment(-ci[:size])
    taken = set(cols.tolist())
    perm = np.array(list(cols) + [c for c in range(C) if c not in taken], dtype=np.int64)
    return ci[:, perm], perm


def permute_to_dense(ci: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    perm = np.argsort(-ci.sum(axis=0), kind="stable")
    return ci[:, perm], perm


def identity_ci_error(ci: np.ndarray, tolerance: float = 0.1) -> int:
    """Entries off the identity pattern after the best column assignment: off-diagonal entries above
    `tolerance` (trailing rows / columns of an overcomplete matrix count as off-diagonal) plus diagonal entries
    below `1 - tolerance`."""
    permuted, _ = permute_to_identity(ci.astype(np.float64))
    size = min(permuted.shape)
    off = np.ones(permuted.shape, dtype=bool)
    off[:size, :size] &= ~np.eye(size, dtype=bool)
    return int((permuted[off] > tolerance).sum()) + int((np.diagonal(permuted[:size, :size]) < 1 - tolerance).sum())


def dense_ci_error(ci: np.ndarray, k: int, tolerance: float = 0.1, min_entries: int = 1) -> int:
    """Columns sorted by mass: each of the first `k` must hold at least `min_entries` strong activations
    (`>= 1 - tolerance`), every later column counts one error per weak activation (`> tolerance`)."""
    assert k <= ci.shape[1], f"expected at least {k} columns, got {ci.shape[1]}"
    srt, _ = permute_to_dense(ci.astype(np.float64))
    strong = (srt >= 1 - tolerance).sum(axis=0)
    return int(np.clip(min_entries - strong, 0, None)[:k].sum()) + int((srt > tolerance).sum(axis=0)[k:].sum())


@dataclass
class PermutationSpec:
    """Which sites the permutation metrics cover and which pattern governs each one's column order."""

    order: dict[str, str] = field(default_factory=dict)  # site -> "identity" | "dense" (plots)
    identity_targets: dict[str, int] = field(default_factory=dict)  # site -> n_features
    dense_targets: dict[str, int] = field(default_factory=dict)  # site -> k

    @property
    def any_plots(self) -> bool:
        return bool(self.order)


def resolve_spec(site_names: list[str], plots_cfg=None, error_cfg=None) -> PermutationSpec:
    """`plots_cfg`: a `PermutedCIPlots` / `UVPlots` config (`identity_patterns`, `dense_patterns`); `error_cfg`: an
    `IdentityCIError` config (`identity_ci`, `dense_ci` lists of `{layer_pattern, n_features | k}`). A site matched
    by both kinds of pattern follows the identity rule."""
    spec = PermutationSpec()
    if plots_cfg is not None:
        for s in site_names:
            if any(fnmatch(s, p) for p in (plots_cfg.dense_patterns or [])):
                spec.order[s] = "dense"
            if any(fnmatch(s, p) for p in (plots_cfg.identity_patterns or [])):
                spec.order[s] = "identity"
    if error_cfg is not None:
        for t in (error_cfg.identity_ci or []):
            for s in site_names:
                if fnmatch(s, t.layer_pattern):
                    spec.identity_targets[s] = t.n_features
        for t in (error_cfg.dense_ci or []):
            for s in site_names:
                if fnmatch(s, t.layer_pattern):
                    spec.dense_targets[s] = t.k
    return spec


def errors(spec: PermutationSpec, probe_ci: dict[str, np.ndarray], tolerance: float = 0.1) -> dict[str, float]:
    out: dict[str, float] = {}
    for s, n in spec.identity_targets.items():
        if s in probe_ci:
            out[f"identity_ci_error/{s}"] = float(identity_ci_error(probe_ci[s][:n], tolerance))
    for s, k in spec.dense_targets.items():
        if s in probe_ci:
            out[f"dense_ci_error/{s}"] = float(dense_ci_error(probe_ci[s], k, tolerance))
    return out


def column_orders(spec: PermutationSpec, probe_ci: dict[str, np.ndarray]) -> dict[str, np.ndarray]:
    return {s: (permute_to_identity if kind == "identity" else permute_to_dense)(probe_ci[s])[1]
            for s, kind in spec.order.items() if s in probe_ci}


def render_permuted_ci(spec: PermutationSpec, probe_ci: dict[str, np.ndarray], run_dir, step: int) -> str | None:
    orders = column_orders(spec, probe_ci)
    if run_dir is None or not orders:
        return None
    arrays = {s: probe_ci[s][:, o] for s, o in orders.items()}
    first = None
    for s, m in arrays.items():
        p = figures.save_figure(run_dir, f"permuted_ci_{s}_step{step}", figures.heatmap(m, cell=3, vmin=0.0, vmax=1.0),
                                {"ci": m, "perm": orders[s]})
        first = first or p
    return str(first)


def render_uv(spec: PermutationSpec, probe_ci: dict[str, np.ndarray], V: dict[str, np.ndarray],
              U: dict[str, np.ndarray], run_dir, step: int) -> str | None:
    """`V [d_in, C]` and `U [C, d_out]` of each covered site with components in the CI order."""
    orders = column_orders(spec, probe_ci)
    if run_dir is None or not orders:
        return None
    first = None
    for s, o in orders.items():
        if s not in V:
            continue
        v, u = V[s][:, o], U[s][o, :]
        p = figures.save_figure(run_dir, f"uv_{s}_V_step{step}", figures.heatmap(v, cell=3), {"V": v, "perm": o})
        figures.save_figure(run_dir, f"uv_{s}_U_step{step}", figures.heatmap(u, cell=3), {"U": u, "perm": o})
        first = first or p
    return str(first) if first else None
