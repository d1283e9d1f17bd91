"""One-shot migrations of stored run configs to the current schema.

  * `schedule_knots`: the old `{start_val, final_val_frac, warmup_pct, fn_type}` schedule spelling
    -> knot schedules;
  * `data_layout`: a bare dataset name with no `layout` -> `unsegmented_tokens` (token-only corpora);
  * `decomposition_apparatus`: top-level `C`/`ci_fn_type`/`ci_fn_hidden_dims` -> `decomposition: {sites, ci}`;
  * `optimizer_type`: optimizer blocks without `type` -> `adamw`.

Parity: param_decomp/migrations/ (schedule_knots, data_layout, decomposition_apparatus, ...).
"""

from __future__ import annotations

import copy
from typing import Any


def migrate_schedule(old: Any) -> Any:
    if not isinstance(old, dict) or "start_val" not in old:
        return old
    start = float(old["start_val"])
    final = float(old.get("final_val_frac", 1.0))
    warm = float(old.get("warmup_pct", 0.0))
    interp = {"linear": "linear", "cosine": "cosine", "constant": "linear"}[old.get("fn_type", "constant")]
    pts = []
    if warm > 0:
        pts += [{"at": 0.0, "frac": 0.0}, {"at": warm, "frac": 1.0}]
    else:
        pts += [{"at": 0.0, "frac": 1.0}]
    pts.append({"at": 1.0, "frac": final if old.get("fn_type", "constant") != "constant" else 1.0, "interp": interp})
    return {"max_val": start, "points": pts}


def _walk(node: Any) -> Any:
    if isinstance(node, dict):
        node = {k: _walk(v) for k, v in node.items()}
        return migrate_schedule(node)
    if isinstance(node, list):
        return [_walk(v) for v in node]
    return node


def migrate_raw(raw: dict[str, Any]) -> dict[str, Any]:
    out = _walk(copy.deepcopy(raw))
    data = out.get("data")
    if isinstance(data, dict) and "train" in data and "layout" not in data:
        data["layout"] = "unsegmented_tokens"
    if "C" in out and "decomposition" not in out:
        out["decomposition"] = {"sites": out.pop("sites", None) or {"kind": "explicit", "sites": []},
                                "ci": {"type": out.pop("ci_fn_type", "layerwise_mlp"),
                                       "hidden_dims": out.pop("ci_fn_hidden_dims", [16])}}
        out.pop("C")
    return out
