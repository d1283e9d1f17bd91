"""Migrations of stored run configs and checkpoints to the current schema.

Config migrations are pure `dict -> dict` transforms applied at the stored-config boundary (`load_run_config`
and the experiment configs' `from_file`): a pinned `launch_config.yaml` written by an older schema still loads,
resumes and serves as a fine-tune parent; newly written configs are already current, for them every step is
the identity.

  * `schedule_knots`           `{start_val, final_val_frac, warmup_pct, fn_type}` -> knot schedules
  * `decomposition_apparatus`  `pd.ci_config` + `pd.decomposition_targets: [{module_pattern, C}]` (and the still
                               older top-level `C` / `ci_fn_type` / `ci_fn_hidden_dims`) -> `decomposition: {sites, ci}`
  * `data_layout`              LM `data` without `layout` / `seq_len` -> the layout its site family read
                               (`documents` for GLU transformers, `unsegmented_tokens` otherwise) and the width
                               recorded in the training dataset's meta file
  * `metric_schema`            `wandb.metric_schema: v2` -> `grouped`

Checkpoint migration (`migrate_ci_attention_keys`, CLI below): CI-transformer blocks once kept their attention
projections next to the feed-forward weights (`blocks.N.wq ...`, QK-norm gains as `qk_norm_scales.{0,1}`); they
now live in the block's attention module (`blocks.N.attn.wq ...`, `attn.q_gain` / `attn.k_gain`). The same
renaming applies to the optimizer moments. Values, shapes and dtypes are untouched.

    python -m param_decomp_b200.infra.migrations ci_attention <ckpt step dir> <new step dir>
    python -m param_decomp_b200.infra.migrations config <old.yaml> <new.yaml>

Parity: param_decomp/migrations/{schedule_knots,decomposition_apparatus,data_layout,ci_attention}.py.
"""

from __future__ import annotations

import copy
import re
from pathlib import Path
from typing import Any

_GLU = re.compile(r"^(?:model\.)?layers\.(\d+|\*)\.(?:self_attn\.(q|k|v|o)|mlp\.(gate|up|down))_proj$")
_SMLP = re.compile(r"^h\.(\d+|\*)\.(?:attn\.(q_proj|k_proj|v_proj|o_proj)|mlp\.(c_fc|down_proj))$")
_LAYOUT_BY_SITES = {"simple_mlp": "unsegmented_tokens", "qwen36_moe": "unsegmented_tokens", "moe": "unsegmented_tokens",
                    "glu_transformer": "documents"}


# ---- schedules / optimizers -------------------------------------------------------------------------

def migrate_schedule(old: Any) -> Any:
    if not isinstance(old, dict) or "start_val" not in old:
        return old
    start = float(old["start_val"])
    kind = old.get("fn_type", "constant")
    final = float(old.get("final_val_frac", 1.0))
    warm = float(old.get("warmup_pct", 0.0))
    interp = {"linear": "linear", "cosine": "cosine", "constant": "linear"}[kind]
    pts = [{"at": 0.0, "frac": 0.0}, {"at": warm, "frac": 1.0}] if warm > 0 else [{"at": 0.0, "frac": 1.0}]
    pts.append({"at": 1.0, "frac": final if kind != "constant" else 1.0, "interp": interp})
    return {"max_val": start, "points": pts}


def _walk_schedules(node: Any) -> Any:
    if isinstance(node, dict):
        return migrate_schedule({k: _walk_schedules(v) for k, v in node.items()})
    if isinstance(node, list):
        return [_walk_schedules(v) for v in node]
    return node


# ---- decomposition apparatus ------------------------------------------------------------------------

def _sites_from_targets(targets: list[dict[str, Any]]) -> dict[str, Any]:
    """`[{module_pattern, C}]` -> a `glu_transformer` / `simple_mlp` C-spec, or an explicit site list for names
    of neither LM grammar (toys)."""
    family, per_layer = None, {}
    for t in targets:
        pat, c = t["module_pattern"], int(t["C"])
        m = _GLU.match(pat)
        fam = "glu_transformer" if m else None
        if m is None:
            m = _SMLP.match(pat)
            fam = "simple_mlp" if m else None
        if m is None:
            return {"kind": "explicit", "sites": [{"name": t["module_pattern"], "C": int(t["C"])} for t in targets]}
        assert family in (None, fam), f"decomposition targets mix site grammars: {pat!r}"
        family = fam
        per_layer.setdefault(m.group(1), {})[m.group(2) or m.group(3)] = c
    cs_sets = {tuple(sorted(v.items())) for v in per_layer.values()}
    assert len(cs_sets) == 1, "per-layer component counts differ: the C-spec holds one count per matrix kind"
    cs = dict(next(iter(cs_sets)))
    layers = {"kind": "all"} if "*" in per_layer else {"kind": "list", "indices": sorted(int(k) for k in per_layer)}
    return {"kind": family, "layers": layers, "cs": cs}


def _decomposition_apparatus(out: dict[str, Any]) -> None:
    pd = out.get("pd") if isinstance(out.get("pd"), dict) else None
    if "decomposition" in out:
        return
    if pd is not None and ("decomposition_targets" in pd or "ci_config" in pd):
        out["decomposition"] = {"sites": _sites_from_targets(pd.pop("decomposition_targets", [])),
                                "ci": pd.pop("ci_config", {"type": "layerwise_mlp", "hidden_dims": [16]})}
    elif "C" in out:  # the oldest toy spelling: one C for every site
        c = int(out.pop("C"))
        names = out.pop("site_names", None) or []
        out["decomposition"] = {"sites": {"kind": "explicit", "sites": [{"name": n, "C": c} for n in names]},
                                "ci": {"type": out.pop("ci_fn_type", "layerwise_mlp"),
                                       "hidden_dims": out.pop("ci_fn_hidden_dims", [16])}}


# ---- data layout ---------------------------------------------------------------------------------------

def _data_layout(out: dict[str, Any], data_root: Path | None) -> None:
    data = out.get("data")
    if not isinstance(data, dict) or "train" not in data or "layout" in data:
        return
    kind = ((out.get("decomposition") or {}).get("sites") or {}).get("kind", "simple_mlp")
    data["layout"] = _LAYOUT_BY_SITES.get(kind, "unsegmented_tokens")
    if "seq_len" not in data and data_root is not None and isinstance(data["train"], dict) and "name" in data["train"]:
        from param_decomp_b200.formats.dataset_store import read_dataset_meta

        try:
            data["seq_len"] = read_dataset_meta(Path(data_root) / "datasets" / data["train"]["name"]).seq_len
        except (OSError, AttributeError, KeyError):
            pass  # the width stays for validation to ask for


def migrate_raw(raw: dict[str, Any], data_root: Path | None = None) -> dict[str, Any]:
    """Every config migration, in order; the identity on a current config."""
    out = _walk_schedules(copy.deepcopy(raw))
    _decomposition_apparatus(out)
    _data_layout(out, data_root)
    if isinstance(out.get("wandb"), dict) and out["wandb"].get("metric_schema") == "v2":
        out["wandb"]["metric_schema"] = "grouped"
    return out


# ---- checkpoints: CI attention ---------------------------------------------------------------------------

_OLD_ATTN = re.compile(r"^(?P<pre>.*blocks\.\d+\.)(?P<leaf>w[qkvo]\.(?:weight|bias)|qk_norm_scales\.[01])(?P<post>(?:/(?:mu|nu|mom))?)$")


def migrate_ci_attention_keys(tensors: dict[str, Any]) -> dict[str, Any]:
    """Rename the legacy attention leaves of CI-transformer blocks (and their optimizer moments); every other key,
    and every value, passes through. A checkpoint that already has `blocks.N.attn.*` keys is returned as is; one
    that mixes both spellings is refused."""
    has_new = any(re.search(r"blocks\.\d+\.attn\.", k) for k in tensors)
    has_old = any(_OLD_ATTN.match(k) for k in tensors)
    assert not (has_new and has_old), "checkpoint mixes old and new attention key paths"
    out = {}
    for k, v in tensors.items():
        m = _OLD_ATTN.match(k)
        if m is None:
            out[k] = v
            continue
        leaf = m["leaf"]
        leaf = {"qk_norm_scales.0": "q_gain", "qk_norm_scales.1": "k_gain"}.get(leaf, leaf)
        out[f"{m['pre']}attn.{leaf}{m['post']}"] = v
    return out


def migrate_checkpoint_step(src: Path, dst: Path) -> None:
    """Copy one `ckpts/<step>` directory with the attention keys migrated; the source stays intact."""
    from safetensors import safe_open
    from safetensors.torch import save_file

    src, dst = Path(src), Path(dst)
    assert src.resolve() != dst.resolve() and not dst.exists(), "the destination must be a new directory"
    dst.mkdir(parents=True)
    for f in sorted(src.glob("*.safetensors")):
        with safe_open(str(f), framework="pt") as h:
            meta = h.metadata() or {}
            tensors = {k: h.get_tensor(k) for k in h.keys()}
        save_file(migrate_ci_attention_keys(tensors), str(dst / f.name), metadata=meta)


def main() -> None:
    import argparse

    import yaml

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["config", "ci_attention"])
    ap.add_argument("source", type=Path)
    ap.add_argument("destination", type=Path)
    ap.add_argument("--data-root", type=Path, default=None)
    a = ap.parse_args()
    if a.what == "config":
        a.destination.write_text(yaml.dump(migrate_raw(yaml.safe_load(a.source.read_text()), a.data_root), sort_keys=False))
    else:
        migrate_checkpoint_step(a.source, a.destination)


if __name__ == "__main__":
    main()
