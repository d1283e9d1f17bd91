"""Metric key grammar shared by `metrics.jsonl`, W&B and the analysis readers.

Local keys: `train/loss/<Term>[/<aux>]`, `train/schedules/<name>`, `train/grad_norm/<group>`,
`train/perf/<name>`, `eval/<metric>/...`, `nontarget/...`. The `legacy` W&B schema mirrors local keys
unchanged; the `v2` schema groups them into panels (`loss/`, `recon/`, `sparsity/`, `perf/`, `eval/`).

Parity: param_decomp/metric_names.py, metric_schema.py, metric_taxonomy.py; docs/wandb-metrics.md.
"""

from __future__ import annotations

import re
from typing import Literal

MetricSchema = Literal["legacy", "v2"]

_SECTIONS = (
    (re.compile(r"^train/loss/(Faithfulness|.*Minimality|Nonlinearity)"), "objective"),
    (re.compile(r"^train/loss/.*Recon"), "recon"),
    (re.compile(r"^train/loss/total$"), "objective"),
    (re.compile(r"^train/schedules/"), "schedules"),
    (re.compile(r"^train/grad_norm/"), "optimization"),
    (re.compile(r"^train/perf/"), "perf"),
    (re.compile(r"^eval/l0/"), "sparsity"),
    (re.compile(r"^eval/(ce|kl|ce_unrecovered)/"), "lm_quality"),
    (re.compile(r"^eval/.*PGDReconLoss"), "adversarial"),
    (re.compile(r"^eval/identity_ci_error/"), "ground_truth"),
    (re.compile(r"^eval/"), "eval"),
)


def section_of(key: str) -> str:
    """Panel/section a metric key belongs to (the taxonomy)."""
    for pat, name in _SECTIONS:
        if pat.search(key):
            return name
    return "other"


def wandb_key(key: str, schema: MetricSchema) -> str:
    if schema == "legacy":
        return key
    leaf = key.split("/", 1)[1] if "/" in key else key
    return f"{section_of(key)}/{leaf}"


def validate_resume_schema(previous_keys: set[str], new_keys: set[str]) -> None:
    """A resumed run must keep logging the keys it logged before (renames break dashboards)."""
    missing = {k for k in previous_keys if k.startswith("train/loss/")} - new_keys
    assert not missing, f"resumed run no longer logs {sorted(missing)}"
