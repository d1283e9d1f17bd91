"""The spelling of metric keys in `metrics.jsonl` and in the W&B mirror under the `legacy` schema.

Inside the engine a metric has a short internal key (`grad_norm/components`, `schedules/lr_ci_fn`, `kl/ci_masked`);
what is WRITTEN uses the reference's spellings, so analysis scripts and dashboards built on its runs read these runs
unchanged. The translation is a pure function of the key. Keys the reference does not have (this package's
additions: `ce/<variant>`, `ce_unrecovered/<variant>`, `l0/per_position/...`, `schedules/p`, throughput and MFU
names) keep a spelling in the same family.

Parity: param_decomp/core/run.py:430-442 (`_METRIC_KEYS`), :1577-1580 (`train/schedules/lr/*`),
core/train.py:192-230 (`grad_norms/summary/*`), experiments/lm/eval.py:383-389 (`ce_kl/kl_*`,
`ce_kl/ce_difference_*`), core/recon_eval.py:253 (`loss/<PGD read-out>`), core/ci_l0_eval.py:89 (`l0/<thr>_<site>`,
spelled by `evals/core.py::ci_l0` itself).
"""

from __future__ import annotations

import re

_TRAIN = {
    "train/grad_norm/components": "train/grad_norms/summary/components",
    "train/grad_norm/ci_fn": "train/grad_norms/summary/ci_fns",
    "train/grad_norm/total": "train/grad_norms/summary/total",
    "train/schedules/gamma": "train/schedules/gamma_imp",
    "train/schedules/lr_components": "train/schedules/lr/components",
    "train/schedules/lr_ci_fn": "train/schedules/lr/ci_fn",
    "train/schedules/lr_src": "train/schedules/lr/src",
    "train/perf/mfu": "train/perf/step_mfu_without_optimizer",
    "train/perf/mfu_with_optimizer": "train/perf/step_mfu_with_optimizer",
}
_PRETRAIN = {  # the pretrainer's records carry no prefix in the reference (param_decomp/pretrain/train.py:217-262)
    "pretrain/loss": "train_loss",
    "pretrain/val_loss": "val_loss",
    "pretrain/lr": "lr",
    "pretrain/step_time_s": "step_time_s",
}
_TRAIN.update(_PRETRAIN)
_NONTARGET = "train/nontarget/loss/"
_CE_KL = re.compile(r"^(?P<head>(?:eval/)(?:ArithmeticCIGrid/probe/)?)(?P<measure>kl|ce|ce_difference|ce_unrecovered)/(?P<variant>[a-z_]+)$")
_PGD = re.compile(r"^(?P<head>eval/(?:ArithmeticCIGrid/probe/)?)(?P<probe>(?:Slow)?PGDReconLoss_\d+step)(?P<rest>(?:/.*)?)$")


def reference_key(key: str) -> str:
    """Internal key (with its `train/` / `eval/` prefix) -> the key that is written."""
    if key in _TRAIN:
        return _TRAIN[key]
    if key.startswith(_NONTARGET):  # the broad stream of a targeted run (param_decomp/core/train.py:1749-1770)
        name = key[len(_NONTARGET):]
        return "train/loss/nontarget/" + ("imp" if name.endswith("ImportanceMinimalityLoss") else name)
    m = _CE_KL.match(key)
    if m is not None:
        return f"{m['head']}ce_kl/{m['measure']}_{m['variant']}"
    m = _PGD.match(key)
    if m is not None:
        return f"{m['head']}loss/{m['probe']}{m['rest']}"
    return key


def reference_keys(record: dict) -> dict:
    out = {reference_key(k): v for k, v in record.items()}
    assert len(out) == len(record), "two internal metric keys were written under one name"
    return out


_TRAIN_BACK = {v: k for k, v in _TRAIN.items()}
_CE_KL_BACK = re.compile(r"^(?P<head>eval/(?:ArithmeticCIGrid/probe/)?)ce_kl/(?P<measure>ce_difference|ce_unrecovered|kl|ce)_(?P<variant>[a-z_]+)$")
_PGD_BACK = re.compile(r"^(?P<head>eval/(?:ArithmeticCIGrid/probe/)?)loss/(?P<probe>(?:Slow)?PGDReconLoss_\d+step(?:/.*)?)$")


def internal_key(key: str) -> str:
    """Inverse of `reference_key`: a written key -> the internal key (identity on internal keys)."""
    if key in _TRAIN_BACK:
        return _TRAIN_BACK[key]
    if key.startswith("train/loss/nontarget/"):
        name = key[len("train/loss/nontarget/"):]
        return _NONTARGET + ("ImportanceMinimalityLoss" if name == "imp" else name)
    m = _CE_KL_BACK.match(key)
    if m is not None:
        return f"{m['head']}{m['measure']}/{m['variant']}"
    m = _PGD_BACK.match(key)
    if m is not None:
        return f"{m['head']}{m['probe']}"
    return key
