"""Metric key grammar: local keys, and the grouped names a W&B workspace is built from.

`metrics.jsonl` always holds the LOCAL keys (`train/loss/<Term>`, `train/schedules/<name>`, `train/grad_norm/
<group>`, `train/perf/<name>`, `eval/<family>/...`). The W&B mirror logs them unchanged under the `legacy`
schema, or - `grouped` - as two-level `<group>/<chart>` names in lowercase dash-separated words, so that a
group is one panel section and its charts sort in reading order (sites by depth, then by their place in a
block). The mapping is a pure function of the key, it refuses names outside the grammar, and two local keys may
never map to the same grouped name. A run keeps the schema it was started with.

Parity: param_decomp/metric_names.py (`MetricKey`, `MetricGroup`, name validation), metric_schema.py (`MetricNames`,
`recorded_metric_schema`, `validate_resume_schema`), metric_taxonomy.py (`grouped_metric_key`: the key -> group /
chart grammar, site labels `layer-NN-CC-<role>`), docs/wandb-metrics.md.
"""

from __future__ import annotations

import re
from collections.abc import Mapping
from dataclasses import dataclass
from typing import Literal

from param_decomp_b200.infra.weight_addressing import try_address

MetricSchema = Literal["legacy", "grouped", "v2"]  # `v2` is the older spelling of `grouped`

_NAME = re.compile(r"[a-z0-9]+(?:[-.][a-z0-9]+)*")
_PERFORMANCE = {"step_time_s", "elapsed_s", "eta_s", "tokens_per_s", "samples_per_s", "mfu", "useful_flops",
                "peak_memory_gb", "allocated_memory_gb"}
_CE_VARIANTS = {"ci_masked", "unmasked", "stoch_masked", "random_masked", "rounded_masked", "zero_masked", "target"}


def _validate(name: str) -> None:
    if _NAME.fullmatch(name) is None:
        raise ValueError(f"expected lowercase words joined by dashes or dots: {name!r}")


@dataclass(frozen=True)
class MetricKey:
    group: str
    chart: str

    def __post_init__(self) -> None:
        _validate(self.group)
        _validate(self.chart)

    @property
    def path(self) -> str:
        return f"{self.group}/{self.chart}"


@dataclass(frozen=True)
class MetricGroup:
    name: str
    charts: tuple[str, ...]

    def __post_init__(self) -> None:
        _validate(self.name)
        if not self.charts or len(set(self.charts)) != len(self.charts):
            raise ValueError(f"a metric group needs a non-empty, unique chart list: {self.name}")
        for c in self.charts:
            _validate(c)

    def key(self, chart: str) -> MetricKey:
        if chart not in self.charts:
            raise ValueError(f"unknown chart {chart!r} in group {self.name!r}")
        return MetricKey(self.name, chart)


def label(value: str) -> str:
    """A key segment as a dash-separated lowercase word: `StochasticReconLoss` -> `stochastic-recon-loss`,
    `ci_masked` -> `ci-masked`, `layer_3` -> `layer-03`, `gt_0.1` -> `gt-0.1`."""
    m = re.fullmatch(r"(layer|block|depth|group)[_.](\d+)", value)
    if m:
        return f"{m[1]}-{int(m[2]):02d}"
    v = re.sub(r"(?<=[a-z0-9])(?=[A-Z])", "-", value).lower()
    v = re.sub(r"[^a-z0-9.]+", "-", v).strip("-.")
    return v or "value"


def site_label(site: str) -> str:
    """`layer-03-02-attn-k` for a site with a canonical address, else the site's own words."""
    addr = try_address(site)
    return addr.label if addr is not None else label(site.replace(".", "-"))


def named(parts: tuple[str, ...], chart: str) -> MetricKey:
    return MetricKey("-".join(label(p) for p in parts), label(chart))


def _strip_brackets(chart: str) -> tuple[str, str | None]:
    """`uv_norm_ratio['layers.0.mlp.up_proj']` -> (`uv_norm_ratio`, `layers.0.mlp.up_proj`)."""
    m = re.fullmatch(r"([\w.]+)\['(.+)'\]", chart)
    return (m[1], m[2]) if m else (chart, None)


def grouped_metric_key(key: str) -> MetricKey:
    """The grouped name of a local key (internal or as written to `metrics.jsonl`, `infra/reference_keys.py`).
    Raises `ValueError` for keys outside the grammar."""
    from param_decomp_b200.infra.reference_keys import internal_key

    key = internal_key(key)
    pretrain = {"pretrain/loss": ("pretrain-loss", "train"), "pretrain/val_loss": ("pretrain-loss", "validation"),
                "pretrain/lr": ("pretrain-schedules", "lr"), "pretrain/step_time_s": ("pretrain-performance", "step-time-s")}
    if key in pretrain:
        return MetricKey(*pretrain[key])
    parts = tuple(key.split("/"))
    match parts:
        case ("train", "loss", "total"):
            return MetricKey("train-loss", "total")
        case ("train", "loss", term):
            return named(("train", "loss"), term)
        case ("train", "loss", term, aux):
            return named(("train", "reconstruction", aux), term)
        case ("train", "nontarget", "loss", term):
            return named(("train", "loss", "nontarget"), term)
        case ("train", "nontarget", "schedules", chart):
            return named(("train", "schedules", "nontarget"), chart)
        case ("train", "schedules", chart):
            return named(("train", "schedules"), chart)
        case ("train", "grad_norm", chart):
            return named(("train", "grad_norm"), chart)
        case ("train", "perf", chart) if chart in _PERFORMANCE or chart.startswith(("mfu", "useful_")):
            return named(("train", "performance"), chart)
        case ("train", "perf", chart):
            return named(("train", "performance"), chart)
        case ("train", "mem", chart):
            return named(("train", "memory"), chart)
        case ("train", chart) if chart.startswith("uv_norm_ratio"):
            base, site = _strip_brackets(chart)
            return MetricKey("train-uv-norm-ratio", site_label(site) if site else label(base[len("uv_norm_ratio"):] or "all"))
        case ("eval", "l0", "per_position", thr, stat):
            return named(("eval", "ci", "l0", "per_position"), f"{thr}-{stat}")
        case ("eval", "l0", site_or_group):
            thr = re.match(r"^(\d+(?:\.\d+)?(?:e-?\d+)?)_(.+)$", site_or_group)  # `<threshold>_<site or group>`
            if thr is not None:
                tag = thr.group(1).replace(".", "p")
                return MetricKey(f"eval-ci-l0-gt-{tag}", site_label(thr.group(2)))
            return MetricKey("eval-ci-l0", site_label(site_or_group))
        case ("eval", ("ce" | "kl" | "ce_unrecovered" | "ce_difference") as measure, variant) if variant in _CE_VARIANTS:
            return named(("eval", "reconstruction", measure), variant)
        case ("eval", ("ci_hist" | "ci_mean" | "activation_density") as family, site, stat):
            return MetricKey(f"eval-ci-{label(family[3:] if family.startswith('ci_') else family)}-{label(stat)}",
                             site_label(site))
        case ("eval", ("identity_ci_error" | "dense_ci_error") as family, site):
            return MetricKey(f"eval-{label(family)}", site_label(site))
        case ("eval", probe) if re.fullmatch(r"(Slow)?PGDReconLoss_\d+step", probe):
            kind, steps = probe.rsplit("_", 1)
            return named(("eval", "reconstruction", "pgd"), f"{label(kind)}-{int(steps[:-4]):05d}-steps")
        case ("eval", probe, aux) if re.fullmatch(r"(Slow)?PGDReconLoss_\d+step", probe):
            kind, steps = probe.rsplit("_", 1)
            return named(("eval", "reconstruction", "pgd", aux), f"{label(kind)}-{int(steps[:-4]):05d}-steps")
        case ("eval", ("CIMaskedAttnPatternsReconLoss" | "StochasticAttnPatternsReconLoss") as fam):
            return named(("eval", "attention_pattern", "kl"), fam.replace("AttnPatternsReconLoss", "") + "-all-layers")
        case ("eval", ("CIMaskedAttnPatternsReconLoss" | "StochasticAttnPatternsReconLoss") as fam, layer):
            return named(("eval", "attention_pattern", "kl", fam.replace("AttnPatternsReconLoss", "")), layer)
        case ("eval", "router", measure, strategy, layer):
            return named(("eval", "router", measure, strategy), layer)
        case ("eval", family, *rest) if rest:
            return MetricKey("eval-" + label(family), "-".join(site_label(r) if try_address(r) else label(r) for r in rest))
        case ("eval", chart):
            return named(("eval", "summary"), chart)
        case ("pretrain", family, chart):
            return named(("pretrain", family), chart)
    raise ValueError(f"metric key outside the naming grammar: {key!r}")


def recorded_metric_schema(config: Mapping[str, object]) -> str:
    """The schema a stored run config was logged with (runs from before the option existed: `legacy`)."""
    wandb = config.get("wandb") or {}
    schema = wandb.get("metric_schema", "legacy") if isinstance(wandb, Mapping) else "legacy"
    return "grouped" if schema == "v2" else str(schema)


def validate_resume_schema(config: Mapping[str, object], requested: str) -> None:
    """A resumed run must keep the names it started with (a rename splits every chart of its workspace)."""
    recorded = recorded_metric_schema(config)
    requested = "grouped" if requested == "v2" else requested
    if recorded != requested:
        raise ValueError(f"cannot resume with wandb.metric_schema={requested!r}: the run was logged with "
                         f"{recorded!r}; start a new run instead")


class MetricNames:
    """Key translation for one run, with collision detection: two local keys never share a grouped name."""

    def __init__(self, schema: str = "legacy") -> None:
        self.schema = "grouped" if schema == "v2" else schema
        assert self.schema in ("legacy", "grouped"), schema
        self._sources: dict[str, str] = {}

    def metric(self, key: str) -> str:
        if self.schema == "legacy":
            return key
        dest = grouped_metric_key(key).path
        prev = self._sources.get(dest)
        if prev is not None and prev != key:
            raise ValueError(f"metric name collision: {prev!r} and {key!r} both map to {dest!r}")
        self._sources[dest] = key
        return dest

    def record(self, record: Mapping[str, object]) -> dict[str, object]:
        return {self.metric(k): v for k, v in record.items()}
