"""From the YAML loss list to the runtime objective.

`PDObjective` holds the faithfulness term, the importance-minimality term, an optional
nonlinearity-locality term and the ordered reconstruction terms; the order of the recon list is the
RNG order (term index keys each term's Philox streams). A recon term = mask-source strategy x
routing sampler x auxiliaries.

Parity: param_decomp/core/objective.py:196-449 (roles from the loss list, unique names),
core/recon.py:46-264 (strategy and routing vocabulary).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Literal

from param_decomp_b200.config import losses as L
from param_decomp_b200.config.run import NontargetConfig, PDConfig, TargetedPDConfig
from param_decomp_b200.config.schedule import ScheduleConfig, scheduled_or_constant

Strategy = Literal["stochastic", "ci_masked", "unmasked", "unmasked_no_delta", "fresh_pgd",
                   "persistent", "merged", "merged_pooled"]

_STRATEGY_OF: dict[type, Strategy] = {
    L.StochasticReconLossConfig: "stochastic",
    L.StochasticReconSubsetLossConfig: "stochastic",
    L.CIMaskedReconLossConfig: "ci_masked",
    L.CIMaskedReconSubsetLossConfig: "ci_masked",
    L.UnmaskedReconLossConfig: "unmasked",
    L.UnmaskedNoDeltaReconLossConfig: "unmasked_no_delta",
    L.PGDReconLossConfig: "fresh_pgd",
    L.PGDReconSubsetLossConfig: "fresh_pgd",
    L.PersistentPGDReconLossConfig: "persistent",
    L.MergedStochasticSubsetPPGDReconLossConfig: "merged",
    L.MergedStochasticSubsetPooledPPGDReconLossConfig: "merged_pooled",
}


@dataclass(frozen=True)
class ReconTerm:
    name: str
    index: int
    strategy: Strategy
    cfg: L.BaseConfig
    routing_kind: str = "all"
    routing_p: float | None = None
    n_samples: int = 1
    delta_pinned: float | None = None  # non-target pass: delta mask pinned to 1

    @property
    def is_persistent(self) -> bool:
        return self.strategy in ("persistent", "merged", "merged_pooled")

    @property
    def auxiliaries(self) -> tuple[L.AuxiliaryReconstructionConfig, ...]:
        return getattr(self.cfg, "auxiliaries", ())

    def coeff(self, step: int, total: int) -> float:
        return scheduled_or_constant(self.cfg.coeff, step, total)  # type: ignore[attr-defined]

    def capture_keys(self) -> tuple[str, ...]:
        return tuple(c.capture for a in self.auxiliaries for c in a.comparisons)


def _routing(cfg: L.BaseConfig) -> tuple[str, float | None]:
    r = getattr(cfg, "routing", None)
    if r is None:
        return "all", None
    return r.type, getattr(r, "p", None)


def build_recon_term(cfg: L.BaseConfig, index: int, delta_pinned: float | None = None) -> ReconTerm:
    kind, p = _routing(cfg)
    return ReconTerm(name=cfg.instance_key, index=index, strategy=_STRATEGY_OF[type(cfg)], cfg=cfg,  # type: ignore[attr-defined]
                     routing_kind=kind, routing_p=p, n_samples=getattr(cfg, "n_samples", 1),
                     delta_pinned=delta_pinned)


@dataclass
class PDObjective:
    faith: L.FaithfulnessLossConfig | None
    minimality: L.ImportanceMinimalityLossConfig | L.LpImportanceMinimalityLossConfig
    nonlinearity: L.NonlinearityLocalityLossConfig | None
    recon: list[ReconTerm] = field(default_factory=list)

    def capture_keys(self) -> tuple[str, ...]:
        return tuple(dict.fromkeys(k for t in self.recon for k in t.capture_keys()))

    def persistent_terms(self) -> list[ReconTerm]:
        return [t for t in self.recon if t.is_persistent]


def build_objective(pd: PDConfig | TargetedPDConfig) -> PDObjective:
    faith = minimality = nonlin = None
    recon: list[ReconTerm] = []
    for cfg in pd.loss_metrics:
        if isinstance(cfg, L.FaithfulnessLossConfig):
            faith = cfg
        elif isinstance(cfg, (L.ImportanceMinimalityLossConfig, L.LpImportanceMinimalityLossConfig)):
            minimality = cfg
        elif isinstance(cfg, L.NonlinearityLocalityLossConfig):
            nonlin = cfg
        else:
            recon.append(build_recon_term(cfg, len(recon)))
    assert minimality is not None
    return PDObjective(faith, minimality, nonlin, recon)


@dataclass
class NontargetObjective:
    impmin_coeff: float | ScheduleConfig
    recon: list[ReconTerm]


def build_nontarget_objective(cfg: NontargetConfig, first_index: int) -> NontargetObjective:
    terms = []
    for i, r in enumerate(cfg.recon):
        pinned = None if isinstance(r, L.UnmaskedNoDeltaReconLossConfig) else 1.0
        terms.append(build_recon_term(r, first_index + i, delta_pinned=pinned))
    return NontargetObjective(cfg.impmin_coeff, terms)
