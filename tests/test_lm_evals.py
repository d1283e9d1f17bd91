"""Slow-tier LM evaluation operations on tiny CPU models."""
import math

import numpy as np
import torch

from param_decomp_b200.core.objective import build_objective
from param_decomp_b200.core.run import init_train_state
from param_decomp_b200.core.train import StepContext
from param_decomp_b200.evals import lm_ops
from param_decomp_b200.experiments.lm.build import build_lm_run
from param_decomp_b200.utils import figures
from tests.test_qwen35 import _config
from param_decomp_b200.models import qwen35


def _setup():
    cs = {k: (12 if k.startswith("experts_") else 8) for k in qwen35.KIND_ORDER}
    cfg = _config(cs)
    run = build_lm_run(cfg, None, "cpu")
    obj = build_objective(cfg.pd)
    ctx = StepContext.build(run.model, obj, cfg.pd, lazy_masks=False)
    state = init_train_state(run.model, run.ci_fn, cfg.pd, obj, torch.device("cpu"), 4, 24)
    return run, ctx, state


def test_router_divergence_and_well_temperedness(tmp_path):
    run, ctx, state = _setup()
    batch = run.sample_eval(0)
    rd = lm_ops.router_divergence(ctx, state, batch, ("ci_masked", "stochastic"))
    assert "RouterDivergence/ci_masked/kl" in rd and all(math.isfinite(v) for v in rd.values())
    assert all(0.0 <= v <= 1.0 for k, v in rd.items() if "topk_kept" in k)
    wt = lm_ops.well_temperedness(ctx, state, batch, n_locations=2, n_components=3, run_dir=tmp_path,
                                  groups={"attention": ["*self_attn*", "*linear_attn*"], "nothing": ["no_such_site*"]})
    assert 0.0 <= wt["WellTemperedness/all"] <= 1.0
    n_regions = sum(wt[f"WellTemperedness/{r}/n"] for r in ("below_zero", "zero_to_one", "above_one"))
    assert 0 < n_regions <= 2 * 3 * 3  # at most locations x regions x quota; padding is discarded
    assert wt["WellTemperedness/group/nothing/n"] == 0.0 and wt["WellTemperedness/group/attention/n"] <= n_regions
    assert (tmp_path / "figures" / "well_temperedness_pre_vs_damage.png").exists()


def test_router_divergence_under_adversarial_strategies():
    """`fresh_pgd` ascends batch-shared sources against the output loss before the read-out; `persistent` reads the
    run's persistent adversary (per-row sources: every evaluation sequence draws one training row)."""
    from param_decomp_b200.config import evals as E
    from param_decomp_b200.config.experiments import LMExperimentConfig

    cs = {k: (12 if k.startswith("experts_") else 8) for k in qwen35.KIND_ORDER}
    raw = _config(cs).model_dump(mode="json")
    raw["pd"]["loss_metrics"] = [
        {"type": "ImportanceMinimalityLoss", "coeff": 1e-3, "gamma": 1.0},
        {"type": "PersistentPGDReconLoss", "name": "ppgd", "coeff": 1.0, "source_shape": "bsc", "n_warmup_steps": 1,
         "optimizer": {"type": "adam", "lr_schedule": 0.05}},
        {"type": "FaithfulnessLoss", "coeff": 10.0}]
    cfg = LMExperimentConfig.model_validate(raw)
    run = build_lm_run(cfg, None, "cpu")
    obj = build_objective(cfg.pd)
    ctx = StepContext.build(run.model, obj, cfg.pd, lazy_masks=False)
    state = init_train_state(run.model, run.ci_fn, cfg.pd, obj, torch.device("cpu"), 4, 24)
    assert "ppgd" in state.adversaries
    metric = E.RouterDivergenceConfig.model_validate({"strategies": [
        {"kind": "ci_masked"}, {"kind": "fresh_pgd", "n_steps": 2, "step_size": 0.2},
        {"kind": "persistent", "state_key": "ppgd"}]})
    batch = run.sample_eval(0)
    rd = lm_ops.router_divergence(ctx, state, batch, tuple(metric.strategies))
    for kind in ("ci_masked", "fresh_pgd", "persistent"):
        assert f"RouterDivergence/{kind}/kl" in rd, sorted(rd)
    assert all(math.isfinite(v) for v in rd.values())
    # an adversary that ascended the output loss does not leave the router closer to the target than plain CI masks
    assert rd["RouterDivergence/fresh_pgd/kl"] >= rd["RouterDivergence/ci_masked/kl"] - 1e-6
    half = tuple(run.sample_eval(0).tokens[:2].shape)
    assert half == (2, 24)
    import dataclasses
    small = dataclasses.replace(batch, tokens=batch.tokens[:2]) if dataclasses.is_dataclass(batch) else batch
    rd2 = lm_ops.router_divergence(ctx, state, small, (metric.strategies[2],))  # 2 sequences, 4 training rows of sources
    assert math.isfinite(rd2["RouterDivergence/persistent/kl"])
    with __import__("pytest").raises(AssertionError):
        lm_ops.router_divergence(ctx, state, batch, (E.PersistentStrategy(state_key="missing"),))


def test_ordering_score():
    pre = torch.tensor([0.1, 0.5, 0.9, 1.5])
    assert lm_ops.fraction_well_ordered_pairs(pre, pre * 2) == 1.0
    assert lm_ops.fraction_well_ordered_pairs(pre, -pre) == 0.0
    assert lm_ops.fraction_well_ordered_pairs(pre, torch.zeros(4)) == 0.5


def test_arithmetic_grid_and_figures(tmp_path):
    run, ctx, state = _setup()
    enc = lambda s: [ord(c) % 97 for c in s]  # noqa: E731  one token per character
    grid = lm_ops.build_arithmetic_prompt_grid(enc, [1, 2, 3], [4, 5], "add")
    assert grid.tokens.shape == (6, 4) and grid.answers == [5, 6, 6, 7, 7, 8]
    out = lm_ops.arithmetic_ci_grid(ctx, state, grid, top_k=4, run_dir=tmp_path)
    assert any(k.endswith("n_alive") for k in out) and any(k.endswith("n_above_0.1") for k in out)
    from param_decomp_b200.config import evals as E

    metric = E.ArithmeticCIGridConfig.model_validate({
        "operation": "add", "a_range": [1, 3], "b_range": [4, 5], "thresholds": [0.1, 0.5], "top_k": 4,
        "probe_metrics": {"ce_kl": {"rounding_threshold": 0.1}, "ci_l0": {"ci_alive_threshold": 0.05, "groups": None},
                          "fresh_pgd": {"n_steps": 2, "step_size": 0.1}}})
    probed = lm_ops.arithmetic_ci_grid(ctx, state, grid, top_k=4, run_dir=tmp_path, thresholds=tuple(metric.thresholds),
                                       probe_metrics=metric.probe_metrics)
    assert "ArithmeticCIGrid/probe/PGDReconLoss_2step" in probed and any("n_above_0.5" in k for k in probed)
    assert any(k.startswith("ArithmeticCIGrid/probe/") and "kl" in k.lower() for k in probed), sorted(probed)[:12]
    assert all(math.isfinite(v) for v in probed.values())
    assert len(list((tmp_path / "figures").glob("arithmetic_ci_*.png"))) == len(run.model.sites)
    pm, perm = lm_ops.permute_to_identity(torch.eye(4)[:, [2, 0, 3, 1]])
    assert torch.equal(pm, torch.eye(4)) and sorted(perm.tolist()) == [0, 1, 2, 3]
    png = figures.heatmap(np.arange(12.0).reshape(3, 4))
    assert png[:8] == b"\x89PNG\r\n\x1a\n" and png[-8:-4] == b"IEND"
