"""Evaluation fidelity: accumulated CI reductions (histograms, mean CI, density, density heat map), permutation
metrics (Hungarian identity / dense distances), the PGD probe with auxiliaries, figures on disk."""
import copy
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch

import __graft_entry__ as ge
from param_decomp_b200.evals import permutation as perm
from param_decomp_b200.evals import reductions as R


def test_fold_matches_direct_statistics_over_batches():
    torch.manual_seed(0)
    acc = R.ReductionAccumulation(n_bins=10, n_comp_bins=5, alive_threshold=0.2)
    batches = [{"s": torch.rand(3, 7, 6)} for _ in range(4)]
    for b in batches:
        R.fold(acc, b)
    red = R.finalize(acc)["s"]
    allv = torch.cat([b["s"].reshape(-1, 6) for b in batches])
    assert red.n_positions == 84
    assert np.allclose(red.mean_ci, allv.mean(0).numpy(), atol=1e-6)
    assert np.allclose(red.density, (allv > 0.2).float().mean(0).numpy(), atol=1e-6)
    assert red.hist.sum() == allv.numel() and red.comp_hist.shape == (6, 5)
    assert np.allclose(red.comp_hist.sum(1), 84)
    sc = R.histogram_scalars({"s": red})
    assert sc["ci_hist/s/frac_above_0.5"] == pytest.approx(float((allv >= 0.5).float().mean()), abs=0.02)
    # two "ranks" holding half of the batches each sum to the same reduction
    a1, a2 = R.ReductionAccumulation(n_bins=10), R.ReductionAccumulation(n_bins=10)
    for b in batches[:2]:
        R.fold(a1, b)
    for b in batches[2:]:
        R.fold(a2, b)
    other = {id(t): u for s1, s2 in zip(a1.sites.values(), a2.sites.values())
             for t, u in ((s1.ci_sum, s2.ci_sum), (s1.alive, s2.alive), (s1.hist, s2.hist))}
    a1.sites["s"].n_positions  # noqa: B018
    def sum_fn(t):
        if t.numel() == 1 and id(t) not in other:
            return t.add_(float(a2.sites["s"].n_positions))
        return t.add_(other[id(t)])
    R.merge_over_ranks(a1, sum_fn)
    merged = R.finalize(a1)["s"]
    assert merged.n_positions == 84 and np.allclose(merged.mean_ci, allv.mean(0).numpy(), atol=1e-6)


def test_permutation_distances():
    eye = np.eye(4)[:, [2, 0, 3, 1]]
    ci = np.concatenate([eye, np.zeros((4, 2))], axis=1)  # 6 components, 4 features, two dead
    permuted, p = perm.permute_to_identity(ci)
    assert np.allclose(permuted[:, :4], np.eye(4)) and sorted(p.tolist()) == list(range(6))
    assert perm.identity_ci_error(ci, 0.1) == 0
    noisy = ci.copy()
    noisy[0, 4] = 0.5  # one off-pattern entry
    noisy[1, p[1]] = 0.6  # one weak diagonal entry
    assert perm.identity_ci_error(noisy, 0.1) == 2
    dense = np.zeros((5, 4))
    dense[:, 1] = 1.0
    assert perm.dense_ci_error(dense, k=1) == 0 and perm.dense_ci_error(dense, k=2) == 1


def test_tms_slow_evals_write_figures_and_scalars():
    from param_decomp_b200.config.experiments import TMSExperimentConfig
    from param_decomp_b200.experiments.tms.run import run_tms

    import yaml

    raw = yaml.safe_load((Path(ge.__file__).parent / "param_decomp_b200/experiments/configs/tms_5-2.yaml").read_text())
    raw["pd"].update({"steps": 4, "batch_size": 64})
    raw["target"]["pretrain"]["steps"] = 20
    raw["pd"]["faithfulness_warmup_steps"] = 0
    raw["eval"] = {"batch_size": 64, "n_steps": 2, "every": 2, "slow_every": 4, "slow_on_first_step": False, "metrics": [
        {"type": "CI_L0", "groups": None}, {"type": "CIHistograms", "n_batches_accum": 3, "density_heatmap_n_bins": 8},
        {"type": "CIMeanPerComponent"}, {"type": "ComponentActivationDensity", "ci_alive_threshold": 0.1},
        {"type": "IdentityCIError", "identity_ci": [{"layer_pattern": "linear1", "n_features": 5}], "dense_ci": None},
        {"type": "PermutedCIPlots", "identity_patterns": ["linear1"], "dense_patterns": ["linear2"]},
        {"type": "UVPlots", "identity_patterns": ["linear*"], "dense_patterns": None},
        {"type": "PGDReconLoss", "init": "random", "source_shape": "c", "n_steps": 2, "step_size": 0.1}]}
    raw["cadence"] = {"train_log_every": 2, "checkpointing": {"kind": "none"}}
    cfg = TMSExperimentConfig.model_validate(raw)
    with tempfile.TemporaryDirectory() as root:
        res = run_tms(cfg, Path(root), run_id="p-0000e7a1")
        import json

        lines = [json.loads(l) for l in (res.run_dir / "metrics.jsonl").read_text().splitlines()]
        keys = {k for l in lines for k in l}
        for want in ("eval/ci_hist/linear1/frac_above_0.5", "eval/ci_mean/linear1/n_dead",
                     "eval/activation_density/linear2/alive_frac", "eval/identity_ci_error/linear1",
                     "eval/loss/PGDReconLoss_2step", "eval/l0/0.0_linear1"):
            assert want in keys, (want, sorted(k for k in keys if k.startswith("eval/"))[:40])
        figs = {p.name for p in (res.run_dir / "figures").iterdir()}
        assert any(n.startswith("ci_histograms_step4") for n in figs) and any(n.startswith("mean_ci_step4") for n in figs)
        assert any(n.startswith("ci_density_heatmap_step4") for n in figs)
        assert any(n.startswith("permuted_ci_linear1") for n in figs) and any(n.startswith("uv_linear1_V") for n in figs)
