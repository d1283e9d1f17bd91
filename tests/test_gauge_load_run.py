"""Gauge utilities, the nonlinearity evaluation and re-opening a finished run."""
import torch

from param_decomp_b200.core import gauge, nonlinearity_eval
from param_decomp_b200.experiments.lm import load_run
from param_decomp_b200.experiments.lm.training import train_lm
from tests.test_targeted_lm import _targeted_config
from param_decomp_b200.config.experiments import LMExperimentConfig


def _config():
    raw = _targeted_config().model_dump(mode="json")
    for k in ("prompts", "nontarget"):
        raw.pop(k)
    raw["pd"]["loss_metrics"].append({"type": "FaithfulnessLoss", "coeff": 10.0})
    raw["pd"]["steps"] = 4
    raw["pd"].pop("ci_scaled_weight_decay", None)
    raw["cadence"] = {"train_log_every": 2, "checkpointing": {"kind": "periodic", "save_every": 2, "retention": {"kind": "keep_all"}}}
    return LMExperimentConfig.model_validate(raw)


def test_gauge_balance_keeps_the_function_and_open_run_restores(tmp_path):
    cfg = _config()
    states: list = []
    res = train_lm(cfg, tmp_path, device="cpu", state_out=states)
    comps = states[0].components
    W0 = {s.name: comps.weight(s.name).clone() for s in comps.sites}
    m0 = gauge.uv_norm_ratio_metrics(comps)
    assert "uv_norm_ratio_mean" in m0 and m0["uv_norm_ratio_max"] >= m0["uv_norm_ratio_mean"]
    gauge.balance(comps)
    for s in comps.sites:
        assert torch.allclose(comps.weight(s.name), W0[s.name], atol=1e-5)
    m1 = gauge.uv_norm_ratio_metrics(comps)
    V, U = comps.site(comps.sites[0].name)
    assert torch.allclose(torch.linalg.vector_norm(V, dim=0), gauge.u_norms_of(U), rtol=1e-4)
    act = torch.randn(5, V.shape[1])
    inv = gauge.gauge_invariant_activation(act, gauge.u_norms_of(U))
    assert torch.allclose(gauge.gauge_variant_activation(inv, gauge.u_norms_of(U)), act, atol=1e-5)
    stats = nonlinearity_eval.component_nonlinearity_stats(comps)
    assert stats and all(v["effective_count"].min() >= 0.99 for v in stats.values())
    assert nonlinearity_eval.nonlinearity_log_entries(stats)
    # re-open the run read-only
    meta = load_run.run_metadata(res.run_dir)
    assert meta.steps_saved and meta.sites["q"] == 8
    opened = load_run.open_run(res.run_dir, None, device="cpu")
    assert opened.step == meta.steps_saved[-1] and opened.ci_fn is not None
    assert all(not p.requires_grad for p in opened.components.parameters())
    only = load_run.open_target_and_components(res.run_dir, None, step=meta.steps_saved[0])
    assert only.ci_fn is None and only.step == meta.steps_saved[0]
    assert m1["uv_norm_ratio_mean"] > 0
    # the stable facts of the run, resolved without a checkpoint (no target tensor is materialised)
    d = load_run.load_deliverable(res.run_dir)
    assert [s.name for s in d.sites] == [s.name for s in opened.model.sites] and d.seed == cfg.pd.seed
    assert all((a.d_in, a.d_out, a.C) == (b.d_in, b.d_out, b.C) for a, b in zip(d.sites, opened.model.sites))
    assert d.arch.n_layer == opened.model.arch.n_layer and d.data.seq_len == cfg.data.seq_len and d.data.train_dir is None
    assert d.ci_tap_widths and all(w > 0 for w in d.ci_tap_widths.values())

