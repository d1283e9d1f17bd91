"""Analytical FLOP accounting: closed-form checks of the terms."""
import copy

import pytest

import __graft_entry__ as ge
from param_decomp_b200.utils import flops as F


def test_newton_schulz_and_optimizer_terms():
    import torch

    from param_decomp_b200.config.run import AdamWOptimizerConfig, MuonOptimizerConfig

    # one 4 x 6 matrix, one step: triangle 10 -> 2*10*6 + 2*10*4 + 2*16*6 = 392
    assert F.newton_schulz_flops(6, 4, 1, 1) == 392
    assert F.newton_schulz_flops(4, 6, 3, 5) == 3 * 5 * 392
    adam = AdamWOptimizerConfig(lr_schedule=1e-3, weight_decay=0.1, grad_clip_norm=1.0)
    c, a = F.optimizer_flops("g", adam, [torch.zeros(10, 3), torch.zeros(5)])
    assert c == 0 and a == 35 * 13 + 3 * 35 + 2
    muon = MuonOptimizerConfig(type="muon", lr_schedule=1e-3)
    c, a = F.optimizer_flops("g", muon, [torch.zeros(2, 4, 6), torch.zeros(5)])
    assert c == F.newton_schulz_flops(4, 6, 2, muon.ns_steps) and a > 0


def test_step_breakdown_matches_hand_count():
    from param_decomp_b200.config.experiments import LMExperimentConfig
    from param_decomp_b200.experiments.lm.build import build_lm_run

    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"]["backend"] = "eager_torch"
    cfg = LMExperimentConfig.model_validate(c)
    run = build_lm_run(cfg, None, "cpu")
    sf = F.step_flops(run.model, run.ci_fn, cfg.pd, cfg.data.seq_len)
    a = run.model.arch
    T, positions = cfg.data.seq_len, cfg.pd.batch_size * cfg.data.seq_len
    hd = a.d_model // a.n_head
    target = a.n_layer * (2 * a.d_model * hd * 4 * a.n_head + 2 * T * a.n_head * hd + 2 * a.d_model * a.d_ff * 3) \
        + 2 * a.d_model * a.vocab_size
    assert sf.model["clean_forward"].forward == pytest.approx(target * positions)
    comp = sum(2 * s.C * (s.d_in + s.d_out) for s in run.model.sites)
    rec = sf.model["recon/StochasticReconLoss"]
    assert rec.forward == pytest.approx((target + comp) * positions * 2) and rec.backward == pytest.approx(2 * rec.forward)
    assert sf.model["faithfulness"].forward == pytest.approx(sum(2 * s.d_in * s.d_out * s.C for s in run.model.sites))
    assert sf.model_total == pytest.approx(F.decomposition_step_flops(run.model, run.ci_fn, cfg.pd, T))
    assert sf.model["ci_fn"].backward > sf.model["ci_fn"].forward
