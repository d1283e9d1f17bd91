"""The train step recorded as a CUDA graph (`core/recorded_step.py`) against the same step issued launch by
launch: the loss trajectory must agree (masks, schedules, learning rates and bias corrections come from the
device scalar table in both), masks must change from replay to replay, and the scheduled `gamma` must follow
its schedule while replaying."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(record: bool, steps: int = 8):
    import __graft_entry__ as ge
    from param_decomp_b200.config.experiments import LMExperimentConfig
    from param_decomp_b200.core.objective import build_objective
    from param_decomp_b200.core.recorded_step import RecordedTrainStep
    from param_decomp_b200.core.run import init_train_state
    from param_decomp_b200.core.train import StepContext
    from param_decomp_b200.experiments.lm.build import build_lm_run

    dev = torch.device("cuda", 0)
    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"]["backend"] = "fused_sm100"
    c["pd"]["steps"] = 20
    c["pd"]["loss_metrics"] = [
        {"type": "ImportanceMinimalityLoss", "coeff": 1e-3,
         "gamma": {"max_val": 1.0, "points": [{"at": 0.0, "frac": 1.0}, {"at": 1.0, "frac": 0.1}]}},
        {"type": "StochasticReconLoss", "coeff": 1.0, "n_samples": 2},
        {"type": "FaithfulnessLoss", "coeff": {"max_val": 10.0, "points": [{"at": 0.0, "frac": 1.0}, {"at": 1.0, "frac": 0.5}]}},
    ]
    c["pd"]["components_optimizer"] = {"lr_schedule": {"max_val": 1e-3, "points": [{"at": 0.0, "frac": 1.0}, {"at": 1.0, "frac": 0.1}]},
                                       "grad_clip_norm": 1.0}
    cfg = LMExperimentConfig.model_validate(c)
    run = build_lm_run(cfg, None, dev)
    obj = build_objective(cfg.pd)
    ctx = StepContext.build(run.model, obj, cfg.pd, lazy_masks=True)
    st = init_train_state(run.model, run.ci_fn, cfg.pd, obj, dev, cfg.pd.batch_size, cfg.data.seq_len, use_fused_optim=True)
    stepper = RecordedTrainStep(ctx, st, enabled=record, eager_steps=2)
    out = []
    for s in range(steps):
        m = stepper(run.sample_train(s))
        out.append({k: float(v) for k, v in m.items()})
    return stepper, st, out, cfg


def test_recorded_step_follows_eager_step():
    from param_decomp_b200.config.schedule import get_scheduled_value
    from param_decomp_b200.ops import native

    rec, st_r, got, cfg = _setup(True)
    assert rec.eligible, rec.reason
    assert rec.graph is not None and rec.replays == 6  # 2 eager, then the recording + 5 replays
    eag, st_e, ref, _ = _setup(False)
    assert eag.graph is None
    native.check_status()
    assert st_r.step == st_e.step == 8
    assert st_r.components_opt.count == st_e.components_opt.count == 8
    for s, (a, b) in enumerate(zip(got, ref)):
        for k in ("loss/total", "loss/StochasticReconLoss", "loss/FaithfulnessLoss", "loss/ImportanceMinimalityLoss",
                  "grad_norm/components", "grad_norm/ci_fn"):
            assert a[k] == pytest.approx(b[k], rel=5e-3, abs=1e-7), (s, k, a[k], b[k])
        # scheduled quantities are read from the device table by the replayed launches
        assert a["schedules/gamma"] == pytest.approx(get_scheduled_value(s, 20, cfg.pd.loss_metrics[0].gamma), rel=1e-6)
        assert a["schedules/lr_components"] == pytest.approx(b["schedules/lr_components"], rel=1e-6)
    # a replay draws new masks (the seed word changes) and sees new tokens: the recon loss moves between replays
    recon = [m["loss/StochasticReconLoss"] for m in got[3:]]
    assert len({round(v, 9) for v in recon}) == len(recon)
    # Adam turns a last-bit difference of a near-zero gradient (the order of the fp32 reduce-adds is not fixed)
    # into a full-size step, so single elements may differ by up to lr x steps; on average they agree
    for a, b in zip(st_r.components.parameters(), st_e.components.parameters()):
        d = (a.detach() - b.detach()).abs()
        assert float(d.mean()) < 5e-5 and float(d.max()) <= 8 * 1e-3 + 1e-6, (float(d.mean()), float(d.max()))


def test_recording_refused_with_reason():
    import __graft_entry__ as ge
    from param_decomp_b200.config.experiments import LMExperimentConfig
    from param_decomp_b200.core.objective import build_objective
    from param_decomp_b200.core.recorded_step import RecordedTrainStep
    from param_decomp_b200.core.run import init_train_state
    from param_decomp_b200.core.train import StepContext
    from param_decomp_b200.experiments.lm.build import build_lm_run

    dev = torch.device("cuda", 0)
    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"]["backend"] = "fused_sm100"
    c["pd"]["loss_metrics"] = [
        {"type": "ImportanceMinimalityLoss", "coeff": 1e-3, "gamma": 1.0},
        {"type": "PersistentPGDReconLoss", "coeff": 1.0, "source_shape": "bc", "n_warmup_steps": 1,
         "optimizer": {"type": "adam", "lr_schedule": 0.05}},
        {"type": "FaithfulnessLoss", "coeff": 10.0},
    ]
    cfg = LMExperimentConfig.model_validate(c)
    run = build_lm_run(cfg, None, dev)
    obj = build_objective(cfg.pd)
    ctx = StepContext.build(run.model, obj, cfg.pd, lazy_masks=True)
    st = init_train_state(run.model, run.ci_fn, cfg.pd, obj, dev, cfg.pd.batch_size, cfg.data.seq_len, use_fused_optim=True)
    stepper = RecordedTrainStep(ctx, st)
    assert not stepper.eligible and "persistent" in stepper.reason
    for s in range(4):
        stepper(run.sample_train(s))  # stays eager
    assert stepper.graph is None and st.step == 4
