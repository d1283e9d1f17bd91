"""Optimizer parity with torch references; adversary ascent rules and storage."""
import math

import pytest
import torch

from param_decomp_b200.config.losses import AdamPGDConfig, MomentumSgdPGDConfig, SgdPGDConfig
from param_decomp_b200.config.run import AdamWOptimizerConfig, MuonOptimizerConfig
from param_decomp_b200.core import adversary as A
from param_decomp_b200.core.components import SiteSpec
from param_decomp_b200.core.optim import build_group_optimizer, clip_scale, global_norm, newton_schulz
from param_decomp_b200.core.rng import StepKey


def test_adamw_matches_torch():
    torch.manual_seed(0)
    p0 = [torch.randn(5, 4), torch.randn(7)]
    ours = [p.clone() for p in p0]
    ref = [p.clone().requires_grad_(True) for p in p0]
    cfg = AdamWOptimizerConfig(lr_schedule=1e-2, weight_decay=0.1, betas=(0.9, 0.95))
    opt = build_group_optimizer(cfg, [("a", ours[0]), ("b", ours[1])], total_steps=100)
    topt = torch.optim.AdamW(ref, lr=1e-2, weight_decay=0.1, betas=(0.9, 0.95), eps=1e-8)
    for step in range(5):
        grads = [torch.randn_like(p) for p in p0]
        for r, g in zip(ref, grads):
            r.grad = g.clone()
        topt.step()
        opt.step(step, grads)
    for o, r in zip(ours, ref):
        assert torch.allclose(o, r.detach(), atol=1e-6)


def test_clip_matches_torch_clip_grad_norm():
    grads = [torch.randn(10) * 5, torch.randn(3, 3) * 5]
    n = global_norm(grads)
    ref = [g.clone().requires_grad_(True) for g in grads]
    for r, g in zip(ref, grads):
        r.grad = g.clone()
    tn = torch.nn.utils.clip_grad_norm_(ref, 1.0)
    assert float(n) == pytest.approx(float(tn), rel=1e-6)
    s = clip_scale(n, 1.0)
    assert torch.allclose(grads[0] * s, ref[0].grad, atol=1e-6)
    assert float(clip_scale(torch.tensor(0.5), 1.0)) == 1.0 and float(clip_scale(n, None)) == 1.0


def test_lr_schedule_is_applied_and_logged():
    cfg = AdamWOptimizerConfig(lr_schedule={"max_val": 1.0, "points": [{"at": 0, "frac": 1.0}, {"at": 1, "frac": 0.1}]})
    p = torch.zeros(2)
    opt = build_group_optimizer(cfg, [("p", p)], total_steps=11)
    opt.step(10, [torch.ones(2)])
    assert opt.applied_learning_rate == pytest.approx(0.1)


def test_newton_schulz_orthogonalises():
    torch.manual_seed(0)
    G = torch.randn(3, 16, 32)
    X = newton_schulz(G, steps=8, dtype=torch.float32)
    s = torch.linalg.svdvals(X)
    assert float(s.min()) > 0.6 and float(s.max()) < 1.3  # singular values pushed towards 1
    Xt = newton_schulz(G.transpose(1, 2).contiguous(), steps=8, dtype=torch.float32)
    assert torch.allclose(Xt, X.transpose(1, 2), atol=1e-4)


def test_muon_update_rule():
    """Three-step trajectory against a restatement of `optax.contrib.muon(nesterov=True)` as the reference
    configures it: EMA momentum, bias-corrected Nesterov mix, Newton-Schulz, shape scale, decoupled weight
    decay; non-matrix leaves by Nesterov Adam(0.9, 0.999) without weight decay."""
    torch.manual_seed(0)
    W, b = torch.randn(2, 8, 4), torch.randn(4)
    cfg = MuonOptimizerConfig(type="muon", lr_schedule=0.1, ns_dtype="float32", weight_decay=0.01)
    opt = build_group_optimizer(cfg, [("W", W), ("b", b)], total_steps=10)
    We, be = W.clone(), b.clone()
    mom, mu, nu = torch.zeros_like(W), torch.zeros_like(b), torch.zeros_like(b)
    beta, lr, s = cfg.beta, 0.1, math.sqrt(8) * 0.2
    for t in range(1, 4):
        gW, gb = torch.randn_like(W), torch.randn_like(b)
        opt.step(t - 1, [gW, gb])
        mom = beta * mom + (1 - beta) * gW
        mix = beta * mom / (1 - beta ** (t + 1)) + (1 - beta) * gW / (1 - beta**t)
        We = We * (1 - lr * 0.01) - lr * s * newton_schulz(mix, 5, torch.float32)
        mu = 0.9 * mu + 0.1 * gb
        nu = 0.999 * nu + 0.001 * gb * gb
        mu_hat = 0.9 * mu / (1 - 0.9 ** (t + 1)) + 0.1 * gb / (1 - 0.9**t)
        be = be - lr * mu_hat / ((nu / (1 - 0.999**t)).sqrt() + 1e-8)
        assert torch.allclose(W, We, atol=1e-5), t
        assert torch.allclose(b, be, atol=1e-5), t


SITES = (SiteSpec("s", 4, 4, 8),)


def test_source_shapes():
    assert A.source_lead_shape("c", 5, None) == (1,) and A.source_lead_shape("bc", 5, None) == (5,)
    assert A.source_lead_shape("c", 5, 7) == (1, 1) and A.source_lead_shape("bc", 5, 7) == (5, 1)
    assert A.source_lead_shape("bsc", 5, 7) == (5, 7)


def test_adam_ascent_and_clip():
    cfg = AdamPGDConfig(beta1=0.5, beta2=0.99, eps=1e-8, lr_schedule=0.1)
    adv = A.PersistentAdversary.init(SITES, cfg, "float32", "bc", 3, None, StepKey(0, 0))
    s0 = adv.sources["s"].clone()
    g = torch.ones_like(s0)
    adv.ascend({"s": g, "d:s": torch.zeros(3, 1)}, lr=0.1)
    # first Adam step moves by lr * g/|g| = +0.1, clipped to [0, 1]
    assert torch.allclose(adv.sources["s"], (s0 + 0.1).clamp(0, 1), atol=1e-5)
    assert adv.n_updates == 1 and "s/mu" in adv.state
    sd = adv.state_dict()
    adv2 = A.PersistentAdversary(optimizer=cfg, source_dtype="float32")
    adv2.load_state_dict(sd)
    adv.ascend({"s": g, "d:s": torch.zeros(3, 1)}, lr=0.1)
    adv2.ascend({"s": g, "d:s": torch.zeros(3, 1)}, lr=0.1)
    assert torch.equal(adv.sources["s"], adv2.sources["s"])  # bias correction survives a resume


def test_sgd_and_momentum_ascent():
    adv = A.PersistentAdversary.init(SITES, SgdPGDConfig(lr_schedule=0.1), "float32", "c", 3, None, StepKey(0, 0))
    s0 = adv.sources["s"].clone()
    adv.ascend({"s": -torch.ones_like(s0), "d:s": torch.zeros(1, 1)}, lr=0.25)
    assert torch.allclose(adv.sources["s"], (s0 - 0.25).clamp(0, 1))
    m = A.PersistentAdversary.init(SITES, MomentumSgdPGDConfig(momentum=0.5, lr_schedule=0.1), "bfloat16", "c", 3, None, StepKey(0, 0))
    for _ in range(2):
        m.ascend({"s": torch.full((1, 8), 0.1), "d:s": torch.zeros(1, 1)}, lr=0.1)
    assert m.state["s/vel"].dtype == torch.bfloat16
    assert torch.allclose(m.state["s/vel"].float(), torch.full((1, 8), 0.15), atol=2e-3)


def test_uint16_storage_is_unbiased():
    v = torch.full((1, 4096), 0.5 + 0.3 / 65535)
    enc = A.encode_sources(v, "uint16", StepKey(0, 1), 7)
    assert enc.dtype == torch.uint16
    dec = A.decode_sources(enc)
    assert abs(float(dec.mean()) - float(v.mean())) < 2e-7 * 20  # stochastic rounding keeps the mean
    assert set(torch.unique(enc.to(torch.int32)).tolist()) <= {32767, 32768}


def test_sign_ascent_clips():
    leaves = {"s": torch.tensor([[0.95, 0.05]])}
    A.sign_ascent_(leaves, {"s": torch.tensor([[3.0, -2.0]])}, 0.1)
    assert torch.allclose(leaves["s"], torch.tensor([[1.0, 0.0]]))
