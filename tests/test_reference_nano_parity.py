"""Numerical parity with the reference's single-file PyTorch implementation, run unmodified as the oracle.

The file is read from the offline install of the reference (`baseline/_ref/nano_param_decomp/run.py`, not part of
this repository's history); without it these tests are skipped. Each test feeds the same tensors to one of its
functions and to this package's statement of the same quantity.
"""
import importlib.util
import math
import sys
import types
from pathlib import Path

import pytest
import torch

NANO = Path(__file__).resolve().parents[1] / "baseline" / "_ref" / "nano_param_decomp" / "run.py"
pytestmark = pytest.mark.skipif(not NANO.exists(), reason="the reference is not installed under baseline/_ref")


@pytest.fixture(scope="module")
def ref():
    for name in ("matplotlib", "matplotlib.pyplot"):  # imported at the top of the file, used by its figures only
        if name not in sys.modules:
            try:
                __import__(name)
            except ModuleNotFoundError:
                sys.modules[name] = types.ModuleType(name)
    if not hasattr(sys.modules["matplotlib"], "pyplot"):
        sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]
    spec = importlib.util.spec_from_file_location("nano_reference_oracle", NANO)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["nano_reference_oracle"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_leaky_hard_sigmoids_values_and_gradients(ref):
    from param_decomp_b200.core.squashing import lower_leaky_hard_sigmoid, upper_leaky_hard_sigmoid

    torch.manual_seed(0)
    x = torch.cat([torch.randn(400) * 1.5, torch.tensor([0.0, 1.0, -1e-9, 1 + 1e-6])])
    g = torch.randn_like(x)
    for ours, theirs in ((lower_leaky_hard_sigmoid, ref.lower_leaky), (upper_leaky_hard_sigmoid, ref.upper_leaky)):
        a, b = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        ya, yb = ours(a, 0.01), theirs(b, 0.01)
        assert torch.equal(ya, yb)
        ya.backward(g)
        yb.backward(g)
        assert torch.equal(a.grad, b.grad)


def test_masked_component_linear_with_delta_and_routing(ref):
    """`((x V) * m) U + d * x (W - V U)^T`, routed against the target output per position: the reference forms the
    weight delta, this package folds it into the coefficients `m - d` and adds `d * x W^T`."""
    from param_decomp_b200.core.decomposed_linear import site_forward
    from param_decomp_b200.core.masking import SiteMask

    torch.manual_seed(1)
    lin = torch.nn.Linear(12, 9, bias=True).double()
    comp = ref.ComponentLinear(lin, 20).double()
    x = torch.randn(3, 5, 12, dtype=torch.float64)
    comp.mode = "component"
    comp.mask = torch.rand(3, 5, 20, dtype=torch.float64)
    comp.delta_mask = torch.rand(3, 5, dtype=torch.float64)
    for routing in (None, torch.rand(3, 5) < 0.5):
        comp.routing_mask = routing
        want = comp(x)
        got = site_forward(x, comp.V, comp.U, comp.W_target,
                           SiteMask(mask=comp.mask, delta=comp.delta_mask.unsqueeze(-1), route=routing), bias=comp.bias)
        assert torch.allclose(got, want, atol=1e-12)


def test_losses(ref):
    from param_decomp_b200.core import losses
    from param_decomp_b200.core.components import ComponentStacks, SiteSpec

    torch.manual_seed(2)
    ci = {"a": torch.rand(4, 6, 10) * 1.2, "b": torch.rand(4, 6, 7)}
    for p, beta in ((2.0, 0.0), (0.9, 0.5), (0.4, 0.5)):
        want = ref.importance_minimality_loss(ci, p, 1e-12, beta, world_size=1)
        assert torch.allclose(losses.lp_importance_minimality(ci, p, 1e-12, beta), want, rtol=1e-6)
    for step in (0, 37, 100):
        assert losses.anneal_linear(2.0, 0.4, min(step / 100, 1.0)) == pytest.approx(ref.anneal_p(step, 100, 2.0, 0.4))

    pred, target = torch.randn(3, 5, 31), torch.randn(3, 5, 31)
    assert torch.allclose(losses.kl_from_logits(target, pred), ref.kl_logits(pred, target), atol=1e-6)

    # the paper form of faithfulness: sum of squared weight deltas over their element count
    wrappers = {"s0": ref.ComponentLinear(torch.nn.Linear(8, 6, bias=False), 5),
                "s1": ref.ComponentLinear(torch.nn.Linear(6, 8, bias=False), 7)}
    stacks = ComponentStacks((SiteSpec("s0", 8, 6, 5), SiteSpec("s1", 6, 8, 7)))
    for n, w in wrappers.items():
        stacks.set_site(n, w.V.detach(), w.U.detach())
    ours = losses.faithfulness_loss(stacks, {n: w.W_target for n, w in wrappers.items()}, relative=False)
    assert torch.allclose(ours, ref.faithfulness_loss(wrappers), rtol=1e-6)


def test_persistent_adversary_adam_ascent(ref):
    """Sources in [0, 1] ascended by bias-corrected Adam and clipped: same update rule, three steps."""
    from param_decomp_b200.config.losses import AdamPGDConfig
    from param_decomp_b200.core.adversary import PersistentAdversary, decode_sources, encode_sources

    torch.manual_seed(3)
    cfg = types.SimpleNamespace(ppgd_beta1=0.5, ppgd_beta2=0.99, ppgd_eps=1e-8)
    theirs = ref.PersistentPGD.__new__(ref.PersistentPGD)
    theirs.cfg, theirs.t = cfg, 0
    start = torch.rand(2, 3, 6)
    theirs.sources = {"s": start.clone()}
    theirs.m = {"s": torch.zeros_like(start)}
    theirs.v = {"s": torch.zeros_like(start)}

    ours = PersistentAdversary(optimizer=AdamPGDConfig(beta1=0.5, beta2=0.99, eps=1e-8, lr_schedule=0.01),
                               source_dtype="float32", pool_size=1, batch_shared=False)
    ours.sources = {"s": encode_sources(start[..., :5].clone(), "float32")}
    ours.delta = {"s": encode_sources(start[..., 5:].clone(), "float32")}
    for _ in range(3):
        g = torch.randn(2, 3, 6) * 10
        theirs._adam_step({"s": g}, lr=0.01)
        ours.ascend({"s": g[..., :5], "d:s": g[..., 5:]}, 0.01)
    got = torch.cat([decode_sources(ours.sources["s"]), decode_sources(ours.delta["s"])], dim=-1)
    assert torch.allclose(got, theirs.sources["s"], atol=1e-6)


def test_stochastic_masks_have_the_reference_form(ref):
    """`m = ci + (1 - ci) u`, one delta scalar per position: the draw differs (counter-based here), the form does not."""
    from param_decomp_b200.core import masking
    from param_decomp_b200.core.rng import StepKey

    ci = {"s": torch.rand(2, 4, 8)}
    torch.manual_seed(4)
    masks, deltas = ref.sample_continuous_masks(ci)
    ours = masking.stochastic_masks(ci, StepKey(0, 0), 0, 0, site_index={"s": 0}, lazy=False)["s"]
    for m, d in ((masks["s"], deltas["s"]), (ours.mask, ours.delta.squeeze(-1))):
        assert m.shape == (2, 4, 8) and d.shape == (2, 4)
        assert bool((m >= ci["s"]).all()) and bool((m <= 1).all()) and bool((d >= 0).all()) and bool((d <= 1).all())
    routes = ref.sample_uniform_k_subset_routing(["a", "b", "c"], (64, 16), torch.device("cpu"))
    k = torch.stack(list(routes.values())).sum(0)
    assert int(k.min()) >= 1 and int(k.max()) <= 3 and abs(float(k.float().mean()) - 2.0) < 0.15
    mine = masking.sample_routing("uniform_k_subset", None, ["a", "b", "c"], (64, 16), StepKey(1, 0), 0, 0, 0, "cpu")
    k2 = torch.stack([mine[n] for n in ("a", "b", "c")]).sum(0)
    assert int(k2.min()) >= 1 and int(k2.max()) <= 3 and abs(float(k2.float().mean()) - 2.0) < 0.15
    assert math.isclose(float(k2.float().var()), float(k.float().var()), abs_tol=0.15)
