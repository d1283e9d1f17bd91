"""Closed-form checks of the pure numerics (squashing, masks, site algebra, losses, RNG)."""
import math

import pytest
import torch

from param_decomp_b200.core import losses, masking
from param_decomp_b200.core.components import ComponentStacks, SelectedCI, BlockSelection, SiteSpec, prepare_compute_weights
from param_decomp_b200.core.decomposed_linear import blocked_site_forward, site_forward
from param_decomp_b200.core.masking import SiteMask, StochasticSpec
from param_decomp_b200.core.rng import StepKey
from param_decomp_b200.core.squashing import lower_leaky_hard_sigmoid, upper_leaky_hard_sigmoid
from param_decomp_b200.ops import philox_ref


def test_lower_leaky_gradient_regions():
    x = torch.tensor([-0.5, -0.5, 0.3, 0.3, 1.5, 1.5], requires_grad=True)
    g = torch.tensor([-2.0, 2.0, -2.0, 2.0, -2.0, 2.0])
    y = lower_leaky_hard_sigmoid(x)
    assert torch.equal(y.detach(), torch.tensor([0, 0, 0.3, 0.3, 1, 1.0]))
    y.backward(g)
    # below 0: leak only when g < 0; inside: pass; above 1: blocked
    assert torch.allclose(x.grad, torch.tensor([-0.02, 0.0, -2.0, 2.0, 0.0, 0.0]))


def test_upper_leaky_values_and_grad():
    x = torch.tensor([-1.0, 0.4, 3.0], requires_grad=True)
    y = upper_leaky_hard_sigmoid(x)
    assert torch.allclose(y.detach(), torch.tensor([0.0, 0.4, 1.02]))
    y.sum().backward()
    assert torch.allclose(x.grad, torch.tensor([0.0, 1.0, 0.01]))


def _site(d_in=6, d_out=5, C=8):
    g = torch.Generator().manual_seed(0)
    V, U = torch.randn(d_in, C, generator=g), torch.randn(C, d_out, generator=g)
    W = torch.randn(d_out, d_in, generator=g)
    x = torch.randn(7, d_in, generator=g)
    return x, V, U, W


def test_site_forward_identities():
    x, V, U, W = _site()
    xw = x @ W.T
    ones_d = torch.ones(7, 1)
    # unmasked + full delta reproduces the target exactly
    assert torch.allclose(site_forward(x, V, U, W, SiteMask(mask=None, delta=ones_d)), xw, atol=1e-5)
    # unmasked, no delta = the full component sum
    assert torch.allclose(site_forward(x, V, U, None, SiteMask()), x @ V @ U, atol=1e-5)
    # general case equals the unfolded form (masked components + d * x (W - (VU)^T)^T)
    m, d = torch.rand(7, 8), torch.rand(7, 1)
    want = ((x @ V) * m) @ U + d * (x @ (W - (V @ U).T).T)
    assert torch.allclose(site_forward(x, V, U, W, SiteMask(mask=m, delta=d)), want, atol=1e-4)
    # unrouted positions fall back to the target
    route = torch.tensor([True, False] * 3 + [True])
    out = site_forward(x, V, U, W, SiteMask(mask=m, delta=d, route=route))
    assert torch.allclose(out[~route], xw[~route], atol=1e-5) and torch.allclose(out[route], want[route], atol=1e-4)


def test_blocked_site_matches_dense_gather():
    g = torch.Generator().manual_seed(1)
    E, d_in, c, d_out, J = 3, 4, 5, 6, 9
    V, U, W = torch.randn(E, d_in, c, generator=g), torch.randn(E, c, d_out, generator=g), torch.randn(E, d_out, d_in, generator=g)
    x, blk = torch.randn(J, d_in, generator=g), torch.randint(0, E, (J,), generator=g)
    m, d = torch.rand(J, c, generator=g), torch.rand(J, 1, generator=g)
    out = blocked_site_forward(x, blk, V, U, W, m, d)
    for j in range(J):
        e = int(blk[j])
        want = site_forward(x[j:j + 1], V[e], U[e], W[e], SiteMask(mask=m[j:j + 1], delta=d[j:j + 1]))
        assert torch.allclose(out[j:j + 1], want, atol=1e-5)


def test_stochastic_mask_is_a_pure_function_of_counters():
    ci = torch.rand(4, 6, 16)
    spec = StochasticSpec(StepKey(3, 11).seed64, StepKey.stream(0, 1, 0, 5))
    a = SiteMask(ci=ci, stochastic=spec).materialize().mask
    b = SiteMask(ci=ci, stochastic=spec).materialize().mask
    assert torch.equal(a, b) and (a >= ci).all() and (a <= 1).all()
    # a rank that owns rows [12, 24) draws the same numbers as the single-process run
    part = SiteMask(ci=ci[2:], stochastic=StochasticSpec(spec.seed64, spec.stream, row_offset=12)).materialize().mask
    assert torch.equal(part, a[2:])


def test_philox_uniform_statistics():
    u = philox_ref.uniform(123, 4, 512, 256)
    assert 0 < float(u.min()) and float(u.max()) < 1
    assert abs(float(u.mean()) - 0.5) < 5e-3 and abs(float(u.var()) - 1 / 12) < 2e-3
    assert abs(float(torch.corrcoef(torch.stack([u[:, :-1].flatten(), u[:, 1:].flatten()]))[0, 1])) < 1e-2


def test_uniform_k_routing_counts():
    key = StepKey(0, 0)
    names = [f"s{i}" for i in range(5)]
    r = masking.sample_routing("uniform_k_subset", None, names, (4000,), key, 0, 0, 0, "cpu")
    k = torch.stack([r[n] for n in names]).sum(0)
    assert int(k.min()) >= 1 and int(k.max()) <= 5
    hist = torch.bincount(k, minlength=6)[1:].float() / 4000
    assert (hist - 0.2).abs().max() < 0.03  # k ~ U{1..S}
    assert masking.sample_routing("all", None, names, (3,), key, 0, 0, 0, "cpu")["s0"] is None


def test_smooth_l0_and_frequency():
    c = torch.tensor([[0.0, 1.0, 0.5]])
    assert torch.allclose(losses.smooth_l0(c, 0.5, False), torch.tensor([[0.0, 0.8, 0.5]]))
    assert torch.allclose(losses.smooth_l0(c, 0.5, True)[0, 1], torch.tensor(1.0))
    f = torch.tensor([0.0, 0.25])
    assert float(losses.frequency_penalty(f, 4)) == pytest.approx(0.25 * math.log2(2.0))
    assert losses.geman_mcclure_max_slope(1.0) == pytest.approx(0.6495, abs=1e-3)


def test_frequency_ema_surrogate_gradient_scale():
    ema = losses.FrequencyEMA(halflife_steps=10.0, value=torch.zeros(3))
    f = torch.tensor([0.1, 0.2, 0.0], requires_grad=True)
    pen = ema.surrogate(f, 100)
    pen.backward()
    smoothed = ema.value / ema.weight
    s = smoothed.clone().requires_grad_(True)
    losses.frequency_penalty(s, 100).backward()
    assert torch.allclose(f.grad, s.grad, atol=1e-6)  # gradient at single-batch scale, taken at the EMA point
    assert torch.allclose(smoothed, f.detach(), atol=1e-6)  # debiased first step equals the batch


def test_lp_minimality_matches_formula():
    ci = {"a": torch.tensor([[0.5, 0.0], [1.0, 0.0]])}
    got = losses.lp_importance_minimality(ci, p=1.0, eps=0.0, beta=0.5, world_size=1)
    mean, s = torch.tensor([0.75, 0.0]), torch.tensor([1.5, 0.0])
    assert float(got) == pytest.approx(float((mean + 0.5 * mean * torch.log2(1 + s)).sum()))


def test_faithfulness_zero_at_exact_factorisation_and_pads_inert():
    sites = (SiteSpec("a", 4, 3, 3, group="g"), SiteSpec("b", 4, 3, 3, group="g"))
    st = ComponentStacks(sites, stack_multiple=4)
    assert st.V["g"].shape[0] == 4 and st.stack_pads["g"] == 2
    st.init_random(torch.Generator().manual_seed(0))
    assert float(st.V["g"][2:].abs().sum()) == 0.0
    W = {s.name: st.weight(s.name).detach().clone() for s in sites}
    assert float(losses.faithfulness_loss(st, W)) < 1e-10
    W["a"] = W["a"] + 1.0
    rel = float(losses.faithfulness_loss(st, W))
    want = 0.5 * 12.0 / float(W["a"].pow(2).sum())
    assert rel == pytest.approx(want, rel=1e-5)


def test_selected_ci_reductions():
    sel = BlockSelection(indices=torch.tensor([[0, 2], [2, 1]]), weights=torch.ones(2, 2))
    s = SelectedCI(values=torch.tensor([[1.0, 2.0, 3.0, 4.0], [5.0, 6.0, 7.0, 8.0]]), selection=sel, n_blocks=3)
    dense = s.scatter_dense()
    assert dense.shape == (2, 6)
    assert torch.equal(dense[0], torch.tensor([1.0, 2, 0, 0, 3, 4])) and torch.equal(dense[1], torch.tensor([0.0, 0, 7, 8, 5, 6]))
    assert torch.equal(s.sum_per_component(), dense.sum(0)) and torch.equal(s.max_per_component(), dense.amax(0))


def test_nonlinearity_locality_prefers_concentrated_components():
    from param_decomp_b200.formats.nonlinearity import Neurons, NonlinearityAlignment

    site = (SiteSpec("w", 4, 8, 2, group="g", alignment=NonlinearityAlignment("output", Neurons())),)
    st = ComponentStacks(site)
    with torch.no_grad():
        st.V["g"].fill_(1.0)
        st.U["g"][0, 0] = torch.tensor([1.0, 0, 0, 0, 0, 0, 0, 0])  # one neuron
        st.U["g"][0, 1] = torch.ones(8)  # all neurons
    v = float(losses.nonlinearity_locality(st, 1.0, {"neuron": 1.0}, False))
    one = 1.0 / (1.0 + (1 / 8) ** 2)
    spread = 8 * ((1 / 8) ** 2 / (2 * (1 / 8) ** 2))
    assert v == pytest.approx((one + spread) / 2, rel=1e-5)


def test_compute_weights_grads_reach_masters():
    sites = (SiteSpec("a", 4, 3, 2, group="g"),)
    st = ComponentStacks(sites)
    st.init_random(torch.Generator().manual_seed(0))
    w = prepare_compute_weights(st, torch.bfloat16)
    V, U = w.site("a")
    (torch.randn(5, 4).to(torch.bfloat16) @ V @ U).float().sum().backward()
    assert st.V["g"].grad is not None and st.V["g"].grad.dtype == torch.float32


def test_host_library_draws_the_reference_stream():
    """The native CPU loop and the pure-torch statement give the same bits for every (seed, stream, row, column),
    including seeds and row offsets that use the top bits."""
    import shutil

    import pytest

    from param_decomp_b200.ops import build, host_native

    if shutil.which("g++") is None and shutil.which("c++") is None:
        pytest.skip("no C++ compiler")
    build.build_host()
    host_native._tried = False  # the library may have been built after the first probe
    assert host_native.available()
    for seed, stream, rows, cols, off in ((123, 4, 17, 24, 0), (2**63 + 5, 2**31 + 3, 100, 8, 2**31 - 50),
                                          (0, 0, 1, 4096, 7), (987654321987, 77, 513, 24, 123456)):
        assert torch.equal(host_native.philox_uniform(seed, stream, rows, cols, off),
                           philox_ref.uniform(seed, stream, rows, cols, off)), (seed, stream)
    from param_decomp_b200.core import rng
    from param_decomp_b200.core.rng import StepKey

    key = StepKey(11, 5)
    u = rng.uniform(key, 9, 33, 20, 4, "cpu")  # a width that is not a multiple of 8 is cut from the padded draw
    assert torch.equal(u, philox_ref.uniform(key.seed64, 9, 33, 24, 4)[:, :20])
    with pytest.raises(ValueError):
        host_native.philox_uniform(1, 1, 4, 12)
