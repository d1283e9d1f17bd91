import copy

import pytest
import torch

import __graft_entry__ as ge
from param_decomp_b200.config.experiments import LMExperimentConfig
from param_decomp_b200.core.components import BlockSelection
from param_decomp_b200.experiments.lm.build import build_lm_run
from param_decomp_b200.models import moe
from param_decomp_b200.models.transformer import LMBatch


def moe_cfg(**arch_over) -> LMExperimentConfig:
    c = copy.deepcopy(ge.SMOKE_CONFIG)
    c["runtime"]["backend"] = "eager_torch"
    c["target"]["weights_dtype"] = "float32"
    c["target"]["attention_implementation"] = "xla"
    c["target"]["spec"]["arch"] = {"family": "moe", "n_layer": 2, "d_model": 32, "n_head": 2, "d_ff": 16,
                                   "vocab_size": 100, "n_experts": 6, "experts_per_token": 2, **arch_over}
    c["decomposition"]["sites"] = {"kind": "moe", "layers": {"kind": "all"},
                                   "cs": {"q": 8, "experts_gate": 24, "experts_up": 24, "experts_down": 24}}
    c["decomposition"]["ci"] = {"type": "layerwise_mlp", "hidden_dims": [16]}
    c["data"]["seq_len"] = 8
    c["pd"]["batch_size"] = 3
    return LMExperimentConfig.model_validate(c)


def test_router_topk_renormalises():
    logits = torch.tensor([[0.0, 1.0, 2.0, 3.0]])
    sel = moe.route_topk(logits, 2, True)
    assert sel.indices.tolist() == [[3, 2]] and float(sel.weights.sum()) == pytest.approx(1.0)
    raw = moe.route_topk(logits, 2, False)
    assert float(raw.weights.sum()) == pytest.approx(float(torch.softmax(logits, -1)[0, 2:].sum()))


def test_routed_forward_matches_dense_oracle_with_empty_experts():
    cfg = moe_cfg()
    run = build_lm_run(cfg, None, "cpu")
    m = run.model
    x = torch.randn(1, 5, 32)
    # force a routing that leaves experts 4 and 5 empty
    sel = BlockSelection(torch.tensor([[[0, 1], [1, 2], [3, 0], [2, 3], [0, 2]]]), torch.rand(1, 5, 2))
    aux = {"pinned_routing": {0: sel}}
    y = m._mlp(0, x, None, None, None, None, aux)
    W = m.w
    ref = moe.dense_moe_oracle(x.reshape(5, 32), BlockSelection(sel.indices[0], sel.weights[0]),
                               W["layers.0.mlp.experts_gate.weight"], W["layers.0.mlp.experts_up.weight"],
                               W["layers.0.mlp.experts_down.weight"])
    assert torch.allclose(y.reshape(5, 32), ref, atol=1e-5)


def test_unmasked_with_delta_reproduces_target_and_step_trains():
    from param_decomp_b200.core import masking
    from param_decomp_b200.core.components import prepare_compute_weights
    from param_decomp_b200.core.objective import build_objective
    from param_decomp_b200.core.run import init_train_state
    from param_decomp_b200.core.train import StepContext, run_ci_fn, train_step

    cfg = moe_cfg()
    run = build_lm_run(cfg, None, "cpu")
    obj = build_objective(cfg.pd)
    ctx = StepContext.build(run.model, obj, cfg.pd)
    st = init_train_state(run.model, run.ci_fn, cfg.pd, obj, "cpu", 3, 8)
    batch = run.sample_train(0)
    with torch.no_grad():
        clean = run.model.clean_forward(batch)
        ci = run_ci_fn(ctx, st, clean)
        assert ci.lower["layers.0.mlp.experts_gate"].values.shape == (3, 8, 2 * 4)  # narrow: k * C_block
        w = prepare_compute_weights(st.components, torch.float32)
        out = run.model.masked_forward(w, batch, masking.unmasked(ci.mask_inputs()), clean=clean)
        assert torch.allclose(out.output, clean.output, atol=1e-4)
        assert float(run.model.recon_loss(clean, out)) < 1e-6
    m = train_step(ctx, st, batch)
    assert torch.isfinite(m["loss/total"]) and float(m["loss/StochasticReconLoss"]) > 0
    g = st.components.V["experts_gate"].grad
    assert g is not None and float(g.abs().sum()) > 0


def test_moe_chunkwise_ci_fn_steps_and_routed_products_match_gathers():
    """The block-selected (expert-routed) chunkwise CI transformer: one engine step trains it, it emits narrow
    `SelectedCI` for expert sites, and its routed products equal the per-token weight-gather formula they replace."""
    from param_decomp_b200.core.ci_fn.transformer import MoEChunkwiseTransformerCIFn, routed_linear
    from param_decomp_b200.core.components import SelectedCI
    from param_decomp_b200.core.objective import build_objective
    from param_decomp_b200.core.run import init_train_state
    from param_decomp_b200.core.train import StepContext, run_ci_fn, train_step

    torch.manual_seed(0)
    sel = BlockSelection(torch.tensor([[[0, 1], [1, 2], [3, 0], [2, 3], [0, 2]]]), torch.rand(1, 5, 2))
    x, W = torch.randn(1, 5, 8), torch.randn(6, 8, 4)  # experts 4 and 5 receive no job
    got = routed_linear(x.reshape(5, 8), W, sel, per_job=False, fused=False).reshape(1, 5, 2, 4)
    ref = (x.unsqueeze(-2).unsqueeze(-2) @ W[sel.indices]).squeeze(-2)
    assert torch.allclose(got, ref, atol=1e-6)
    jobs = torch.randn(10, 8)
    got = routed_linear(jobs, W, sel, per_job=True, fused=False).reshape(1, 5, 2, 4)
    ref = (jobs.reshape(1, 5, 2, 1, 8) @ W[sel.indices]).squeeze(-2)
    assert torch.allclose(got, ref, atol=1e-6)

    c = moe_cfg().model_dump(mode="json")
    c["decomposition"]["ci"] = {
        "type": "moe_chunkwise_transformer", "d_model": 16, "n_blocks": 1, "blocks_per_chunk": 1,
        "attention": {"kind": "mha", "n_heads": 2, "implementation": "xla", "mask": "causal"},
        "expert_ffn_hidden": 8, "shared_ffn_hidden": 16,
        "expert_implementation": "ragged_dot", "input_tap": "all_block_taps"}
    cfg = LMExperimentConfig.model_validate(c)
    run = build_lm_run(cfg, None, "cpu")
    assert isinstance(run.ci_fn, MoEChunkwiseTransformerCIFn)
    obj = build_objective(cfg.pd)
    ctx = StepContext.build(run.model, obj, cfg.pd)
    st = init_train_state(run.model, run.ci_fn, cfg.pd, obj, "cpu", 3, 8)
    batch = run.sample_train(0)
    with torch.no_grad():
        ci = run_ci_fn(ctx, st, run.model.clean_forward(batch))
    narrow = ci.lower["layers.0.mlp.experts_gate"]
    assert isinstance(narrow, SelectedCI) and narrow.values.shape == (3, 8, 2 * 4)
    assert ci.lower["layers.0.self_attn.q_proj"].shape == (3, 8, 8)
    before = [p.detach().clone() for p in run.ci_fn.parameters()]
    m = train_step(ctx, st, batch)
    assert torch.isfinite(m["loss/total"])
    assert sum(int(not torch.equal(a, b)) for a, b in zip(before, run.ci_fn.parameters())) > len(before) // 2


def test_router_logits_are_captured_in_clean_and_masked_passes():
    """The quantity a router-KL auxiliary compares: what the router would decide on each pass's own residual
    stream, although masked passes keep the clean pass's expert choice."""
    from param_decomp_b200.core import masking
    from param_decomp_b200.core.components import prepare_compute_weights
    from param_decomp_b200.core.objective import build_objective
    from param_decomp_b200.core.run import init_train_state
    from param_decomp_b200.core.train import StepContext, run_ci_fn

    cfg = moe_cfg()
    run = build_lm_run(cfg, None, "cpu")
    obj = build_objective(cfg.pd)
    ctx = StepContext.build(run.model, obj, cfg.pd)
    st = init_train_state(run.model, run.ci_fn, cfg.pd, obj, "cpu", 3, 8)
    batch = run.sample_train(0)
    keys = ("router_logits.0", "router_logits.1")
    with torch.no_grad():
        clean = run.model.clean_forward(batch, capture=keys)
        assert clean.captures["router_logits.1"].shape == (3, 8, 6)
        ci = run_ci_fn(ctx, st, clean)
        w = prepare_compute_weights(st.components, torch.float32)
        same = run.model.masked_forward(w, batch, masking.unmasked(ci.mask_inputs()), capture=keys, clean=clean)
        assert torch.allclose(same.captures["router_logits.1"], clean.captures["router_logits.1"], atol=1e-4)
        zero = run.model.masked_forward(w, batch, masking.constant_masks(ci.mask_inputs(), 0.0, None), capture=keys,
                                        clean=clean)
        assert not torch.allclose(zero.captures["router_logits.1"], clean.captures["router_logits.1"], atol=1e-4)


def test_adversary_sources_act_only_on_the_selected_expert_blocks():
    """A per-position full-width source at an expert site influences the output only through the blocks of the
    experts that position was routed to: its gradient is zero everywhere else."""
    from param_decomp_b200.core import masking
    from param_decomp_b200.core.components import prepare_compute_weights
    from param_decomp_b200.core.objective import build_objective
    from param_decomp_b200.core.run import init_train_state
    from param_decomp_b200.core.train import StepContext, run_ci_fn

    cfg = moe_cfg()
    run = build_lm_run(cfg, None, "cpu")
    obj = build_objective(cfg.pd)
    ctx = StepContext.build(run.model, obj, cfg.pd)
    st = init_train_state(run.model, run.ci_fn, cfg.pd, obj, "cpu", 3, 8)
    batch = run.sample_train(0)
    with torch.no_grad():
        clean = run.model.clean_forward(batch)
        ci = run_ci_fn(ctx, st, clean)
        w = prepare_compute_weights(st.components, torch.float32)
    inputs = ci.mask_inputs().map(lambda v: v * 0.5)
    site = "layers.0.mlp.experts_up"
    sources = {n: torch.rand(3, 8, s.C, requires_grad=True) for n, s in ((s.name, s) for s in run.model.sites)}
    out = run.model.masked_forward(w, batch, masking.source_masks(inputs, sources, None), clean=clean)
    (g,) = torch.autograd.grad(run.model.recon_loss(clean, out), sources[site])
    idx, E = inputs.selections[site]
    c = g.shape[-1] // E
    chosen = torch.zeros(3, 8, E, dtype=torch.bool).scatter_(-1, idx, True)
    per_block = g.reshape(3, 8, E, c).abs().sum(-1)
    assert float(per_block[~chosen].sum()) == 0.0
    assert bool((per_block[chosen] > 0).all())


def test_locality_loss_is_job_wide_when_experts_are_split():
    """A unit kind's mean runs over every component of the job. With the expert blocks dealt to two ranks (and a
    padding expert on the second) each rank must report the one-process value, and give its own blocks the
    one-process gradient."""
    from types import SimpleNamespace

    from param_decomp_b200.core import losses
    from param_decomp_b200.core.components import ComponentStacks, SiteSpec
    from param_decomp_b200.formats.nonlinearity import Neurons, NonlinearityAlignment

    al = NonlinearityAlignment(side="output", partition=Neurons())
    E, e_loc, c = 3, 2, 2  # three experts on two ranks: rank 1 holds one real expert and one padding expert

    def stacks(n_blocks: int) -> ComponentStacks:
        return ComponentStacks((SiteSpec("shared_up", 6, 8, 4, alignment=al),
                                SiteSpec("experts_up", 6, 8, n_blocks * c, n_blocks=n_blocks, alignment=al, routed=True)))

    torch.manual_seed(0)
    whole = stacks(E)
    whole.init_random()
    coeffs = {"neuron": 2.0}
    ref = losses.nonlinearity_locality(whole, 4.0, coeffs, True)
    ref.backward()
    key = ComponentStacks.param_key(whole.site_by_name["experts_up"].group)

    parts = []
    for r in range(2):
        st = stacks(e_loc)
        with torch.no_grad():
            for name in ("V", "U"):
                getattr(st, name)[ComponentStacks.param_key(st.site_by_name["shared_up"].group)].copy_(
                    getattr(whole, name)[ComponentStacks.param_key(whole.site_by_name["shared_up"].group)])
                src = getattr(whole, name)[key][:, r * e_loc:(r + 1) * e_loc]
                getattr(st, name)[ComponentStacks.param_key(st.site_by_name["experts_up"].group)][:, :src.shape[1]].copy_(src)
        parts.append(st)
    sent: dict[int, torch.Tensor] = {}
    for second_pass in (False, True):  # first pass records what each rank would send, second adds the peer's
        for r, st in enumerate(parts):
            def add(t, r=r):
                if not second_pass:
                    sent[r] = t.clone()
                    return t
                return t + sent[1 - r]
            shard = SimpleNamespace(by_component=False, n_real=min(E, (r + 1) * e_loc) - r * e_loc, sum_over_group=add)
            st.zero_grad()
            val = losses.nonlinearity_locality(st, 4.0, coeffs, True, expert_shard=shard)
            if second_pass:
                assert torch.allclose(val, ref, atol=1e-6), (r, float(val), float(ref))
                val.backward()
                k2 = ComponentStacks.param_key(st.site_by_name["experts_up"].group)
                n = shard.n_real
                assert torch.allclose(st.U[k2].grad[:, :n], whole.U[key].grad[:, r * e_loc:r * e_loc + n], atol=1e-7)
                assert float(st.U[k2].grad[:, n:].abs().sum()) == 0.0  # the padding expert is not a component
                ks = ComponentStacks.param_key(st.site_by_name["shared_up"].group)
                assert torch.allclose(st.U[ks].grad, whole.U[ComponentStacks.param_key(whole.site_by_name["shared_up"].group)].grad, atol=1e-7)
