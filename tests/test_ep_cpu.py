"""Expert parallelism on gloo ranks against the single-process model (host-side logic of the
dispatch / combine, variable counts, padded dummy experts, both EP modes)."""
import copy
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as ge
from param_decomp_b200.config.experiments import LMExperimentConfig, TransformerArchConfig
from param_decomp_b200.core import masking
from param_decomp_b200.core.components import ComponentStacks, prepare_compute_weights
from param_decomp_b200.core.rng import StepKey
from param_decomp_b200.models import moe
from param_decomp_b200.models.transformer import LMBatch

ARCH = TransformerArchConfig(family="moe", n_layer=1, d_model=16, n_head=2, d_ff=8, vocab_size=50, n_experts=5,
                             experts_per_token=2)
C_PER_EXPERT = 4
B, T = 4, 6


from param_decomp_b200.config.experiments import MoeCSpec

_Sites = MoeCSpec(layers={"kind": "all"}, cs={"experts_gate": 5 * C_PER_EXPERT, "experts_up": 5 * C_PER_EXPERT,
                                              "experts_down": 5 * C_PER_EXPERT})


class _Target:
    attention_implementation = "xla"


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _global_components(model) -> ComponentStacks:
    st = ComponentStacks(model.sites)
    st.init_random(torch.Generator().manual_seed(5))
    return st


def _run(model, stacks, tokens, ci_all, row_offset):
    batch = LMBatch(tokens)
    clean = model.clean_forward(batch)
    lead = tokens.shape
    ci = {s.name: ci_all[s.name][row_offset // T: row_offset // T + lead[0]] for s in model.sites}
    masks = masking.stochastic_masks(ci, StepKey(1, 2), 0, 0, site_index={s.name: i for i, s in enumerate(model.sites)},
                                     row_offset=row_offset, lazy=False)
    w = prepare_compute_weights(stacks, torch.float32)
    out = model.masked_forward(w, batch, masks, clean=clean)
    out.output.pow(2).sum().backward()
    return out.output.detach()


def _reference():
    from param_decomp_b200.config.experiments import select_layers  # noqa: F401

    weights = moe.random_init_moe_weights(ARCH, 0, torch.float32)
    model = moe.build_moe_model(ARCH, weights, _Sites, _Target, "eager_torch")
    stacks = _global_components(model)
    g = torch.Generator().manual_seed(9)
    tokens = torch.randint(0, 50, (B, T), generator=g)
    ci_all = {s.name: torch.rand(B, T, 2 * C_PER_EXPERT, generator=g) for s in model.sites}
    y = _run(model, stacks, tokens, ci_all, 0)
    return model, stacks, tokens, ci_all, y


def _worker(rank: int, world: int, port: int, mode: str, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from param_decomp_b200.parallel.ep import ExpertParallel, local_expert_range

    ref_model, ref_stacks, tokens, ci_all, _ = _reference()
    ep = ExpertParallel(dist.group.WORLD, ARCH.n_experts, mode=mode)
    weights = moe.random_init_moe_weights(ARCH, 0, torch.float32)
    model = moe.build_moe_model(ARCH, weights, _Sites, _Target, "eager_torch", ep=ep)
    stacks = ComponentStacks(model.sites)
    lo, hi = local_expert_range(ARCH.n_experts, rank, world)
    with torch.no_grad():
        for s in model.sites:  # this rank's expert blocks of the reference components (dummies stay zero)
            Vg, Ug = ref_stacks.site(s.name)
            V, U = stacks.site(s.name)
            n = max(0, min(hi, ARCH.n_experts) - lo)
            V[:n].copy_(Vg[lo:lo + n])
            U[:n].copy_(Ug[lo:lo + n])
    if mode == "all_to_all":  # tokens are data-parallel: each rank takes its rows
        rows = B // world
        y = _run(model, stacks, tokens[rank * rows:(rank + 1) * rows], ci_all, rank * rows * T)
    else:  # activation slicing: every rank sees all tokens
        y = _run(model, stacks, tokens, ci_all, 0)
    grads = {s.name: stacks.V[stacks.param_key(s.group)].grad[0].clone() for s in model.sites}
    out[rank] = (y, grads, lo, hi)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["all_to_all", "allreduce"])
def test_expert_parallel_matches_single_process(mode):
    world, port = 2, _free_port()
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, mode, out), nprocs=world, join=True)
    _, ref_stacks, _, _, y_ref = _reference()
    if mode == "all_to_all":
        y = torch.cat([out[r][0] for r in range(world)])
    else:
        y = out[0][0]
        assert torch.allclose(out[1][0], y, atol=1e-5)
    assert torch.allclose(y, y_ref, atol=1e-4)
    for r in range(world):
        _, grads, lo, hi = out[r]
        n = max(0, min(hi, ARCH.n_experts) - lo)
        for name, g in grads.items():
            ref_g = ref_stacks.V[ref_stacks.param_key(name.split(".")[-1])].grad[0][lo:lo + n]
            got = g[:n]
            assert torch.allclose(got, ref_g, atol=1e-4), (name, r)  # exact in both modes
            assert float(g[n:].abs().sum()) == 0.0  # padded dummy experts never receive a job
