"""The rank-count invariance tool, and the property it caught: fresh per-row adversary sources are drawn at their
global rows, so two ranks together hold exactly the rows one process would."""
import torch

from param_decomp_b200.core import adversary as adv
from param_decomp_b200.core.components import SiteSpec
from param_decomp_b200.core.rng import StepKey
from param_decomp_b200.experiments.lm import invariance_check as ic


def test_fresh_per_row_sources_tile_the_global_batch():
    sites = (SiteSpec("a", 8, 8, 16), SiteSpec("b", 8, 8, 24))
    key = StepKey(7, 3)
    for shape, positions in (("bc", None), ("bsc", 5)):
        whole = adv.fresh_sources(sites, "random", shape, 6, positions, key, 2, "cpu")
        rows = adv.fresh_source_rows(shape, 3, positions)
        halves = [adv.fresh_sources(sites, "random", shape, 3, positions, key, 2, "cpu", row_offset=r * rows)
                  for r in range(2)]
        for k in whole:
            assert torch.equal(torch.cat([h[k] for h in halves]), whole[k]), (shape, k)
        assert not torch.equal(halves[0]["a"], halves[1]["a"])
    shared = [adv.fresh_sources(sites, "random", "c", 3, None, key, 2, "cpu", row_offset=r * 3) for r in range(2)]
    assert torch.equal(shared[0]["a"], shared[1]["a"]), "batch-shared sources are one draw for every rank"


def test_two_ranks_follow_the_one_process_trajectory():
    assert ic.check(world=2, steps=2, sharding="zero1", batch=4, device="cpu", verbose=False) == []


def test_compare_reports_what_differs():
    one = {0: {"train/loss/total": 1.0, "train/perf/step_ms": 5.0, "train/grad_norm/ci_fn": 1.0}}
    many = {0: {"train/loss/total": 1.001, "train/perf/step_ms": 9.0, "train/grad_norm/ci_fn": 1.0005}}
    bad = ic.compare(one, many, rtol=1e-4, atol=0.0)
    assert len(bad) == 1 and "loss/total" in bad[0]


def test_full_width_sources_are_read_at_the_selected_blocks():
    """Expert-blocked sites have narrow importances `[.., k * c]`; an adversary source is full width `[.., E * c]`.
    The mask must pair every slot with the source values of ITS block, for every source shape."""
    from param_decomp_b200.core import masking
    from param_decomp_b200.core.ci_fn.interface import MaskInputs
    from param_decomp_b200.core.components import BlockSelection, SelectedCI

    torch.manual_seed(0)
    B, T, E, c, k = 3, 4, 5, 2, 2
    idx = torch.stack([torch.randperm(E)[:k] for _ in range(B * T)]).reshape(B, T, k)
    narrow = torch.rand(B, T, k * c)
    dense_ci = SelectedCI(narrow, BlockSelection(idx, torch.ones(B, T, k)), E).scatter_dense()
    for shape in ((1, E * c), (B, 1, E * c), (B, T, E * c)):
        src = torch.rand(*shape, requires_grad=True)
        got = masking.select_source_blocks(src, idx, E)
        want = torch.gather(src.expand(B, T, E * c).reshape(B, T, E, c), 2,
                            idx[..., None].expand(B, T, k, c)).reshape(B, T, k * c)
        assert torch.equal(got, want), shape
        m = masking.source_masks(MaskInputs({"x": narrow}, {"x": (idx, E)}), {"x": src}, None)["x"].mask
        dense_m = dense_ci + (1 - dense_ci) * src.expand(B, T, E * c)
        picked_dense = torch.gather(dense_m.reshape(B, T, E, c), 2, idx[..., None].expand(B, T, k, c)).reshape(B, T, k * c)
        assert torch.allclose(m, picked_dense, atol=1e-6), shape
        (g,) = torch.autograd.grad(got.sum(), src)
        counts = torch.zeros(E).index_add_(0, idx.reshape(-1), torch.ones(idx.numel()))
        if shape[0] == 1:  # a batch-shared source collects one unit of gradient per (position, slot) of a block
            assert torch.equal(g.reshape(E, c)[:, 0], counts)


def test_adversaries_on_a_mixture_of_experts_are_rank_count_invariant():
    """Persistent and fresh adversaries on expert-blocked sites (narrow importances), one process against two ranks
    that split the experts and exchange token jobs."""
    assert ic.check(world=2, steps=2, sharding="ddp", batch=4, device="cpu", verbose=False, tp=2, family="moe",
                    expert_mode="all_to_all") == []


def test_evaluation_metrics_do_not_depend_on_the_rank_count():
    """CE / KL under the six mask variants (stochastic draws keyed on global rows), the CE-unrecovered fraction
    (a ratio, formed from the averaged values), CI statistics and the fresh-PGD probe: one process against two."""
    assert ic.check(world=2, steps=2, sharding="ddp", batch=4, device="cpu", verbose=False, with_eval=True) == []


def test_ce_unrecovered_is_formed_from_averages():
    from param_decomp_b200.evals.lm import ce_unrecovered

    a = {"ce/target": 1.0, "ce/zero_masked": 3.0, "ce/ci_masked": 2.0}
    b = {"ce/target": 1.0, "ce/zero_masked": 2.0, "ce/ci_masked": 2.0}
    mean = {k: (a[k] + b[k]) / 2 for k in a}
    assert ce_unrecovered(mean)["ce_unrecovered/ci_masked"] == (2.0 - 1.0) / (2.5 - 1.0)  # not (0.5 + 1.0) / 2
    assert ce_unrecovered({"kl/x": 1.0}) == {}


def test_muon_orthogonalises_whole_matrices_when_the_component_axis_is_split():
    """Two ranks that each hold half of every site's components must take the step one process takes: the
    Newton-Schulz factor of a slice is not the slice of the factor, and the clip norm covers both halves."""
    assert ic.check(world=2, steps=2, sharding="ddp", batch=4, device="cpu", verbose=False, tp=2, muon=True,
                    with_noise_floor=True) == []
