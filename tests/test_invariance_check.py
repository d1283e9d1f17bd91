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
