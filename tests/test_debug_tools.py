"""Census, memory ledger and the deviceless fit check."""
import torch
import torch.distributed as dist

from param_decomp_b200.config.experiments import LMExperimentConfig
from param_decomp_b200.core.debug import fit_check, memory_ledger
from param_decomp_b200.core.debug.census import census


def test_fit_check_orders_configs():
    cfg = LMExperimentConfig.from_file("param_decomp_b200/experiments/configs/lm_llama4l_c4096.yaml")
    one, eight = fit_check.estimate(cfg, 1), fit_check.estimate(cfg, 8)
    assert one.fits and eight.total_gib < one.total_gib
    assert not fit_check.estimate(cfg, 1, pool_gib=10.0).fits
    moe = LMExperimentConfig.from_file("param_decomp_b200/experiments/configs/lm_moe4l_e42.yaml")
    assert not fit_check.estimate(moe, 1).fits and fit_check.estimate(moe, 8).fits
    # the 8B-shaped config: its fsdp 4 x tp 2 mesh (components split over tp, optimizer state over the batch shards)
    # fits eight 180 GB parts; the same eight GPUs as pure data parallel (tp = 1) would not
    big = LMExperimentConfig.from_file("param_decomp_b200/experiments/configs/lm_llama8b_mlp_c8192.yaml")
    assert big.runtime.mesh.tp == 2 and fit_check.estimate(big, 8).fits
    flat = big.model_copy(update={"runtime": big.runtime.model_copy(update={"mesh": big.runtime.mesh.model_copy(
        update={"fsdp": 8, "tp": 1})})})
    assert not fit_check.estimate(flat, 8).fits
    assert "TOTAL" in str(one)


def test_memory_ledger_roundtrip(tmp_path):
    led = memory_ledger.Ledger(top_n=3)
    keep = torch.zeros(1000, 100)
    led.mark("after_alloc")
    led.mark("end")
    led.save(tmp_path / "a.json")
    other = memory_ledger.Ledger.load(tmp_path / "a.json")
    assert [m.name for m in other.marks] == ["after_alloc", "end"]
    assert memory_ledger.diff(led, other) == [("after_alloc", 0), ("end", 0)]
    assert "peak" in led.report() and keep.numel() == 100000


def test_census_counts_collectives(monkeypatch):
    calls = []
    monkeypatch.setattr(dist, "all_reduce", lambda t, *a, **k: calls.append(t.numel()))
    with census() as c:
        dist.all_reduce(torch.zeros(10))
        dist.all_reduce(torch.zeros(6))
    assert c.collectives["all_reduce"] == 2 and c.collective_bytes["all_reduce"] == 64 and calls == [10, 6]
    c.assert_collectives({"all_reduce"})
    try:
        c.assert_collectives({"reduce_scatter_tensor"})
        raise RuntimeError("should have refused")
    except AssertionError:
        pass


def test_ledger_diff_groups_created_destroyed_resized(tmp_path):
    from param_decomp_b200.core.debug import ledger_diff
    from param_decomp_b200.core.debug.memory_ledger import Ledger, Mark

    a = Ledger(marks=[Mark("step", 100, 200, 150, [("(4, 4) float32", 64), ("(8,) float32", 32), ("(8,) float32", 32)]),
                      Mark("only_a", 1, 1, 1, [])])
    b = Ledger(marks=[Mark("step", 300, 200, 400, [("(4, 4) float32", 64), ("(8,) float32", 32), ("(16, 16) bfloat16", 512)])])
    a.save(tmp_path / "a.json"), b.save(tmp_path / "b.json")
    (d,) = ledger_diff.diff_ledgers(Ledger.load(tmp_path / "a.json"), Ledger.load(tmp_path / "b.json"))
    assert d.mark == "step" and d.allocated == (100, 300) and d.peak == (150, 400)
    assert [g.key for g in d.created] == ["(16, 16) bfloat16"] and d.created[0].delta_bytes == 512
    assert not d.destroyed and [g.key for g in d.resized] == ["(8,) float32"] and d.resized[0].delta_bytes == -32
    (p,) = ledger_diff.diff_ledgers(a, b, peak_only=True)
    assert p.mark.startswith("peak (step -> step)")
    text = ledger_diff.render([d])
    assert "created" in text and "resized" in text and "+0.0 MiB" in text

