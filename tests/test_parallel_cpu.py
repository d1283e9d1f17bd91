"""Host-side distributed logic on CPU: mesh coordinates, placement resolution, gloo collectives."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from param_decomp_b200.config.run import HsdpMeshShape, ResidentMeshShape
from param_decomp_b200.core.components import SiteSpec
from param_decomp_b200.parallel import placement as pl
from param_decomp_b200.parallel.topology import axis_coords, axis_group_ranks, mesh_axes


def test_mesh_coordinates_tp_fastest():
    axes = mesh_axes(HsdpMeshShape(replicate=2, fsdp=2, tp=2))
    assert axis_coords(0, axes) == {"replicate": 0, "fsdp": 0, "tp": 0}
    assert axis_coords(5, axes) == {"replicate": 1, "fsdp": 0, "tp": 1}
    assert axis_group_ranks(5, axes, ("tp",)) == [4, 5]
    assert axis_group_ranks(5, axes, ("replicate", "fsdp")) == [1, 3, 5, 7]
    assert mesh_axes(ResidentMeshShape(data=4, tp=2)) == [("data", 4), ("tp", 2)]


def test_presets_resolve_and_shard():
    mesh = {"replicate": 1, "fsdp": 4, "tp": 2}
    rules = pl.from_config("owner", mesh)
    assert rules.batch_axes() == ("replicate", "fsdp")
    spec = pl.shard_of((3, 768, 4096), ("stack", "d_in", "C"), rules.components.optimizer_state, mesh,
                       {"replicate": 0, "fsdp": 2, "tp": 1})
    assert spec.slices == [(0, 3), (384, 192), (2048, 2048)]
    z = pl.from_config("zero1", {"replicate": 2, "fsdp": 2, "tp": 2})
    s = pl.shard_of((768, 4096), ("d_in", "C"), z.components.optimizer_state, {"replicate": 2, "fsdp": 2, "tp": 2},
                    {"replicate": 1, "fsdp": 0, "tp": 1})
    assert s.slices == [(0, 384), (3072, 1024)]  # C linearised over (tp, replicate): index 1*2+1 = 3
    assert set(pl.PRESETS) == set(pl.PRESET_NAMES)
    with pytest.raises(AssertionError):
        pl.from_config("zero1-replicated-resident", mesh)  # resident presets need the (data, tp) mesh
    res = pl.from_config("owner-replicated-resident-moe", {"data": 4, "tp": 2})
    assert res.resident and res.expert_blocked and pl.stack_multiple(res, {"data": 4, "tp": 2}) == 4
    assert pl.stack_multiple(pl.from_config("ddp", mesh), mesh) == 1


def test_validate_sites_refuses_untileable():
    mesh = {"replicate": 1, "fsdp": 4, "tp": 1}
    rules = pl.from_config("owner", mesh)
    pl.validate_sites(rules, mesh, [SiteSpec("a", 768, 768, 4096)])
    with pytest.raises(AssertionError):
        pl.validate_sites(rules, mesh, [SiteSpec("a", 770, 768, 4096)])


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from param_decomp_b200.parallel import topology

    topo = topology.initialize(HsdpMeshShape(replicate=1, fsdp=world // 2, tp=2), "cpu", timeout_s=60)
    col = topo.collectives()
    # differentiable mean over the data group
    x = torch.tensor([float(topo.data_rank + 1)], requires_grad=True)
    m = col.mean(x)
    m.backward()
    # grads averaged over the data group only (tp peers hold replicas of the batch)
    p = torch.nn.Parameter(torch.zeros(3))
    p.grad = torch.full((3,), float(topo.data_rank))
    col.reduce_grads([p])
    flag = col.host_any(1.0 if rank == world - 1 else 0.0)
    rid = topo.broadcast_object("p-abc" if rank == 0 else None)
    out[rank] = (float(m), float(x.grad), p.grad.tolist(), flag, rid, topo.tp_rank, topo.data_rank,
                 col.row_offset(10))
    topo.shutdown()


def test_gloo_collectives_world4():
    world, port = 4, _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    for r in range(world):
        mean, gx, g, flag, rid, tp_rank, data_rank, off = out[r]
        # the backward of the mean all-reduces the cotangents: every rank holds dL/dx_r of the SUM over ranks of its loss copies
        assert mean == pytest.approx(1.5) and gx == pytest.approx(1.0)
        assert g == pytest.approx([0.5] * 3)
        assert flag is True and rid == "p-abc"
        assert tp_rank == r % 2 and data_rank == r // 2 and off == 10 * (r // 2)


def _sharded_worker(rank: int, world: int, port: int, out):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from param_decomp_b200.config.run import AdamWOptimizerConfig
    from param_decomp_b200.parallel.sharded_optim import ShardedFlatAdamW

    torch.manual_seed(0)
    params = [torch.randn(5, 7), torch.randn(13)]
    cfg = AdamWOptimizerConfig(lr_schedule=1e-2, weight_decay=0.1, grad_clip_norm=0.5)
    opt = ShardedFlatAdamW(cfg, ["a", "b"], params, total_steps=10, group=dist.group.WORLD)
    for step in range(3):
        opt.zero_grad()
        g = torch.Generator().manual_seed(100 * step + rank)  # each rank has its own local gradient
        for p in params:
            p.grad.add_(torch.randn(p.shape, generator=g))
        opt.step(step)
    opt.refresh_full_fp32()
    out[rank] = ([p.detach().clone() for p in params], opt.working_view(0).float().clone(), opt.grad_norm())
    dist.destroy_process_group()


def test_sharded_adamw_matches_single_process_mean_gradient():
    from param_decomp_b200.config.run import AdamWOptimizerConfig
    from param_decomp_b200.core.optim import build_group_optimizer

    world, port = 2, _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_sharded_worker, args=(world, port, out), nprocs=world, join=True)
    torch.manual_seed(0)
    ref = [torch.randn(5, 7), torch.randn(13)]
    cfg = AdamWOptimizerConfig(lr_schedule=1e-2, weight_decay=0.1, grad_clip_norm=0.5)
    opt = build_group_optimizer(cfg, [("a", ref[0]), ("b", ref[1])], total_steps=10)
    for step in range(3):
        grads = []
        for p in ref:
            gs = []
            for r in range(world):
                pass
            grads.append(None)
        gens = [torch.Generator().manual_seed(100 * step + r) for r in range(world)]
        grads = [sum(torch.randn(p.shape, generator=g) for g in gens) / world for p in ref]
        opt.step(step, grads)
    for r in range(world):
        params, work0, norm = out[r]
        for a, b in zip(params, ref):
            assert torch.allclose(a, b, atol=1e-6)
        assert torch.allclose(work0, ref[0].to(torch.bfloat16).float(), atol=1e-6)
    assert out[0][2] == pytest.approx(float(opt.last_grad_norm_t), rel=1e-5)
