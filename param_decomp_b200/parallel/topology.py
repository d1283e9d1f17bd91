"""Process topology: one process per GPU, a logical `(replicate, fsdp, tp)` or `(data, tp)` mesh over
`torch.distributed` (NCCL for device tensors, a gloo group for host-side consensus and barriers).

Rank layout: `tp` is the fastest-varying axis, then `fsdp`, then `replicate`, so tensor-parallel
peers are adjacent ranks. `batch axes` = every non-`tp` axis: the batch is sharded over them and
replicated over `tp`.

Parity: param_decomp/core/sharding.py:19-25,58-116 (topology init, meshes), core/placement.py:96-101
(`batch_axes`), core/run.py:335-379 (SIGTERM consensus as a host all-reduce).
"""

from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor

from param_decomp_b200.config.run import HsdpMeshShape, ResidentMeshShape
from param_decomp_b200.core.train import DataCollectives


def mesh_axes(shape: HsdpMeshShape | ResidentMeshShape) -> list[tuple[str, int]]:
    if isinstance(shape, HsdpMeshShape):
        return [("replicate", shape.replicate), ("fsdp", shape.fsdp), ("tp", shape.tp)]
    return [("data", shape.data), ("tp", shape.tp)]


def axis_coords(rank: int, axes: list[tuple[str, int]]) -> dict[str, int]:
    """Row-major coordinates with the LAST axis fastest."""
    out = {}
    for name, size in reversed(axes):
        out[name] = rank % size
        rank //= size
    return out


def axis_group_ranks(rank: int, axes: list[tuple[str, int]], names: tuple[str, ...]) -> list[int]:
    """Ranks that share this rank's coordinates on every axis NOT in `names`, ordered by their
    (row-major) coordinates on `names`."""
    me = axis_coords(rank, axes)
    world = 1
    for _, s in axes:
        world *= s
    out = []
    for r in range(world):
        c = axis_coords(r, axes)
        if all(c[n] == me[n] for n, _ in axes if n not in names):
            out.append(r)
    return out


class DistCollectives(DataCollectives):
    """Data-parallel collectives over the batch axes of the mesh."""

    def __init__(self, topo: "Topology") -> None:
        self.topo = topo
        self.world_size = topo.data_world
        self.rank = topo.rank
        self.data_rank = topo.data_rank

    def mean(self, t: Tensor) -> Tensor:
        if self.world_size == 1:
            return t
        import torch.distributed.nn.functional as dfn

        return dfn.all_reduce(t, op=dist.ReduceOp.SUM, group=self.topo.data_group) / self.world_size

    def sum_(self, t: Tensor) -> Tensor:
        if self.world_size > 1:
            dist.all_reduce(t, group=self.topo.data_group)
        return t

    def row_offset(self, local_rows: int) -> int:
        return self.data_rank * local_rows

    def gather_rows(self, t: Tensor) -> Tensor:
        if self.world_size == 1:
            return t
        src = t.contiguous()
        as_int = src.dtype == torch.uint16  # no collective for uint16: move the bits
        if as_int:
            src = src.view(torch.int16)
        parts = [torch.empty_like(src) for _ in range(self.world_size)]
        dist.all_gather(parts, src, group=self.topo.data_group)
        full = torch.cat(parts, dim=0)
        return full.view(torch.uint16) if as_int else full

    def reduce_grads_everywhere(self, params: list[Tensor]) -> None:
        self.reduce_grads(params, group=None, world=self.topo.world)

    def reduce_grads(self, params: list[Tensor], group: Any = "data", world: int | None = None) -> None:
        """Average gradients over the data group (or, `group=None`, the whole job) in few large flat
        buckets (NVSwitch makes the cost launch-bound, not link-bound, so buckets are sized for
        latency: 256 MiB)."""
        group = self.topo.data_group if group == "data" else group
        world = self.world_size if world is None else world
        if world == 1 or self.topo.world == 1:
            return
        grads = [p.grad for p in params if p.grad is not None]
        bucket, size, limit = [], 0, 64 * 1024 * 1024  # elements
        def flush() -> None:
            nonlocal bucket, size
            if not bucket:
                return
            flat = torch.cat([g.reshape(-1) for g in bucket]) if len(bucket) > 1 else bucket[0].reshape(-1)
            dist.all_reduce(flat, group=group)
            flat.div_(world)
            if len(bucket) > 1:
                off = 0
                for g in bucket:
                    g.copy_(flat[off:off + g.numel()].view_as(g))
                    off += g.numel()
            bucket, size = [], 0
        for g in grads:
            if g.numel() >= limit:
                dist.all_reduce(g, group=group)
                g.div_(world)
                continue
            bucket.append(g)
            size += g.numel()
            if size >= limit:
                flush()
        flush()

    def average_scalars(self, values: dict) -> dict:
        """Evaluation metrics are computed by every rank on its own rows of the evaluation batch: average the
        scalar entries over the job on the host group (same keys on every rank; other entries pass through)."""
        if self.topo.world == 1:
            return values
        keys = sorted(k for k, v in values.items()
                      if isinstance(v, (int, float)) or (isinstance(v, Tensor) and v.numel() == 1))
        if not keys:
            return values
        t = torch.tensor([float(values[k]) for k in keys], dtype=torch.float64)
        dist.all_reduce(t, group=self.topo.cpu_group)
        out = dict(values)
        out.update({k: float(x) / self.topo.world for k, x in zip(keys, t)})
        return out

    @property
    def in_first_tp_group(self) -> bool:
        """Ranks `0 .. tp-1` (tp is the fastest axis): the one tp group that assembles split stacks for a save."""
        return self.topo.rank < self.topo.tp_world

    @property
    def split_grad_scale(self) -> float:
        """Factor for batch-independent loss terms on split leaves: `reduce_split_grads` divides by the number of
        batch shards, of which only `1 / tp` contributed such a term to a given part."""
        return float(self.topo.tp_world) if self.topo.batch_over_tp else 1.0

    def reduce_split_grads(self, params: list[Tensor]) -> None:
        """Gradients of leaves that are split over the tp axis (each rank holds its own part). When the batch
        is replicated over tp they average over the batch axes like everything else. When the batch is also
        sharded over tp (all-to-all expert dispatch) a part's gradient already holds the sum over its tp group's
        tokens: sum over the ranks holding the same part, divide by the number of batch shards (all ranks)."""
        if self.topo.batch_over_tp:
            self.reduce_grads(params, group=self.topo.replica_group, world=self.topo.world)
        else:
            self.reduce_grads(params)

    def host_any(self, flag: float) -> bool:
        if self.topo.world == 1:
            return bool(flag)
        t = torch.tensor([flag], dtype=torch.float32)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.topo.cpu_group)
        return bool(t.item() > 0)

    def barrier(self) -> None:
        if self.topo.world > 1:
            dist.barrier(group=self.topo.cpu_group)


@dataclass
class Topology:
    rank: int
    world: int
    local_rank: int
    device: torch.device
    axes: list[tuple[str, int]]
    coords: dict[str, int]
    groups: dict[str, Any] = field(default_factory=dict)  # axis name -> process group
    data_group: Any = None
    cpu_group: Any = None
    owns_process_group: bool = False
    batch_over_tp: bool = False  # True: the batch is sharded over the tp axis as well (all-to-all expert dispatch)
    replica_group: Any = None  # ranks sharing this rank's tp coordinate (they hold the same split parts)

    @property
    def tp_world(self) -> int:
        return dict(self.axes).get("tp", 1)

    @property
    def tp_rank(self) -> int:
        return self.coords.get("tp", 0)

    @property
    def data_world(self) -> int:
        return self.world if self.batch_over_tp else self.world // self.tp_world

    @property
    def data_rank(self) -> int:
        return self.rank if self.batch_over_tp else self.rank // self.tp_world

    def axis_size(self, name: str) -> int:
        return dict(self.axes).get(name, 1)

    def collectives(self) -> DataCollectives:
        return DistCollectives(self) if self.world > 1 else DataCollectives()

    def broadcast_object(self, obj: Any) -> Any:
        if self.world == 1:
            return obj
        box = [obj]
        dist.broadcast_object_list(box, src=0, group=self.cpu_group)
        return box[0]

    def shutdown(self, failed: bool = False) -> None:
        """Leave the job. A rank that is unwinding from an exception (`failed`) does not wait for the others
        at a barrier they may never reach - their next collective ends with an error instead."""
        if self.owns_process_group and dist.is_initialized():
            if failed:
                return  # no barrier, no communicator teardown (it can block on peers): the process is about to exit
            dist.barrier(group=self.cpu_group)
            dist.destroy_process_group()


def initialize(shape: HsdpMeshShape | ResidentMeshShape | None, device: str | None = None,
               timeout_s: float = 600.0, batch_over_tp: bool = False) -> Topology:
    """Join the job named by `RANK/WORLD_SIZE/LOCAL_RANK/MASTER_*` (single process if unset) and
    build one process group per mesh axis plus the data (batch-axes) group and a gloo group."""
    env_world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() and (device is None or str(device).startswith("cuda"))
    if use_cuda:
        dev = torch.device("cuda", local_rank if device in (None, "cuda") else torch.device(device).index or 0)
        torch.cuda.set_device(dev)
    else:
        dev = torch.device("cpu")
    axes = mesh_axes(shape) if shape is not None else [("data", env_world), ("tp", 1)]
    mesh_world = 1
    for _, s in axes:
        mesh_world *= s
    if env_world == 1:
        # A single process runs any mesh config as its own 1-rank slice (tests, smoke, 1-GPU bench).
        axes = [(n, 1) for n, _ in axes]
        return Topology(0, 1, 0, dev, axes, {n: 0 for n, _ in axes})
    assert mesh_world == env_world, f"mesh {axes} needs {mesh_world} ranks, job has {env_world}"
    owns = False
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=env_world,
                                timeout=datetime.timedelta(seconds=timeout_s),
                                device_id=dev if use_cuda else None)
        owns = True
    coords = axis_coords(rank, axes)
    topo = Topology(rank, env_world, local_rank, dev, axes, coords, owns_process_group=owns)
    topo.cpu_group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
    # every rank must take part in every new_group call, in the same order
    for name, _ in axes:
        seen: set[tuple[int, ...]] = set()
        for r in range(env_world):
            members = tuple(axis_group_ranks(r, axes, (name,)))
            if members in seen:
                continue
            seen.add(members)
            g = dist.new_group(ranks=list(members))
            if rank in members:
                topo.groups[name] = g
    batch_names = tuple(n for n, _ in axes if n != "tp")
    seen = set()
    for r in range(env_world):
        members = tuple(axis_group_ranks(r, axes, batch_names))
        if members in seen:
            continue
        seen.add(members)
        g = dist.new_group(ranks=list(members))
        if rank in members:
            topo.data_group = g
    topo.replica_group = topo.data_group
    if batch_over_tp and topo.tp_world > 1:
        topo.batch_over_tp = True
        topo.data_group = dist.new_group(ranks=list(range(env_world)))  # every rank takes its own batch rows
    return topo
