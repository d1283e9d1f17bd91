"""Autograd pieces for computations split over a process group whose ranks all see the same batch
(tensor / expert parallelism): the conjugate identity / all-reduce pair and a column slice of a
replicated tensor. With them every rank holds exact gradients - full ones for replicated leaves,
its own for split leaves - so the data-parallel reduction needs no special cases.

Parity: the reshard points GSPMD inserts around `param_decomp/core/decomposed_linear.py:142-175`
(contraction over `C / tp` -> all-reduce of the site output) and `param_decomp/routed/experts.py:864-885`.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import Tensor


class CopyToGroup(torch.autograd.Function):
    """Identity whose adjoint sums over the group: for a replicated tensor that every rank feeds to
    its own (different) part of the weights, so the partial gradients add up to the full one."""

    @staticmethod
    def forward(ctx, x: Tensor, group) -> Tensor:  # type: ignore[override]
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        g = g.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class ReduceFromGroup(torch.autograd.Function):
    """Sum over the group whose adjoint is the identity: the summed output feeds a computation that is
    replicated on every rank, so each rank's partial receives the (identical) full gradient."""

    @staticmethod
    def forward(ctx, x: Tensor, group) -> Tensor:  # type: ignore[override]
        # the partial is a fresh product nobody else reads: reduce it in place (no producer here keeps its own
        # output for backward) instead of copying a [tokens, d_out] tensor per site
        if x.is_contiguous() and not x.is_leaf:
            ctx.mark_dirty(x)
            dist.all_reduce(x, group=group)
            return x
        out = x.contiguous().clone()
        dist.all_reduce(out, group=group)
        return out

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        return g, None


class SliceColumns(torch.autograd.Function):
    """`x[..., lo:hi]` of a replicated tensor, rank `r` of the group taking the `r`-th equal slice. Each
    rank's gradient lives on its own columns only, so the adjoint is an all-gather along the last axis
    (every rank ends with the full gradient) rather than an all-reduce of mostly-zero tensors."""

    @staticmethod
    def forward(ctx, x: Tensor, group) -> Tensor:  # type: ignore[override]
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        width = x.shape[-1] // world
        assert width * world == x.shape[-1], f"{x.shape[-1]} columns do not tile {world} ranks"
        ctx.group, ctx.world = group, world
        return x[..., rank * width:(rank + 1) * width]

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        g = g.contiguous()
        parts = [torch.empty_like(g) for _ in range(ctx.world)]
        dist.all_gather(parts, g, group=ctx.group)
        return torch.cat(parts, dim=-1), None


class GatherSequence(torch.autograd.Function):
    """`[B, T / W, d]` position shards -> the whole `[B, T, d]` on every rank. The consumers (the sites of a
    block) already hand every rank the FULL gradient of their input (their own adjoint sums the partial
    gradients over the group), so the adjoint here is this rank's slice of it, with no further reduction."""

    @staticmethod
    def forward(ctx, x: Tensor, group) -> Tensor:  # type: ignore[override]
        world = dist.get_world_size(group)
        ctx.rank, ctx.width = dist.get_rank(group), x.shape[1]
        x = x.contiguous()
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x, group=group)
        return torch.cat(parts, dim=1)

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        return g[:, ctx.rank * ctx.width:(ctx.rank + 1) * ctx.width], None


class SliceSequence(torch.autograd.Function):
    """This rank's `[B, T / W, d]` positions of a tensor every rank holds whole. Downstream each rank only
    produces gradients for its own positions while upstream (a site output summed over the group) expects the
    whole gradient on every rank: the adjoint all-gathers along the sequence."""

    @staticmethod
    def forward(ctx, x: Tensor, group) -> Tensor:  # type: ignore[override]
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        width = x.shape[1] // world
        assert width * world == x.shape[1], f"{x.shape[1]} positions do not tile {world} ranks"
        ctx.group, ctx.world = group, world
        return x[:, rank * width:(rank + 1) * width]

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        g = g.contiguous()
        parts = [torch.empty_like(g) for _ in range(ctx.world)]
        dist.all_gather(parts, g, group=ctx.group)
        return torch.cat(parts, dim=1), None


def gather_sequence(x: Tensor, group) -> Tensor:
    return GatherSequence.apply(x, group)


def slice_sequence(x: Tensor, group) -> Tensor:
    if not x.requires_grad:
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        width = x.shape[1] // world
        assert width * world == x.shape[1], f"{x.shape[1]} positions do not tile {world} ranks"
        return x[:, rank * width:(rank + 1) * width]
    return SliceSequence.apply(x, group)


def copy_to_group(x: Tensor, group) -> Tensor:
    return CopyToGroup.apply(x, group) if x.requires_grad else x


def slice_columns(x: Tensor, group) -> Tensor:
    return SliceColumns.apply(x, group)
