"""Expert parallelism for the MoE target: experts (frozen weights + their component blocks) are
sharded over the expert group, tokens stay data-parallel, and jobs travel to their expert's owner.

Two modes
  * `all_to_all` (default): each job's activation row and its per-job mask rows are sent to the
    owning rank (variable counts, exchanged first), the owner runs its experts' gate/up/down sites on
    the received jobs, and the output rows return by the reverse all-to-all. Differentiable: the
    backward of a dispatch is a combine and vice versa.
  * `allreduce`: the reference's scheme ("EP by activation slicing", param_decomp/routed/
    experts.py:28-40,864-885): every rank sees all tokens of its data shard's group, computes only
    its local experts' jobs, partial outputs are summed over the group. Kept for parity and as the
    baseline the all-to-all path is measured against.

Experts are padded with never-routed dummies so their count tiles the group (the analogue of stack
padding): `E_pad = ceil(E / W) * W`, rank `r` owns experts `[r E_loc, (r+1) E_loc)`.

The transport here is `torch.distributed` (NCCL on GPUs, gloo on CPU). The peer-memory kernel that
writes dispatched rows straight into the owner's receive buffer, ordered by expert, is
`ops/csrc/collectives_sm100.cu::pd_ep_dispatch` (selected with `transport="p2p"`).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor

from param_decomp_b200.core.masking import SiteMask


def padded_experts(n_experts: int, world: int) -> int:
    return (n_experts + world - 1) // world * world


def local_expert_range(n_experts: int, rank: int, world: int) -> tuple[int, int]:
    e_loc = padded_experts(n_experts, world) // world
    return rank * e_loc, (rank + 1) * e_loc


def shard_expert_weights(weights: dict[str, Tensor], n_experts: int, rank: int, world: int) -> dict[str, Tensor]:
    """Keep this rank's slice of every `experts_*` weight (zero-padded dummies at the tail)."""
    lo, hi = local_expert_range(n_experts, rank, world)
    out = {}
    for k, w in weights.items():
        if ".experts_" in k and w.dim() == 3:
            pad = padded_experts(n_experts, world) - w.shape[0]
            if pad:
                w = torch.cat([w, w.new_zeros(pad, *w.shape[1:])], dim=0)
            out[k] = w[lo:hi].contiguous()
        else:
            out[k] = w
    return out


class _AllToAll(torch.autograd.Function):
    """Variable-count all-to-all of rows; backward is the transposed exchange."""

    @staticmethod
    def forward(ctx, x: Tensor, send: list[int], recv: list[int], group) -> Tensor:  # type: ignore[override]
        ctx.send, ctx.recv, ctx.group = send, recv, group
        out = x.new_empty(sum(recv), *x.shape[1:])
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=group)
        return out

    @staticmethod
    def backward(ctx, g: Tensor):  # type: ignore[override]
        out = g.new_empty(sum(ctx.send), *g.shape[1:])
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv,
                               group=ctx.group)
        return out, None, None, None


@dataclass
class ExpertParallel:
    group: Any
    n_experts: int  # the model's true expert count (before padding)
    mode: str = "all_to_all"

    def __post_init__(self) -> None:
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.e_loc = padded_experts(self.n_experts, self.world) // self.world

    # ---------------------------------------------------------------------------------------------
    def run_experts(self, model, layer: int, xt: Tensor, expert_of_job: Tensor, token_of_job: Tensor,
                    slot_of_job: Tensor, weights, masks) -> Tensor:
        """`xt [N, d]` local tokens; returns `[J, d]` outputs in job order (token-major, slot-minor)."""
        if self.mode == "allreduce":
            return self._allreduce(model, layer, xt, expert_of_job, token_of_job, slot_of_job, weights, masks)
        J = expert_of_job.numel()
        dest = expert_of_job // self.e_loc
        order = dest.argsort(stable=True)
        send = torch.bincount(dest, minlength=self.world)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        send_l, recv_l = send.tolist(), recv.tolist()

        def ship(rows: Tensor) -> Tensor:
            return _AllToAll.apply(rows[order], send_l, recv_l, self.group)

        x_recv = ship(xt[token_of_job])
        e_recv = _AllToAll.apply((expert_of_job % self.e_loc)[order], send_l, recv_l, self.group)
        # per-job mask payload of the three expert sites
        names = [f"layers.{layer}.mlp.experts_{k}" for k in ("gate", "up", "down")]
        job_masks: dict[str, SiteMask] = {}
        if masks is not None:
            for name in names:
                if name not in masks:
                    continue
                sm = masks[name].materialize()
                spec = next(s for s in model.sites if s.name == name)
                c = spec.C_block
                m = d = r = None
                if sm.mask is not None:
                    flat = sm.mask.reshape(-1, sm.mask.shape[-1])
                    m = ship(flat.reshape(flat.shape[0], -1, c)[token_of_job, slot_of_job])
                if sm.delta is not None:
                    d = ship(sm.delta.reshape(-1, 1)[token_of_job])
                if sm.route is not None:
                    r = ship(sm.route.reshape(-1, 1)[token_of_job].float())[:, 0] > 0.5
                job_masks[name] = SiteMask(mask=m, delta=d, route=r)
        Jr = x_recv.shape[0]
        ar = torch.arange(Jr, device=xt.device)
        y_recv = self._local(model, layer, x_recv, e_recv, weights, job_masks if masks is not None else None, ar)
        y_sorted = _AllToAll.apply(y_recv, recv_l, send_l, self.group)
        inv = torch.empty_like(order)
        inv[order] = torch.arange(J, device=order.device)
        return y_sorted[inv]

    def _local(self, model, layer: int, x_jobs: Tensor, e_local: Tensor, weights, masks, ar: Tensor) -> Tensor:
        order, bounds = e_local, [0]
        if not model._fused(x_jobs):
            order = e_local.argsort(stable=True)
            for n in torch.bincount(e_local, minlength=self.e_loc).tolist():
                bounds.append(bounds[-1] + n)
        return model.expert_jobs(layer, x_jobs, e_local, order, bounds, weights, masks, ar, torch.zeros_like(ar))

    def _allreduce(self, model, layer, xt, expert_of_job, token_of_job, slot_of_job, weights, masks) -> Tensor:
        import torch.distributed.nn.functional as dfn

        lo = self.rank * self.e_loc
        mine = (expert_of_job >= lo) & (expert_of_job < lo + self.e_loc)
        idx = mine.nonzero()[:, 0]
        y = xt.new_zeros(expert_of_job.numel(), xt.shape[-1])
        if idx.numel():
            sub_masks = None
            if masks is not None:
                sub_masks = {}
                for name, sm in masks.items():
                    if ".experts_" not in name or f"layers.{layer}." not in name:
                        continue
                    sm = sm.materialize()
                    c = next(s for s in model.sites if s.name == name).C_block
                    m = None
                    if sm.mask is not None:
                        flat = sm.mask.reshape(-1, sm.mask.shape[-1])
                        m = flat.reshape(flat.shape[0], -1, c)[token_of_job[idx], slot_of_job[idx]]
                    d = None if sm.delta is None else sm.delta.reshape(-1, 1)[token_of_job[idx]]
                    r = None if sm.route is None else sm.route.reshape(-1)[token_of_job[idx]]
                    sub_masks[name] = SiteMask(mask=m, delta=d, route=r)
            ar = torch.arange(idx.numel(), device=xt.device)
            y_local = self._local(model, layer, xt[token_of_job[idx]], expert_of_job[idx] - lo, weights, sub_masks, ar)
            y = y.index_copy(0, idx, y_local.to(y.dtype))
        return dfn.all_reduce(y, group=self.group)
