"""Muon with its Newton-Schulz work and momentum split over the data-parallel group.

Each stacked leaf `[g, m, n]` (one matrix per site of a kind) is split along its stack axis: rank `r` of `W`
owns matrices `[r g / W, (r + 1) g / W)`. It keeps the momentum of its own matrices only, runs the batched
Newton-Schulz iteration on them (whole matrices per rank, so the iteration itself needs no communication),
updates them, and the updated slices are all-gathered back into every rank's copy of the leaf. Stacks are
padded with inert zero matrices to a multiple of `W` (`ComponentStacks(stack_multiple=W)`; an all-zero
gradient orthogonalises to zero, so pads stay zero). Leaves that are not stacks of matrices take Muon's
Nesterov-Adam rule, replicated. Gradients arrive already averaged over the group (the engine all-reduces
them, as for any replicated optimizer); the clip norm is therefore the same number on every rank.

This is the reference's Newton-Schulz staging - each kind's stack split over the mesh, matrices whole per
device, a hop in and a hop out (param_decomp/core/muon_stacked.py:120-147,207-310;
core/placement.py:1028-1038) - with the momentum sharded the same way, so optimizer state is 1 / W per rank.
Checkpoints store whole per-parameter moments (`gather_state`), so a run resumes on any device count.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor

from param_decomp_b200.config.run import MuonOptimizerConfig
from param_decomp_b200.config.schedule import get_scheduled_value
from param_decomp_b200.core.optim import clip_scale, global_norm, newton_schulz_of_slice


@dataclass
class StackShardedMuon:
    cfg: MuonOptimizerConfig
    names: list[str]
    params: list[Tensor]
    total_steps: int
    group: Any = None
    state: dict[str, Tensor] = field(default_factory=dict)  # "<leaf>/mom" (own slice), "<leaf>/mu", "<leaf>/nu"
    count: int = 0
    applied_learning_rate: float = 0.0
    last_grad_norm_t: Tensor | None = None
    norm_fn: Any = None  # (names, grads) -> global L2 norm where leaves are split over a process group
    column_split: Any = None  # `StackSharding` in component mode: whole matrices are gathered for Newton-Schulz

    def __post_init__(self) -> None:
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        self.rank = dist.get_rank(self.group) if self.group is not None else 0
        for n, p in zip(self.names, self.params):
            if self._is_stack(p):
                assert p.shape[0] % self.world == 0, (
                    f"{n}: stack of {p.shape[0]} matrices does not tile {self.world} ranks "
                    "(build the component stacks with stack_multiple = the group size)")

    @staticmethod
    def _is_stack(p: Tensor) -> bool:
        return p.dim() >= 3 and min(p.shape[-2:]) > 1

    def _own(self, p: Tensor) -> slice:
        per = p.shape[0] // self.world
        return slice(self.rank * per, (self.rank + 1) * per)

    def lr_at(self, step: int) -> float:
        return get_scheduled_value(min(step, self.total_steps), self.total_steps, self.cfg.lr_schedule)

    def grad_norm(self) -> float:
        return float(self.last_grad_norm_t)

    def _get(self, key: str, like: Tensor) -> Tensor:
        if key not in self.state:
            self.state[key] = torch.zeros_like(like, dtype=torch.float32)
        return self.state[key]

    @torch.no_grad()
    def step(self, step_idx: int, grads: list[Tensor | None] | None = None) -> dict[str, float]:
        cfg = self.cfg
        if grads is None:
            grads = [p.grad for p in self.params]
        live = [(n, p, g) for n, p, g in zip(self.names, self.params, grads) if g is not None]
        if self.norm_fn is not None and live:
            norm = self.norm_fn([n for n, _, _ in live], [g for _, _, g in live])
        else:
            norm = global_norm([g for _, _, g in live])
        scale = clip_scale(norm, cfg.grad_clip_norm)
        lr = self.lr_at(step_idx)
        self.count += 1
        t, b = self.count, cfg.beta
        self.applied_learning_rate, self.last_grad_norm_t = lr, norm
        ns_dtype = torch.bfloat16 if cfg.ns_dtype == "bfloat16" else torch.float32
        for n, p, g in live:
            g = g.float() * scale.to(g.device)
            if not self._is_stack(p):
                if p.dim() >= 2 and min(p.shape[-2:]) > 1:  # a single matrix: orthogonalised on every rank
                    self._muon_update(n, p, g, slice(None), lr, t, b, ns_dtype)
                else:
                    self._nadam(n, p, g, lr, t)
                continue
            own = self._own(p)
            self._muon_update(n, p, g, own, lr, t, b, ns_dtype)
            if self.world > 1:  # egress hop: every rank receives the other ranks' updated matrices
                dist.all_gather_into_tensor(p.data.view(-1), p.data[own].reshape(-1).clone(), group=self.group)
        return {"lr": lr}

    def _muon_update(self, n: str, p: Tensor, g: Tensor, own: slice, lr: float, t: int, b: float, ns_dtype) -> None:
        cfg = self.cfg
        mom = self._get(n + "/mom", p[own])
        mom.mul_(b).add_(g[own], alpha=1 - b)
        mix = (b / (1 - b ** (t + 1))) * mom + ((1 - b) / (1 - b**t)) * g[own]
        O, fan_in, fan_out = newton_schulz_of_slice(n, mix, self.column_split, cfg.ns_steps, ns_dtype)
        s = (math.sqrt(max(fan_in, fan_out)) * cfg.consistent_rms if cfg.consistent_rms is not None
             else math.sqrt(max(1.0, fan_out / fan_in)))
        if cfg.weight_decay:
            p[own].mul_(1 - lr * cfg.weight_decay)
        p[own].add_(O.float(), alpha=-lr * s)

    def _nadam(self, n: str, p: Tensor, g: Tensor, lr: float, t: int) -> None:
        b1, b2 = 0.9, 0.999
        mu, nu = self._get(n + "/mu", p), self._get(n + "/nu", p)
        mu.mul_(b1).add_(g, alpha=1 - b1)
        nu.mul_(b2).addcmul_(g, g, value=1 - b2)
        mu_hat = (b1 / (1 - b1 ** (t + 1))) * mu + ((1 - b1) / (1 - b1**t)) * g
        p.add_(mu_hat / ((nu / (1 - b2**t)).sqrt() + 1e-8), alpha=-lr)

    # -- checkpoint (layout-independent) ----------------------------------------------------------------
    def gather_state(self) -> None:
        """Collective: assemble whole per-parameter momenta so `state_dict` (called by the writing rank only)
        does not depend on how many ranks shared them."""
        out = {}
        for n, p in zip(self.names, self.params):
            key = n + "/mom"
            if key not in self.state:
                continue
            m = self.state[key]
            if self._is_stack(p) and self.world > 1:
                full = torch.empty(p.shape, device=m.device, dtype=m.dtype)
                dist.all_gather_into_tensor(full.view(-1), m.reshape(-1).contiguous(), group=self.group)
                out[key] = full
            else:
                out[key] = m
        self._gathered = out

    def state_dict(self) -> dict[str, Tensor]:
        gathered = getattr(self, "_gathered", None)
        assert self.world == 1 or gathered is not None, "call gather_state() on every rank before saving"
        self._gathered = None
        out = {k: v for k, v in self.state.items() if not k.endswith("/mom")}
        out.update(gathered if gathered is not None else {k: v for k, v in self.state.items() if k.endswith("/mom")})
        out["count"] = torch.tensor(self.count, dtype=torch.int64)
        return out

    def load_state_dict(self, sd: dict[str, Tensor]) -> None:
        by_name = dict(zip(self.names, self.params))
        for k, v in sd.items():
            if k == "count":
                self.count = int(v.item())
                continue
            leaf, suffix = k.rsplit("/", 1)
            p = by_name.get(leaf)
            if suffix == "mom" and p is not None and self._is_stack(p) and v.shape[0] == p.shape[0] and self.world > 1:
                v = v[self._own(p)].contiguous()  # the file holds whole momenta: keep this rank's matrices
            self.state[k] = v
