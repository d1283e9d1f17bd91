"""ZeRO-style sharded AdamW over the data-parallel group, with the collective fused into the update.

Layout per optimizer group (component stacks, CI function):
  * one flat fp32 gradient buffer `[n]` per rank (every parameter's `.grad` is a view into it, so
    the wgrad kernels and autograd accumulate straight into the communication buffer);
  * one flat bf16 working copy `[n]` per rank (every compute weight is a view into it);
  * fp32 masters and Adam moments only for the rank's contiguous shard `[n / W]`.
One step = reduce-scatter(grads) -> clip by the global norm -> AdamW on the shard -> all-gather(bf16).

Backends
  * `fused_p2p` (CUDA, symmetric memory): ONE cooperative kernel per rank does all of it with plain
    P2P loads/stores over NVLink (`ops/csrc/collectives_sm100.cu::pd_rs_adamw_ag`); gradients cross
    NVLink once (each rank pulls only its shard from every peer) and updated weights cross once in
    bf16. No NCCL call, no separate cast, no separate optimizer launch.
  * `collective` (NCCL or gloo): `reduce_scatter_tensor` + local AdamW + `all_gather_into_tensor`;
    the correctness oracle and the measured baseline for the fused path.

Reference behaviour covered: the `zero1` / `owner` optimizer-state rows and the once-per-step entry
all-gather / exit reduce-scatter (param_decomp/core/placement.py:636-688,1013-1068;
core/PLACEMENT_DESIGN.md:86-151), which the reference leaves un-overlapped.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import torch
import torch.distributed as dist
from torch import Tensor

from param_decomp_b200.config.run import AdamWOptimizerConfig
from param_decomp_b200.config.schedule import get_scheduled_value

MAX_RANKS = 8


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class PdPeerPtrs(C.Structure):
    _fields_ = [("ptr", C.c_void_p * MAX_RANKS)]


class PdRsAdamwCall(C.Structure):
    _fields_ = [
        ("grads", PdPeerPtrs), ("work", PdPeerPtrs), ("work_lo", PdPeerPtrs), ("flags", PdPeerPtrs), ("norms", PdPeerPtrs),
        ("p", C.c_void_p), ("m", C.c_void_p), ("v", C.c_void_p),
        ("shard_off", C.c_longlong), ("shard_len", C.c_longlong),
        ("rank", C.c_int), ("world", C.c_int), ("seq", C.c_uint),
        ("lr", C.c_float), ("b1", C.c_float), ("b2", C.c_float), ("eps", C.c_float), ("wd", C.c_float),
        ("bc1", C.c_float), ("bc2", C.c_float), ("max_norm", C.c_float),
        ("norm_out", C.c_void_p), ("status", C.c_void_p), ("limit_s", C.c_double),
        ("hyper_dev", C.c_void_p), ("seq_dev", C.c_void_p),
    ]  # fmt: skip


def _peer_table(ptrs: list[int]) -> PdPeerPtrs:
    t = PdPeerPtrs()
    for i, p in enumerate(ptrs):
        t.ptr[i] = p
    return t


def symmetric_empty(numel: int, dtype: torch.dtype, device, group) -> tuple[Tensor, list[int]]:
    """A buffer every rank of `group` can address: returns (local tensor, peer pointers by rank)."""
    import torch.distributed._symmetric_memory as symm

    t = symm.empty(numel, dtype=dtype, device=device)
    hdl = symm.rendezvous(t, group=group)
    return t, [int(p) for p in hdl.buffer_ptrs]


@dataclass
class ShardedFlatAdamW:
    """AdamW over named fp32 parameters whose storage is re-homed into flat buffers."""

    cfg: AdamWOptimizerConfig
    names: list[str]
    params: list[Tensor]
    total_steps: int
    group: object | None  # data-parallel process group (None = single process)
    backend: str = "collective"  # "fused_p2p" | "collective"
    wait_limit_s: float = 30.0  # a peer may be late by a checkpoint write or an evaluation, not by a dead process
    keep_lo: bool = False  # also publish bf16(p - bf16(p)): split-precision operands for faithfulness
    norm_group: object | None = None  # leaves are slices of stacks split over this group: its ranks' squares add up
    count: int = 0
    applied_learning_rate: float = 0.0
    last_grad_norm_t: Tensor | None = None
    scalars: object | None = None  # ops.step_scalars.StepScalars: lr, bias corrections and barrier sequence in device memory
    label: str = "components"
    _seq: int = 1
    state: dict[str, Tensor] = field(default_factory=dict)

    def __post_init__(self) -> None:
        assert self.norm_group is None or self.backend == "collective", \
            "the fused kernel computes the clip norm among its own peers; split stacks use the collective form"
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        self.rank = dist.get_rank(self.group) if self.group is not None else 0
        dev = self.params[0].device
        sizes = [p.numel() for p in self.params]
        self.offsets, off = [], 0
        for n in sizes:
            self.offsets.append(off)
            off += _align(n, 8)
        self.n = _align(off, 8 * self.world)
        self.shard_len = self.n // self.world
        self.shard_off = self.rank * self.shard_len
        if self.backend == "fused_p2p":
            self.grad_flat, self.grad_ptrs = symmetric_empty(self.n, torch.float32, dev, self.group)
            self.work_flat, self.work_ptrs = symmetric_empty(self.n, torch.bfloat16, dev, self.group)
            self.work_lo_flat, self.work_lo_ptrs = (symmetric_empty(self.n, torch.bfloat16, dev, self.group)
                                                    if self.keep_lo else (None, [0] * self.world))
            self.flags, self.flag_ptrs = symmetric_empty(MAX_RANKS, torch.int32, dev, self.group)
            self.norms, self.norm_ptrs = symmetric_empty(8, torch.float32, dev, self.group)
            self.flags.zero_()
            self.norms.zero_()
        else:
            self.grad_flat = torch.zeros(self.n, device=dev, dtype=torch.float32)
            self.work_flat = torch.zeros(self.n, device=dev, dtype=torch.bfloat16)
            self.work_lo_flat = torch.zeros(self.n, device=dev, dtype=torch.bfloat16) if self.keep_lo else None
        self.grad_flat.zero_()
        full = torch.zeros(self.n, device=dev, dtype=torch.float32)
        for p, o in zip(self.params, self.offsets):
            full[o:o + p.numel()].copy_(p.detach().reshape(-1))
        self.work_flat.copy_(full)
        if self.work_lo_flat is not None:
            self.work_lo_flat.copy_(full - self.work_flat.float())
        self.master = full[self.shard_off:self.shard_off + self.shard_len].clone()
        self.mu = torch.zeros_like(self.master)
        self.nu = torch.zeros_like(self.master)
        self.norm_out = torch.zeros(1, device=dev, dtype=torch.float32)
        self.full_fp32 = full  # kept so `.data` of every parameter stays a valid fp32 view
        self._attach_views()
        if self.group is not None and self.backend == "fused_p2p":
            torch.cuda.synchronize()
            dist.barrier(group=self.group)

    # -- views ---------------------------------------------------------------------------------
    def _attach_views(self) -> None:
        """Point every parameter's storage and `.grad` at its slice of the flat buffers."""
        for p, o in zip(self.params, self.offsets):
            p.data = self.full_fp32[o:o + p.numel()].view_as(p)
            p.grad = self.grad_flat[o:o + p.numel()].view_as(p)

    def _grads_attached(self) -> bool:
        base = self.grad_flat.data_ptr()
        return all(p.grad is not None and p.grad.data_ptr() == base + 4 * o for p, o in zip(self.params, self.offsets))

    def working_lo_view(self, index: int) -> Tensor:
        assert self.work_lo_flat is not None
        p, o = self.params[index], self.offsets[index]
        return self.work_lo_flat[o:o + p.numel()].view_as(p)

    def working_view(self, index: int) -> Tensor:
        """bf16 working copy of parameter `index` (a view into the flat all-gathered buffer)."""
        p, o = self.params[index], self.offsets[index]
        return self.work_flat[o:o + p.numel()].view_as(p)

    def zero_grad(self) -> None:
        self.grad_flat.zero_()

    def lr_at(self, step: int) -> float:
        return get_scheduled_value(min(step, self.total_steps), self.total_steps, self.cfg.lr_schedule)

    def grad_norm(self) -> float:
        return float(self.norm_out)

    # -- the step ------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, step_idx: int) -> dict[str, float]:
        assert self._grads_attached(), \
            "a parameter's .grad no longer aliases the flat gradient buffer (something replaced it; gradients would be lost)"
        lr = self.lr_at(step_idx)
        self.count += 1
        self._step_idx = step_idx
        self.applied_learning_rate = lr
        b1, b2 = self.cfg.betas
        bc1, bc2 = 1 - b1**self.count, 1 - b2**self.count
        max_norm = self.cfg.grad_clip_norm or 0.0
        if self.backend == "fused_p2p":
            self._fused(lr, b1, b2, bc1, bc2, max_norm)
        else:
            self._collective(lr, b1, b2, bc1, bc2, max_norm)
        self.last_grad_norm_t = self.norm_out[0]
        # fp32 view of the whole parameter vector is refreshed lazily (checkpoints, faithfulness)
        self._full_stale = True
        return {"lr": lr}

    def _fused(self, lr, b1, b2, bc1, bc2, max_norm) -> None:
        from param_decomp_b200.ops import native as nv

        call = PdRsAdamwCall()
        call.grads, call.work = _peer_table(self.grad_ptrs), _peer_table(self.work_ptrs)
        call.work_lo = _peer_table(self.work_lo_ptrs)
        call.flags, call.norms = _peer_table(self.flag_ptrs), _peer_table(self.norm_ptrs)
        call.p, call.m, call.v = self.master.data_ptr(), self.mu.data_ptr(), self.nu.data_ptr()
        call.shard_off, call.shard_len = self.shard_off, self.shard_len
        call.rank, call.world, call.seq = self.rank, self.world, self._seq
        if self.scalars is not None:
            off, seq0, s0 = self.count - self._step_idx, self._seq, self._step_idx
            call.hyper_dev = self.scalars.f32_block(f"opt/{self.label}/hyper", 3, lambda s: (
                self.lr_at(s), 1.0 / (1 - b1 ** (s + off)), 1.0 / (1 - b2 ** (s + off)))).data_ptr()
            call.seq_dev = self.scalars.u32(f"opt/{self.label}/seq", lambda s: seq0 + 3 * (s - s0)).data_ptr()
        self._seq += 3
        call.lr, call.b1, call.b2, call.eps, call.wd = lr, b1, b2, 1e-8, self.cfg.weight_decay
        call.bc1, call.bc2, call.max_norm = bc1, bc2, max_norm
        call.norm_out, call.status = self.norm_out.data_ptr(), nv.status_word().data_ptr()
        call.limit_s = self.wait_limit_s
        lib = nv.lib()
        lib.pd_rs_adamw_ag.argtypes = [C.POINTER(PdRsAdamwCall), C.c_void_p]
        lib.pd_rs_adamw_ag.restype = C.c_int
        rc = lib.pd_rs_adamw_ag(C.byref(call), nv.current_stream_ptr())
        nv.count_launch()
        if rc != 0:
            raise nv.NativeError(f"pd_rs_adamw_ag refused the call (code {rc})")

    def _collective(self, lr, b1, b2, bc1, bc2, max_norm) -> None:
        if self.world > 1:
            if dist.get_backend(self.group) == "gloo":  # gloo has no reduce-scatter
                summed = self.grad_flat.clone()
                dist.all_reduce(summed, group=self.group)
                shard = summed[self.shard_off:self.shard_off + self.shard_len]
            else:
                shard = torch.empty(self.shard_len, device=self.grad_flat.device, dtype=torch.float32)
                dist.reduce_scatter_tensor(shard, self.grad_flat, group=self.group)
        else:
            shard = self.grad_flat[self.shard_off:self.shard_off + self.shard_len]
        sumsq = shard.pow(2).sum()
        if self.world > 1:
            dist.all_reduce(sumsq, group=self.group)
        if self.norm_group is not None:
            dist.all_reduce(sumsq, group=self.norm_group)
        norm = sumsq.sqrt() / self.world
        scale = torch.clamp(max_norm / (norm + 1e-6), max=1.0) if max_norm > 0 else torch.ones_like(norm)
        g = shard * (scale / self.world)
        self.mu.mul_(b1).add_(g, alpha=1 - b1)
        self.nu.mul_(b2).addcmul_(g, g, value=1 - b2)
        if self.scalars is not None:  # lr and bias corrections read from device memory (recordable)
            off = self.count - self._step_idx
            h = self.scalars.f32_block(f"opt/{self.label}/hyper", 3, lambda s: (
                self.lr_at(s), 1.0 / (1 - b1 ** (s + off)), 1.0 / (1 - b2 ** (s + off))))
            upd = (self.mu * h[1]) / ((self.nu * h[2]).sqrt() + 1e-8) + self.cfg.weight_decay * self.master
            self.master.sub_(upd * h[0])
        else:
            upd = (self.mu / bc1) / ((self.nu / bc2).sqrt() + 1e-8) + self.cfg.weight_decay * self.master
            self.master.add_(upd, alpha=-lr)
        self.norm_out.copy_(norm.reshape(1))
        mine = self.master.to(torch.bfloat16)
        parts = [(self.work_flat, mine)]
        if self.work_lo_flat is not None:
            parts.append((self.work_lo_flat, (self.master - mine.float()).to(torch.bfloat16)))
        for dst, src in parts:
            if self.world > 1:
                dist.all_gather_into_tensor(dst, src, group=self.group)
            else:
                dst.copy_(src)

    def advance_replayed(self) -> None:
        """Host bookkeeping of a step whose launches ran from a recording (no Python ran for it)."""
        self.count += 1
        self._step_idx += 1
        self._seq += 3
        self.applied_learning_rate = self.lr_at(self._step_idx)
        self._full_stale = True

    def refresh_compute_fp32(self) -> None:
        """Local, no communication: rebuild every parameter's fp32 storage from the published split-precision
        working copy (`bf16(p) + bf16(p - bf16(p))`, about 16 mantissa bits) so that modules which read their
        parameters directly see this step's values. The exact fp32 masters stay with their owners
        (`refresh_full_fp32` gathers those for checkpoints and evaluation)."""
        assert self.work_lo_flat is not None, "needs the split-precision working copy (keep_lo=True)"
        self.full_fp32.copy_(self.work_flat)
        self.full_fp32.add_(self.work_lo_flat)

    def refresh_full_fp32(self) -> None:
        """All-gather the fp32 masters into the parameters' own storage (checkpoint / eval time)."""
        if self.world > 1:
            dist.all_gather_into_tensor(self.full_fp32, self.master, group=self.group)
        else:
            self.full_fp32.copy_(self.master)

    def _gather_flat(self, shard: Tensor) -> Tensor:
        if self.world == 1:
            return shard.clone()
        full = torch.empty(self.n, device=shard.device, dtype=shard.dtype)
        dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
        return full

    def gather_state(self) -> None:
        """Collective (every rank of the group): assemble the moments of all shards so that `state_dict` -
        which only the writing rank calls - can return them per parameter. Masters are gathered into the
        parameters' own storage at the same time."""
        self.refresh_full_fp32()
        self._gathered = (self._gather_flat(self.mu), self._gather_flat(self.nu))

    def state_dict(self) -> dict[str, Tensor]:
        """Per-parameter moments under the replicated optimizer's key grammar (`V.<key>/mu`, `.../nu`), so a
        checkpoint does not depend on how many ranks shared the optimizer state."""
        if self.world > 1:
            assert getattr(self, "_gathered", None) is not None, "call gather_state() on every rank before saving"
            mu, nu = self._gathered
            self._gathered = None
        else:
            mu, nu = self.mu, self.nu
        out: dict[str, Tensor] = {"count": torch.tensor(self.count, dtype=torch.int64)}
        for n, p, o in zip(self.names, self.params, self.offsets):
            key = n.replace("/", ".", 1)
            out[key + "/mu"] = mu[o:o + p.numel()].view_as(p).clone()
            out[key + "/nu"] = nu[o:o + p.numel()].view_as(p).clone()
        return out

    def load_state_dict(self, sd: dict[str, Tensor]) -> None:
        """Moments from the per-parameter entries; masters and working copies from the parameters' storage
        (restored before this call)."""
        self.count = int(sd["count"].item())
        sl = slice(self.shard_off, self.shard_off + self.shard_len)
        for suffix, dst in (("mu", self.mu), ("nu", self.nu)):
            full = torch.zeros(self.n, device=dst.device, dtype=torch.float32)
            for n, p, o in zip(self.names, self.params, self.offsets):
                v = sd.get(n.replace("/", ".", 1) + "/" + suffix)
                if v is not None:
                    full[o:o + p.numel()].copy_(v.reshape(-1))
            dst.copy_(full[sl])
        self.sync_from_parameters()

    def sync_from_parameters(self) -> None:
        """Adopt the values currently in the parameters' storage (after a restore or an in-place edit)."""
        if not self._grads_attached():  # an outside optimizer replaced the views: adopt values, re-home gradients
            self._attach_views()
            self.grad_flat.zero_()
        self.master.copy_(self.full_fp32[self.shard_off:self.shard_off + self.shard_len])
        self.work_flat.copy_(self.full_fp32)
        if self.work_lo_flat is not None:
            self.work_lo_flat.copy_(self.full_fp32 - self.work_flat.float())
