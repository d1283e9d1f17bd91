"""Tensor-parallel linears whose collective is inside the GEMM kernel (NVLink peer memory).

  * `gemm_reduce_scatter`: `Y = A B` where every rank holds a K-slice of the contraction (row-parallel
    linear, or the component contraction with `C` split over tp). The epilogue reduce-adds each output
    row block (fp32, TMA `cp.reduce.async.bulk`) straight into the buffer of the rank that owns those
    rows; after a peer barrier every rank holds its `[M / tp, N]` slice of the sum. No partial
    result ever exists in local HBM and no separate collective runs.
  * `allgather_gemm`: `Y = A_full B` where `A` is sharded by rows. A gather warp in every CTA pulls
    remote 128-row blocks over NVLink into the local full-size `A` buffer - each block exactly once
    per GPU - and releases it with a flag; the TMA producer waits (bounded) on the flag of the block it
    is about to load, and tiles are rasterised so the local blocks are consumed first while remote
    ones stream in. tcgen05 is fed by local, non-multicast TMA only.
  * `allgather_weight_gemm`: `Y = X W_full` where the weight (`V [d_in, C]`, row-sharded over the
    fsdp ranks) lives 1/W per GPU. A few CTAs bulk-copy the peers' 64-row K slabs into the local
    full-size buffer; the TMA producer walks K starting at this rank's own slab and waits (bounded)
    on a slab's flag only the first time it needs it. Any epilogue works, so this is how the masked
    `x V` product consumes component shards without a separate all-gather.
All have NCCL twins (`*_nccl`) that serve as oracle and as the measured baseline.

Reference behaviour covered: the tp all-reduce / reduce-scatter of row-linear outputs and of the
`(...)@U` contraction over `C / tp`, and the all-gather of sequence-parallel activations
(param_decomp/core/decomposed_linear.py:142-175, core/linear_plan.py:199-225,
core/placement.py:1040-1048,1552-1566).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import Tensor

from param_decomp_b200.ops import native as nv
from param_decomp_b200.parallel.sharded_optim import PdPeerPtrs, _peer_table, symmetric_empty


@dataclass
class TPWorkspace:
    """Symmetric buffers of one tp group: an fp32 reduce-scatter target, a bf16 gather source, the
    barrier flags, and the sequence counters that make flags single-use without clearing them."""

    group: object
    max_rows: int  # full (un-sharded) row count
    max_cols: int
    device: torch.device
    wait_limit_s: float = 2.0
    _bar_seq: int = 0
    _ag_seq: int = 0

    def __post_init__(self) -> None:
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        rows_per = self.max_rows // self.world
        self.rs_buf, self.rs_ptrs = symmetric_empty(rows_per * self.max_cols, torch.float32, self.device, self.group)
        self.ag_buf, self.ag_ptrs = symmetric_empty(rows_per * self.max_cols, torch.bfloat16, self.device, self.group)
        self.flags, self.flag_ptrs = symmetric_empty(8, torch.int32, self.device, self.group)
        self.flags.zero_()
        self.ag_full = torch.empty(self.max_rows * self.max_cols, device=self.device, dtype=torch.bfloat16)
        self.ag_flags = torch.zeros(max((self.max_rows + 127) // 128, 64), device=self.device, dtype=torch.int32)
        self.w_buf = self.w_ptrs = self.w_full = None
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def barrier(self) -> None:
        """Stream-ordered cross-GPU barrier (bounded wait, status word on time-out)."""
        self._bar_seq += 1
        lib = nv.lib()
        lib.pd_peer_barrier.argtypes = [C.POINTER(PdPeerPtrs), C.c_int, C.c_int, C.c_uint, C.c_void_p, C.c_double,
                                        C.c_void_p]
        table = _peer_table(self.flag_ptrs)
        rc = lib.pd_peer_barrier(C.byref(table), self.rank, self.world, self._bar_seq, nv.status_word().data_ptr(),
                                 self.wait_limit_s, nv.current_stream_ptr())
        nv.count_launch()
        if rc != 0:
            raise nv.NativeError("pd_peer_barrier failed to launch")


def gemm_reduce_scatter(ws: TPWorkspace, a: Tensor, b: Tensor, *, b_mn: bool = False, a1: Tensor | None = None,
                        b1: Tensor | None = None, b1_mn: bool = False) -> Tensor:
    """`a [M, K_local]`, `b` its matching K-slice; returns this rank's fp32 `[M / tp, N]` rows of the sum."""
    M = a.shape[0]
    N = b.shape[-1] if b_mn else b.shape[0]
    assert M % (128 * ws.world) == 0, "row count must tile 128 x tp"
    rows = M // ws.world
    out = ws.rs_buf[: rows * N].view(rows, N)
    out.zero_()
    ws.barrier()  # every rank's target is zero before anyone adds into it
    nv.gemm(a, b, _RSOut(out, M, N), b_mn=b_mn, a1=a1, b1=b1, b1_mn=b1_mn, rs=(ws.rs_ptrs, rows))
    ws.barrier()  # all partial sums have landed
    return out


class _RSOut:
    """Shape carrier: the kernel's output is logically `[M, N]` but physically the owners' slices."""

    def __init__(self, local: Tensor, M: int, N: int) -> None:
        self.local, self.shape, self.dtype = local, (M, N), local.dtype

    def dim(self) -> int:
        return 2

    def stride(self, i: int) -> int:
        return self.local.stride(i)

    def data_ptr(self) -> int:
        return self.local.data_ptr()


def allgather_gemm(ws: TPWorkspace, a_local: Tensor, b: Tensor, out: Tensor, *, b_mn: bool = False, **kw) -> Tensor:
    """`a_local [M / tp, K]` bf16 (this rank's rows); `out [M, N] = all_gather(a) @ b`."""
    rows, K = a_local.shape
    M = rows * ws.world
    assert rows % 128 == 0 and K % 8 == 0
    src = ws.ag_buf[: rows * K].view(rows, K)
    src.copy_(a_local)
    full = ws.ag_full[: M * K].view(M, K)
    full[ws.rank * rows:(ws.rank + 1) * rows].copy_(a_local)
    ws.barrier()  # every rank's shard is published before anyone pulls it
    ws._ag_seq += 1
    nv.gemm(full, b, out, b_mn=b_mn, ag=(ws.ag_ptrs, ws.rank, rows, ws.ag_flags, ws._ag_seq), **kw)
    ws.barrier()  # nobody overwrites its shard while a peer may still be reading it
    return out


def allgather_weight_gemm(ws: TPWorkspace, x: Tensor, w_local: Tensor, out: Tensor, publish: bool = True, **kw) -> Tensor:
    """`x [M, K]`, `w_local [K / W, N]` bf16 (this rank's K rows of the MN-major weight);
    `out = x @ all_gather(w_local)`; keyword arguments select the epilogue (e.g. the mask epilogue).
    `publish=False` re-uses the shard already sitting in the symmetric buffer (same weights, next draw)."""
    kr, N = w_local.shape
    K = kr * ws.world
    assert kr % 64 == 0 and N % 8 == 0 and x.shape[1] == K
    if ws.w_buf is None or ws.w_buf.numel() < kr * N:
        ws.w_buf, ws.w_ptrs = symmetric_empty(kr * N, torch.bfloat16, ws.device, ws.group)
        ws.w_full = torch.empty(K * N, device=ws.device, dtype=torch.bfloat16)
    full = ws.w_full[: K * N].view(K, N)
    if publish:
        ws.w_buf[: kr * N].view(kr, N).copy_(w_local)
        full[ws.rank * kr:(ws.rank + 1) * kr].copy_(w_local)
        ws.barrier()
    ws._ag_seq += 1
    nv.gemm(x, full, out, b_mn=True, ag_b=(ws.w_ptrs, ws.rank, kr, ws.ag_flags, ws._ag_seq), **kw)
    return out


def allgather_weight_gemm_nccl(group, x: Tensor, w_local: Tensor, out: Tensor, **kw) -> Tensor:
    world = dist.get_world_size(group)
    full = torch.empty(w_local.shape[0] * world, w_local.shape[1], device=x.device, dtype=w_local.dtype)
    dist.all_gather_into_tensor(full, w_local.contiguous(), group=group)
    nv.gemm(x, full, out, b_mn=True, **kw)
    return out


# ---- NCCL twins (oracle + baseline) ----------------------------------------------------------------


def gemm_reduce_scatter_nccl(group, a: Tensor, b: Tensor, b_mn: bool = False) -> Tensor:
    world = dist.get_world_size(group)
    M = a.shape[0]
    N = b.shape[-1] if b_mn else b.shape[0]
    full = torch.empty(M, N, device=a.device, dtype=torch.float32)
    nv.gemm(a, b, full, b_mn=b_mn)
    out = torch.empty(M // world, N, device=a.device, dtype=torch.float32)
    dist.reduce_scatter_tensor(out, full, group=group)
    return out


def allgather_gemm_nccl(group, a_local: Tensor, b: Tensor, out: Tensor, b_mn: bool = False) -> Tensor:
    world = dist.get_world_size(group)
    full = torch.empty(a_local.shape[0] * world, a_local.shape[1], device=a_local.device, dtype=a_local.dtype)
    dist.all_gather_into_tensor(full, a_local.contiguous(), group=group)
    nv.gemm(full, b, out, b_mn=b_mn)
    return out
