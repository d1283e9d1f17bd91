// Compute fused with collectives over NVLink peer memory (plain P2P loads/stores, no multimem,
// no TMA from peers): ranks are processes, one per GPU; every pointer table below holds the
// addresses at which THIS process has mapped each rank's symmetric buffer.
//
//   pd_rs_adamw_ag   reduce-scatter of the fp32 gradient buffer + global-norm clip + AdamW on the
//                    owned master shard + all-gather of the updated bf16 working copy, one
//                    cooperative kernel per rank:
//        barrier(peers' gradients complete)
//        gsum[i]   = sum_r grad_r[shard + i]          (P2P loads)      partial sum of squares
//        barrier(partial norms published)
//        scale     = clip(sqrt(sum_r sumsq_r) / W)                     (P2P loads of W scalars)
//        p,m,v    <- AdamW(p, m, v, gsum / W * scale)                  (local fp32 masters)
//        work_r[shard + i] = bf16(p[i])  for every rank r              (P2P stores)
//        barrier(working copies complete)
//   pd_peer_barrier  the barrier alone (used by tests and by phases that are separate launches).
//
// Cross-GPU barrier: each rank bumps a sequence number and stores it into slot [my_rank] of every
// peer's flag array (st.release.sys after __threadfence_system), then polls its own array until all
// slots reach the sequence (ld.acquire.sys). The poll is bounded by %globaltimer; on time-out the
// kernel writes kTimeoutPeerFlag to *status, skips nothing else (all phases still run to completion
// so no block is left waiting inside the grid), and returns. Inside the grid, phases are separated
// by cooperative grid syncs, so the kernel must be launched cooperatively with a co-resident grid.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int kMaxRanks = 8;
constexpr int kThreads = 256;

struct PeerTable {
  void* ptr[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One thread. flags[r] point at rank r's flag array (kMaxRanks words each).
__device__ bool peer_barrier(const PeerTable& flags, int rank, int world, unsigned int seq, int* status,
                             unsigned long long limit_ns) {
  __threadfence_system();
  for (int r = 0; r < world; ++r)
    st_release_sys(static_cast<unsigned int*>(flags.ptr[r]) + rank, seq);
  const unsigned int* mine = static_cast<const unsigned int*>(flags.ptr[rank]);
  const unsigned long long t0 = pd::globaltimer_ns();
  for (int r = 0; r < world; ++r) {
    // signed distance so that a wrapped counter still compares correctly
    while (static_cast<int>(ld_acquire_sys(mine + r) - seq) < 0) {
      if (pd::globaltimer_ns() - t0 > limit_ns) {
        if (status) atomicCAS(status, 0, pd::kTimeoutPeerFlag);
        return false;
      }
    }
  }
  return true;
}

__global__ void peer_barrier_kernel(PeerTable flags, int rank, int world, unsigned int seq, int* status,
                                    unsigned long long limit_ns) {
  if (threadIdx.x == 0 && blockIdx.x == 0) peer_barrier(flags, rank, world, seq, status, limit_ns);
}

struct RsAdamwArgs {
  PeerTable grads;   // fp32 [n_total] per rank
  PeerTable work;    // bf16 [n_total] per rank: hi part, bf16(p)
  PeerTable work_lo; // bf16 [n_total] per rank: lo part, bf16(p - hi); entries may be null
  PeerTable flags;   // u32 [kMaxRanks] per rank
  PeerTable norms;   // fp32 [1] per rank: partial sum of squares of the rank's reduced shard
  float* p; float* m; float* v;  // local master shard [shard_len]
  long long shard_off, shard_len;
  int rank, world;
  unsigned int seq;  // three sequence numbers seq, seq+1, seq+2 are consumed
  float lr, b1, b2, eps, wd, inv_bc1, inv_bc2, max_norm;
  float* norm_out;   // local fp32: the global gradient norm (for logging)
  int* status;
  unsigned long long limit_ns;
  // Recorded launches (CUDA graphs): when set, {lr, 1/bc1, 1/bc2} and the first of the three sequence
  // numbers are read from device memory at run time, so one recording serves every step.
  const float* hyper_dev;
  const unsigned int* seq_dev;
};

__global__ void __launch_bounds__(kThreads) rs_adamw_ag_kernel(RsAdamwArgs a) {
  cg::grid_group grid = cg::this_grid();
  if (a.hyper_dev != nullptr) {
    a.lr = a.hyper_dev[0];
    a.inv_bc1 = a.hyper_dev[1];
    a.inv_bc2 = a.hyper_dev[2];
  }
  if (a.seq_dev != nullptr) a.seq = *a.seq_dev;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  float* my_norm = static_cast<float*>(a.norms.ptr[a.rank]);

  if (tid == 0) {
    *my_norm = 0.f;
    peer_barrier(a.flags, a.rank, a.world, a.seq, a.status, a.limit_ns);  // everyone's grads are final
  }
  grid.sync();

  // ---- reduce-scatter: sum my shard over all ranks, keep it in my own gradient buffer ----
  float* my_grad = static_cast<float*>(a.grads.ptr[a.rank]) + a.shard_off;
  float acc = 0.f;
  const long long n4 = a.shard_len / 4;
  for (long long i = tid; i < n4; i += nthreads) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < a.world; ++r) {
      const float4 g = *reinterpret_cast<const float4*>(static_cast<const float*>(a.grads.ptr[r]) + a.shard_off + 4 * i);
      s.x += g.x; s.y += g.y; s.z += g.z; s.w += g.w;
    }
    *reinterpret_cast<float4*>(my_grad + 4 * i) = s;
    acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
  }
  for (long long i = 4 * n4 + tid; i < a.shard_len; i += nthreads) {
    float s = 0.f;
    for (int r = 0; r < a.world; ++r) s += static_cast<const float*>(a.grads.ptr[r])[a.shard_off + i];
    my_grad[i] = s;
    acc += s * s;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) atomicAdd(my_norm, acc);
  grid.sync();
  if (tid == 0) peer_barrier(a.flags, a.rank, a.world, a.seq + 1, a.status, a.limit_ns);  // norms published
  grid.sync();

  // ---- global norm of the MEAN gradient, clip factor ----
  float total = 0.f;
  for (int r = 0; r < a.world; ++r) total += *static_cast<const volatile float*>(a.norms.ptr[r]);
  const float inv_w = 1.f / a.world;
  const float norm = sqrtf(total) * inv_w;
  const float gs = (a.max_norm > 0.f ? fminf(a.max_norm / (norm + 1e-6f), 1.f) : 1.f) * inv_w;
  if (tid == 0 && a.norm_out) *a.norm_out = norm;

  // ---- AdamW on the owned shard, updated weights broadcast in bf16 to every rank ----
  const long long n8 = a.shard_len / 8;
  for (long long i = tid; i < n8; i += nthreads) {
    float pv[8], gv[8], mv[8], vv[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      *reinterpret_cast<float4*>(pv + 4 * h) = *reinterpret_cast<const float4*>(a.p + 8 * i + 4 * h);
      *reinterpret_cast<float4*>(gv + 4 * h) = *reinterpret_cast<const float4*>(my_grad + 8 * i + 4 * h);
      *reinterpret_cast<float4*>(mv + 4 * h) = *reinterpret_cast<const float4*>(a.m + 8 * i + 4 * h);
      *reinterpret_cast<float4*>(vv + 4 * h) = *reinterpret_cast<const float4*>(a.v + 8 * i + 4 * h);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float g = gv[k] * gs;
      mv[k] = a.b1 * mv[k] + (1.f - a.b1) * g;
      vv[k] = a.b2 * vv[k] + (1.f - a.b2) * g * g;
      pv[k] -= a.lr * ((mv[k] * a.inv_bc1) / (sqrtf(vv[k] * a.inv_bc2) + a.eps) + a.wd * pv[k]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      *reinterpret_cast<float4*>(a.p + 8 * i + 4 * h) = *reinterpret_cast<float4*>(pv + 4 * h);
      *reinterpret_cast<float4*>(a.m + 8 * i + 4 * h) = *reinterpret_cast<float4*>(mv + 4 * h);
      *reinterpret_cast<float4*>(a.v + 8 * i + 4 * h) = *reinterpret_cast<float4*>(vv + 4 * h);
    }
    __nv_bfloat162 o[4] = {__floats2bfloat162_rn(pv[0], pv[1]), __floats2bfloat162_rn(pv[2], pv[3]),
                           __floats2bfloat162_rn(pv[4], pv[5]), __floats2bfloat162_rn(pv[6], pv[7])};
    const uint4 packed = *reinterpret_cast<uint4*>(o);
    for (int r = 0; r < a.world; ++r)
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.work.ptr[r]) + a.shard_off + 8 * i) = packed;
    if (a.work_lo.ptr[0] != nullptr) {
      __nv_bfloat162 l[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 h = __bfloat1622float2(o[k]);
        l[k] = __floats2bfloat162_rn(pv[2 * k] - h.x, pv[2 * k + 1] - h.y);
      }
      const uint4 packed_lo = *reinterpret_cast<uint4*>(l);
      for (int r = 0; r < a.world; ++r)
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.work_lo.ptr[r]) + a.shard_off + 8 * i) = packed_lo;
    }
  }
  for (long long i = 8 * n8 + tid; i < a.shard_len; i += nthreads) {
    const float g = my_grad[i] * gs;
    const float mm = a.b1 * a.m[i] + (1.f - a.b1) * g, vv = a.b2 * a.v[i] + (1.f - a.b2) * g * g;
    const float pp = a.p[i] - a.lr * ((mm * a.inv_bc1) / (sqrtf(vv * a.inv_bc2) + a.eps) + a.wd * a.p[i]);
    a.p[i] = pp; a.m[i] = mm; a.v[i] = vv;
    const __nv_bfloat16 hi = __float2bfloat16(pp);
    for (int r = 0; r < a.world; ++r) {
      static_cast<__nv_bfloat16*>(a.work.ptr[r])[a.shard_off + i] = hi;
      if (a.work_lo.ptr[0] != nullptr)
        static_cast<__nv_bfloat16*>(a.work_lo.ptr[r])[a.shard_off + i] = __float2bfloat16(pp - __bfloat162float(hi));
    }
  }
  grid.sync();
  if (tid == 0) peer_barrier(a.flags, a.rank, a.world, a.seq + 2, a.status, a.limit_ns);  // copies complete
}

}  // namespace


// ---------------------------------------------------------------------------------------------
// Expert-parallel dispatch / combine: rows travel to their owner by direct peer stores.
//   row j of `src` (optionally row `gather[j]`: the router's permutation is applied on the fly)
//   goes to rank dest_rank[j], row dest_row[j] of that rank's receive buffer (16-byte vectors over
//   NVLink). Up to two payloads with the same routing move in one launch (activations and their
//   mask rows). After its rows are stored and fenced, each block takes a ticket; the last block of
//   the grid signals every peer and waits (bounded) for every peer's signal, so when the kernel
//   completes the receive buffers of THIS rank are complete too. No block waits on another block,
//   so the launch needs no co-residency.
// Replaces the all-to-all-free "EP by activation slicing" of the reference
// (param_decomp/routed/experts.py:28-40,864-885) on the all-to-all path.
// ---------------------------------------------------------------------------------------------
struct PdPeerPtrs {
  void* ptr[kMaxRanks];
};

struct ScatterArgs {
  const uint4* src[2];
  int vecs[2];             // 16-byte vectors per row of each payload (0 = payload unused)
  PeerTable dst[2];        // per-rank receive buffers of each payload
  const long long* gather; // [n] source row of job j, or null for j
  const int* dest_rank;    // [n]
  const long long* dest_row;  // [n]
  long long n;
  PeerTable flags;
  int rank, world;
  unsigned int seq;
  unsigned int* ticket;    // local counter, zero between launches
  int* status;
  unsigned long long limit_ns;
};

__global__ void __launch_bounds__(256) ep_scatter_rows_kernel(ScatterArgs a) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (long long j = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5); j < a.n;
       j += static_cast<long long>(gridDim.x) * warps_per_block) {
    const long long srow = a.gather ? a.gather[j] : j;
    const int r = a.dest_rank[j];
    const long long drow = a.dest_row[j];
    if (r < 0 || r >= a.world) continue;  // job not sent anywhere
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      const int vecs = a.vecs[p];
      if (vecs == 0) continue;
      const uint4* s = a.src[p] + srow * vecs;
      uint4* d = static_cast<uint4*>(a.dst[p].ptr[r]) + drow * vecs;
      for (int v = lane; v < vecs; v += 32) d[v] = s[v];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(a.ticket, 1u);
    if (t == gridDim.x - 1) {  // every block of this rank has stored and fenced its rows
      *a.ticket = 0u;
      peer_barrier(a.flags, a.rank, a.world, a.seq, a.status, a.limit_ns);
    }
  }
}

struct PdEpScatterCall {
  const void* src[2];
  int row_bytes[2];
  PdPeerPtrs dst[2];
  const long long* gather;
  const int* dest_rank;
  const long long* dest_row;
  long long n;
  PdPeerPtrs flags;
  int rank, world;
  unsigned int seq;
  unsigned int* ticket;
  int* status;
  double limit_s;
};

extern "C" int pd_peer_barrier(const PdPeerPtrs* flags, int rank, int world, unsigned int seq, int* status,
                               double limit_s, void* stream) {
  if (world < 1 || world > kMaxRanks) return pd::kBadArgument;
  PeerTable t;
  for (int r = 0; r < kMaxRanks; ++r) t.ptr[r] = flags->ptr[r];
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      t, rank, world, seq, status, static_cast<unsigned long long>(limit_s * 1e9));
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

struct PdRsAdamwCall {
  PdPeerPtrs grads, work, work_lo, flags, norms;
  float* p; float* m; float* v;
  long long shard_off, shard_len;
  int rank, world;
  unsigned int seq;
  float lr, b1, b2, eps, wd, bc1, bc2, max_norm;
  float* norm_out;
  int* status;
  double limit_s;
  const float* hyper_dev;         // {lr, 1/bc1, 1/bc2} in device memory, or null to use the fields above
  const unsigned int* seq_dev;    // first sequence number in device memory, or null to use `seq`
};

extern "C" int pd_rs_adamw_ag(const PdRsAdamwCall* c, void* stream) {
  if (c->world < 1 || c->world > kMaxRanks || c->shard_len <= 0) return pd::kBadArgument;
  if ((c->shard_off % 8) != 0) return pd::kBadArgument;  // 16-byte bf16 stores and float4 loads
  RsAdamwArgs a;
  for (int r = 0; r < kMaxRanks; ++r) {
    a.grads.ptr[r] = c->grads.ptr[r]; a.work.ptr[r] = c->work.ptr[r]; a.work_lo.ptr[r] = c->work_lo.ptr[r];
    a.flags.ptr[r] = c->flags.ptr[r]; a.norms.ptr[r] = c->norms.ptr[r];
  }
  a.p = c->p; a.m = c->m; a.v = c->v;
  a.shard_off = c->shard_off; a.shard_len = c->shard_len;
  a.rank = c->rank; a.world = c->world; a.seq = c->seq;
  a.lr = c->lr; a.b1 = c->b1; a.b2 = c->b2; a.eps = c->eps; a.wd = c->wd;
  a.inv_bc1 = 1.f / c->bc1; a.inv_bc2 = 1.f / c->bc2; a.max_norm = c->max_norm;
  a.norm_out = c->norm_out; a.status = c->status;
  a.limit_ns = static_cast<unsigned long long>(c->limit_s * 1e9);
  a.hyper_dev = c->hyper_dev; a.seq_dev = c->seq_dev;
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rs_adamw_ag_kernel, kThreads, 0);
  if (per_sm < 1) return 2;
  int blocks = sms * (per_sm > 4 ? 4 : per_sm);  // co-resident by construction (cooperative launch checks it)
  void* params[] = {&a};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(rs_adamw_ag_kernel), dim3(blocks),
                                              dim3(kThreads), params, 0, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : 100 + static_cast<int>(e);
}

extern "C" int pd_ep_scatter_rows(const PdEpScatterCall* c, void* stream) {
  if (c->world < 1 || c->world > kMaxRanks || c->n < 0 || c->ticket == nullptr) return pd::kBadArgument;
  ScatterArgs a;
  for (int p = 0; p < 2; ++p) {
    if (c->row_bytes[p] % 16 != 0 || (reinterpret_cast<uintptr_t>(c->src[p]) & 15)) return pd::kBadArgument;
    a.src[p] = static_cast<const uint4*>(c->src[p]);
    a.vecs[p] = c->src[p] ? c->row_bytes[p] / 16 : 0;
    for (int r = 0; r < kMaxRanks; ++r) a.dst[p].ptr[r] = c->dst[p].ptr[r];
  }
  for (int r = 0; r < kMaxRanks; ++r) a.flags.ptr[r] = c->flags.ptr[r];
  a.gather = c->gather; a.dest_rank = c->dest_rank; a.dest_row = c->dest_row; a.n = c->n;
  a.rank = c->rank; a.world = c->world; a.seq = c->seq; a.ticket = c->ticket; a.status = c->status;
  a.limit_ns = static_cast<unsigned long long>(c->limit_s * 1e9);
  long long blocks = (c->n + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  ep_scatter_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}
