// Flash attention for sm_100a: QK^T and PV (and the five backward products) on tcgen05 with the
// accumulators in TMEM, operands staged by non-multicast TMA into 128-byte-swizzled shared memory.
//
// Layout: q [B, T, H, hd], k / v [B, T, Hkv, hd] (bf16, hd contiguous, hd = 64 or 128), out like q;
// T a multiple of 128. Causal and/or document-segmented (block-diagonal) masks; grouped-query
// attention by head // (H / Hkv). The log-sum-exp is kept per (b, h, t) in base-2 units of the
// scaled scores for the backward.
//
// Forward, one CTA per (128 query rows, head, batch); warps 0-3 = softmax (one query row per
// thread = one TMEM lane), warp 4 = TMA producer, warp 5 = MMA issuer:
//     S = Q K_j^T  (TMEM)  ->  online softmax in registers  ->  P_j (bf16, shared)  ->  O_j = P_j V_j (TMEM)
// O_j is read back and accumulated in registers with the usual running-max correction, so nothing
// in TMEM ever has to be rescaled. With hd = 64 a CTA takes 256 TMEM columns and 112 KB of shared
// memory, so two CTAs share an SM and overlap each other's softmax and tensor phases.
//
// Backward, one CTA per (128 key rows, kv head, batch), looping over the query heads of the group
// and the query tiles that see this key tile:
//     S = Q_i K_j^T, dP = dO_i V_j^T (TMEM) -> P = exp2(S - L), dS = P * (dP - D) * scale (bf16, shared)
//     dV += P^T dO_i, dK += dS^T Q_i (TMEM, across the whole loop), dQ_i = dS K_j (TMEM -> fp32 atomics)
// P and dS are written once, row-major in the key index, and read both as a K-major operand (dQ) and
// as an MN-major operand (the transposed products), which the descriptor's major bits allow.
//
// Every wait is bounded; on a time-out the status word is set and all roles leave.
//
// Replaces the reference's cuDNN fused attention and its tokamax Mosaic alternative
// (param_decomp/attention.py:116-137,148-245).
#include <algorithm>

#include "attention_common.cuh"

namespace {

using namespace pd_attn;

struct AttnArgs {
  int B, T, H, Hkv;
  int causal;
  float scale_log2;       // log2(e) / sqrt(hd)
  float scale;            // 1 / sqrt(hd)
  const int* segment_ids; // [B, T] or null
  __nv_bfloat16* out;     // [B, T, H, hd]
  float* lse;             // [B, H, T] base-2 log-sum-exp of the scaled scores
  // backward only
  const float* delta;     // [B, H, T] rowsum(dO * O)
  float* dq_accum;        // [B, T, H, hd] fp32, zero on entry
  __nv_bfloat16* dk;      // [B, T, Hkv, hd]
  __nv_bfloat16* dv;
  int* status;
};

template <int HD>
struct FwdPlan {
  static constexpr int kQBytes = kTile * HD * 2;
  static constexpr int kKVBytes = kTile * HD * 2;
  static constexpr int kPBytes = kTile * kTile * 2;
  static constexpr int kStages = 2;                 // K ring
  static constexpr int kVStages = HD == 64 ? 1 : 2;  // one V buffer keeps a CTA under half an SM's shared memory
  static constexpr int kTotal = kQBytes + (kStages + kVStages) * kKVBytes + kPBytes + 1024 /*align*/ + 1024 /*barriers, seg ids*/;
  static constexpr uint32_t kTmemCols = 256;  // S: 128 columns, O: HD columns at column 128
};

// ------------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(kFwdThreads, HD == 64 ? 2 : 1) attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                const __grid_constant__ CUtensorMap tmK,
                                                                const __grid_constant__ CUtensorMap tmV,
                                                                const AttnArgs args) {
  using Plan = FwdPlan<HD>;
  constexpr int kStages = Plan::kStages;
  constexpr int kVStages = Plan::kVStages;
  constexpr int kKB = HD / 64;  // 64-wide K blocks of the head dimension
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sm_q = base;
  const uint32_t sm_k = sm_q + Plan::kQBytes;
  const uint32_t sm_v = sm_k + kStages * Plan::kKVBytes;
  const uint32_t sm_p = sm_v + kVStages * Plan::kKVBytes;
  const uint32_t sm_bar = sm_p + Plan::kPBytes;
  // barriers: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full, p_full, o_full
  const uint32_t bar_q = sm_bar;
  const uint32_t bar_kf = bar_q + 8, bar_ke = bar_kf + 16, bar_vf = bar_ke + 16, bar_ve = bar_vf + 16;
  const uint32_t bar_s = bar_ve + 16, bar_p = bar_s + 8, bar_o = bar_p + 8;
  const uint32_t tmem_slot = bar_o + 8;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gbase + (tmem_slot - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + (tmem_slot + 4 - base));
  int* seg_k = reinterpret_cast<int*>(gbase + (sm_bar + 256 - base));  // [128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query tiles first so the causal triangle packs well
  const int n_qt = args.T / kTile;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (args.H / args.Hkv);
  const int n_kv = args.causal ? qt + 1 : n_qt;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_kf + 8 * s, 1);
      mbar_init(bar_ke + 8 * s, 1);
      mbar_init(bar_vf + 8 * s, 1);
      mbar_init(bar_ve + 8 * s, 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_p, kSoftmaxThreads);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, Plan::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_s = *tmem_slot_ptr;
  const uint32_t tmem_o = tmem_s + 128;

  if (warp == 4) {
    // ---------------- TMA producer (whole warp walks the loop, one elected lane issues) ----------------
    if (elect_one_sync()) {
      mbar_expect_tx(bar_q, Plan::kQBytes);
      for (int c = 0; c < kKB; ++c) tma_load_3d(sm_q + c * (kTile * 128), &tmQ, bar_q, h * HD + 64 * c, qt * kTile, b);
    }
    for (int j = 0; j < n_kv; ++j) {
      const int st = j % kStages;
      const uint32_t ph = static_cast<uint32_t>((j / kStages) & 1);
      if (!mbar_wait_warp(bar_ke + 8 * st, ph ^ 1, abort_flag)) {
        if (lane == 0) atomicCAS(args.status, 0, kTimeoutProducer);
        break;
      }
      if (elect_one_sync()) {
        mbar_expect_tx(bar_kf + 8 * st, Plan::kKVBytes);
        for (int c = 0; c < kKB; ++c)
          tma_load_3d(sm_k + st * Plan::kKVBytes + c * (kTile * 128), &tmK, bar_kf + 8 * st, hk * HD + 64 * c,
                      j * kTile, b);
      }
      const int vs = j % kVStages;
      const uint32_t vph = static_cast<uint32_t>((j / kVStages) & 1);
      if (!mbar_wait_warp(bar_ve + 8 * vs, vph ^ 1, abort_flag)) {
        if (lane == 0) atomicCAS(args.status, 0, kTimeoutProducer);
        break;
      }
      if (elect_one_sync()) {
        mbar_expect_tx(bar_vf + 8 * vs, Plan::kKVBytes);
        for (int c = 0; c < kKB; ++c)
          tma_load_3d(sm_v + vs * Plan::kKVBytes + c * (kTile * 128), &tmV, bar_vf + 8 * vs, hk * HD + 64 * c,
                      j * kTile, b);
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer (whole warp walks the loop, one elected lane issues) ----------------
    {
      constexpr uint32_t idesc_s = make_idesc_bf16(kTile, kTile, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(kTile, HD, 0, 1);
      bool ok = mbar_wait_warp(bar_q, 0, abort_flag);
      auto issue_s = [&](int j) {
        const int st = j % kStages;
        if (!mbar_wait_warp(bar_kf + 8 * st, static_cast<uint32_t>((j / kStages) & 1), abort_flag)) return false;
        tc_fence_after();
        if (elect_one_sync()) {
#pragma unroll
          for (int c = 0; c < kKB; ++c) {
            const uint64_t ad = make_smem_desc(sm_q + c * (kTile * 128), 16, 1024);
            const uint64_t bd = make_smem_desc(sm_k + st * Plan::kKVBytes + c * (kTile * 128), 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_bf16(tmem_s, ad + k * 2, bd + k * 2, idesc_s, (c > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(bar_ke + 8 * st);
          umma_commit(bar_s);
        }
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        // P_j is in shared memory; the softmax warps are also done with S_j and O_{j-1}
        if (!mbar_wait_warp(bar_p, static_cast<uint32_t>(j & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (j + 1 < n_kv && !issue_s(j + 1)) { ok = false; break; }
        const int vs = j % kVStages;
        if (!mbar_wait_warp(bar_vf + 8 * vs, static_cast<uint32_t>((j / kVStages) & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (elect_one_sync()) {
          const uint64_t vd = make_smem_desc(sm_v + vs * Plan::kKVBytes, kTile * 128, 1024);
#pragma unroll
          for (int c = 0; c < 2; ++c) {  // two 64-wide blocks of the key index
            const uint64_t pd_ = make_smem_desc(sm_p + c * (kTile * 128), 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16(tmem_o, pd_ + k * 2, vd + (c * 4 + k) * (2048 >> 4), idesc_o, (c > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(bar_ve + 8 * vs);
          umma_commit(bar_o);
        }
      }
      if (!ok && lane == 0) atomicCAS(args.status, 0, kTimeoutMma);
    }
  } else {
    // ---------------- softmax + output (one query row per thread) ----------------
    const int row = threadIdx.x;  // 0..127 = TMEM lane
    const int q_idx = qt * kTile + row;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int seg_q = args.segment_ids ? args.segment_ids[b * args.T + q_idx] : 0;
    float m_run = -INFINITY, l_run = 0.0f;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      if (args.segment_ids) {
        named_barrier_softmax();  // everyone is done with the previous tile's ids
        seg_k[row] = args.segment_ids[b * args.T + j * kTile + row];
        named_barrier_softmax();
      }
      if (!mbar_wait(bar_s, static_cast<uint32_t>(j & 1), abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = args.causal && j == qt;
      // pass 1: row maximum of the scaled, masked scores
      float m_new = m_run;
      uint32_t r[32];
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        tmem_ld_32x32(tmem_s + lane_base + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int col = c * 32 + i;
          const bool keep = (!diag || col <= row) && (!args.segment_ids || seg_k[col] == seg_q);
          if (keep) m_new = fmaxf(m_new, __uint_as_float(r[i]) * args.scale_log2);
        }
      }
      // O_{j-1} (computed against the previous maximum) joins the register accumulator first
      if (j > 0) {
        if (!mbar_wait(bar_o, static_cast<uint32_t>((j - 1) & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          tmem_ld_32x32(tmem_o + lane_base + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(r[i]);
        }
      }
      const float alpha = (m_run == -INFINITY) ? 0.0f : fast_exp2(m_run - m_new);
      l_run *= alpha;
#pragma unroll
      for (int i = 0; i < HD; ++i) o[i] *= alpha;
      m_run = m_new;
      // pass 2: probabilities -> shared memory (bf16, swizzled K-major blocks of 64 keys)
      float l_add = 0.0f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        tmem_ld_32x32(tmem_s + lane_base + c * 32, r);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = c * 32 + i + e;
            const bool keep = (!diag || col <= row) && (!args.segment_ids || seg_k[col] == seg_q);
            p2[e] = keep ? fast_exp2(__uint_as_float(r[i + e]) * args.scale_log2 - m_new) : 0.0f;
          }
          packed[i >> 1] = pack_bf16(p2[0], p2[1]);
          // the sum uses the rounded values the tensor core will see
          const __nv_bfloat162 hb = *reinterpret_cast<__nv_bfloat162*>(&packed[i >> 1]);
          const float2 f = __bfloat1622float2(hb);
          l_add += f.x + f.y;
        }
        const uint32_t blk = sm_p + (c >> 1) * (kTile * 128);
#pragma unroll
        for (int g = 0; g < 4; ++g)
          st_shared_v4(blk + swz(row, (c & 1) * 4 + g),
                       make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]));
      }
      l_run += l_add;
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(bar_p);
    }
    if (ok && n_kv > 0) {
      if (!mbar_wait(bar_o, static_cast<uint32_t>((n_kv - 1) & 1), abort_flag)) ok = false;
      if (ok) {
        tc_fence_after();
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          tmem_ld_32x32(tmem_o + lane_base + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] += __uint_as_float(r[i]);
        }
        const float inv = 1.0f / l_run;
        __nv_bfloat16* dst = args.out + ((static_cast<long long>(b) * args.T + q_idx) * args.H + h) * HD;
#pragma unroll
        for (int g = 0; g < HD / 8; ++g) {
          uint4 v;
          v.x = pack_bf16(o[8 * g] * inv, o[8 * g + 1] * inv);
          v.y = pack_bf16(o[8 * g + 2] * inv, o[8 * g + 3] * inv);
          v.z = pack_bf16(o[8 * g + 4] * inv, o[8 * g + 5] * inv);
          v.w = pack_bf16(o[8 * g + 6] * inv, o[8 * g + 7] * inv);
          *reinterpret_cast<uint4*>(dst + 8 * g) = v;
        }
        if (args.lse) args.lse[(static_cast<long long>(b) * args.H + h) * args.T + q_idx] = m_run + log2f(l_run);
      }
    }
    if (!ok) atomicCAS(args.status, 0, kTimeoutEpilogue);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_s, Plan::kTmemCols);
}

// ------------------------------------------------------------------------------------------------
// backward
// ------------------------------------------------------------------------------------------------
// D[b, h, t] = sum_d dO * O  (one warp per row)
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int B, int T, int H, int hd) {
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (b, t, h)
  if (row >= static_cast<long long>(B) * T * H) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* po = o + row * hd;
  const __nv_bfloat16* pd = d_o + row * hd;
  float acc = 0.0f;
  for (int i = lane * 2; i < hd; i += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(po + i));
    const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pd + i));
    acc += a.x * g.x + a.y * g.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) {
    const long long bt = row / H;
    const int h = static_cast<int>(row % H);
    const long long b = bt / T, t = bt % T;
    delta[(b * H + h) * T + t] = acc;
  }
}

__global__ void attn_dq_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long n) {
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(acc + i);
    uint2 o;
    o.x = pack_bf16(v.x, v.y);
    o.y = pack_bf16(v.z, v.w);
    *reinterpret_cast<uint2*>(dq + i) = o;
  }
}

template <int HD>
struct BwdPlan {
  static constexpr int kTileBytes = kTile * HD * 2;  // K, V, Q or dO tile
  static constexpr int kStages = HD == 64 ? 2 : 1;   // Q / dO ring
  static constexpr int kPBytes = kTile * kTile * 2;
  static constexpr int kTotal = 2 * kTileBytes + 2 * kStages * kTileBytes + 2 * kPBytes + 1024 + 1024;
  // TMEM: [0,128) S, later dQ; [128,256) dP; [256,256+HD) dV; [256+HD, 256+2HD) dK
  static constexpr uint32_t kTmemCols = 512;
};

template <int HD>
__global__ void __launch_bounds__(kFwdThreads, 1) attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ,
                                                                   const __grid_constant__ CUtensorMap tmK,
                                                                   const __grid_constant__ CUtensorMap tmV,
                                                                   const __grid_constant__ CUtensorMap tmdO,
                                                                   const AttnArgs args) {
  using Plan = BwdPlan<HD>;
  constexpr int kStages = Plan::kStages;
  constexpr int kKB = HD / 64;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sm_k = base;
  const uint32_t sm_v = sm_k + Plan::kTileBytes;
  const uint32_t sm_q = sm_v + Plan::kTileBytes;
  const uint32_t sm_do = sm_q + kStages * Plan::kTileBytes;
  const uint32_t sm_p = sm_do + kStages * Plan::kTileBytes;
  const uint32_t sm_ds = sm_p + Plan::kPBytes;
  const uint32_t sm_bar = sm_ds + Plan::kPBytes;
  // barriers: kv_full, qdo_full[2], qdo_empty[2], sdp_full, pds_full, dq_full, dq_empty, final
  const uint32_t bar_kv = sm_bar;
  const uint32_t bar_qf = bar_kv + 8, bar_qe = bar_qf + 16;
  const uint32_t bar_sdp = bar_qe + 16, bar_pds = bar_sdp + 8, bar_dqf = bar_pds + 8, bar_dqe = bar_dqf + 8;
  const uint32_t bar_fin = bar_dqe + 8;
  const uint32_t tmem_slot = bar_fin + 8;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gbase + (tmem_slot - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + (tmem_slot + 4 - base));
  int* seg_k = reinterpret_cast<int*>(gbase + (sm_bar + 256 - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = args.T / kTile;
  const int kt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int group = args.H / args.Hkv;
  const int qt_lo = args.causal ? kt : 0;
  const int per_head = n_qt - qt_lo;
  const int n_it = per_head * group;  // iteration it -> head hk*group + it / per_head, q tile qt_lo + it % per_head

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_qf + 8 * s, 1);
      mbar_init(bar_qe + 8 * s, 1);
    }
    mbar_init(bar_sdp, 1);
    mbar_init(bar_pds, kSoftmaxThreads);
    mbar_init(bar_dqf, 1);
    mbar_init(bar_dqe, kSoftmaxThreads);
    mbar_init(bar_fin, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, Plan::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_s = *tmem_slot_ptr;
  const uint32_t tmem_dp = tmem_s + 128;
  const uint32_t tmem_dv = tmem_s + 256;
  const uint32_t tmem_dk = tmem_dv + HD;

  if (warp == 4) {
    if (elect_one_sync()) {
      mbar_expect_tx(bar_kv, 2 * Plan::kTileBytes);
      for (int c = 0; c < kKB; ++c) {
        tma_load_3d(sm_k + c * (kTile * 128), &tmK, bar_kv, hk * HD + 64 * c, kt * kTile, b);
        tma_load_3d(sm_v + c * (kTile * 128), &tmV, bar_kv, hk * HD + 64 * c, kt * kTile, b);
      }
    }
    for (int it = 0; it < n_it; ++it) {
      const int st = it % kStages;
      const uint32_t ph = static_cast<uint32_t>((it / kStages) & 1);
      if (!mbar_wait_warp(bar_qe + 8 * st, ph ^ 1, abort_flag)) {
        if (lane == 0) atomicCAS(args.status, 0, kTimeoutProducer);
        break;
      }
      const int h = hk * group + it / per_head;
      const int qt = qt_lo + it % per_head;
      if (elect_one_sync()) {
        mbar_expect_tx(bar_qf + 8 * st, 2 * Plan::kTileBytes);
        for (int c = 0; c < kKB; ++c) {
          tma_load_3d(sm_q + st * Plan::kTileBytes + c * (kTile * 128), &tmQ, bar_qf + 8 * st, h * HD + 64 * c,
                      qt * kTile, b);
          tma_load_3d(sm_do + st * Plan::kTileBytes + c * (kTile * 128), &tmdO, bar_qf + 8 * st, h * HD + 64 * c,
                      qt * kTile, b);
        }
      }
    }
  } else if (warp == 5) {
    {
      constexpr uint32_t idesc_s = make_idesc_bf16(kTile, kTile, 0, 0);   // Q K^T, dO V^T
      constexpr uint32_t idesc_t = make_idesc_bf16(kTile, HD, 1, 1);      // P^T dO, dS^T Q
      constexpr uint32_t idesc_q = make_idesc_bf16(kTile, HD, 0, 1);      // dS K
      bool ok = mbar_wait_warp(bar_kv, 0, abort_flag);
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it % kStages;
        if (!mbar_wait_warp(bar_qf + 8 * st, static_cast<uint32_t>((it / kStages) & 1), abort_flag)) { ok = false; break; }
        // the softmax warps have read dQ of the previous iteration out of the S columns
        if (!mbar_wait_warp(bar_dqe, static_cast<uint32_t>((it & 1) ^ 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t q_s = sm_q + st * Plan::kTileBytes, do_s = sm_do + st * Plan::kTileBytes;
        if (elect_one_sync()) {
#pragma unroll
          for (int c = 0; c < kKB; ++c) {
            const uint64_t qd = make_smem_desc(q_s + c * (kTile * 128), 16, 1024);
            const uint64_t kd = make_smem_desc(sm_k + c * (kTile * 128), 16, 1024);
            const uint64_t dod = make_smem_desc(do_s + c * (kTile * 128), 16, 1024);
            const uint64_t vd = make_smem_desc(sm_v + c * (kTile * 128), 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              umma_bf16(tmem_s, qd + k * 2, kd + k * 2, idesc_s, (c > 0 || k > 0) ? 1u : 0u);
              umma_bf16(tmem_dp, dod + k * 2, vd + k * 2, idesc_s, (c > 0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit(bar_sdp);
        }
        if (!mbar_wait_warp(bar_pds, static_cast<uint32_t>(it & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (elect_one_sync()) {
          // transposed products: A = P or dS read MN-major (K = query rows), B = dO or Q read MN-major
          const uint64_t pt = make_smem_desc(sm_p, kTile * 128, 1024);
          const uint64_t dst = make_smem_desc(sm_ds, kTile * 128, 1024);
          const uint64_t dob = make_smem_desc(do_s, kTile * 128, 1024);
          const uint64_t qb = make_smem_desc(q_s, kTile * 128, 1024);
#pragma unroll
          for (int k = 0; k < kTile / 16; ++k) {
            umma_bf16(tmem_dv, pt + k * (2048 >> 4), dob + k * (2048 >> 4), idesc_t, (it > 0 || k > 0) ? 1u : 0u);
            umma_bf16(tmem_dk, dst + k * (2048 >> 4), qb + k * (2048 >> 4), idesc_t, (it > 0 || k > 0) ? 1u : 0u);
          }
          // dQ_i = dS K_j: A = dS K-major in the key index, B = K_j read MN-major (K = key rows)
          const uint64_t kb_ = make_smem_desc(sm_k, kTile * 128, 1024);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const uint64_t dsd = make_smem_desc(sm_ds + c * (kTile * 128), 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16(tmem_s, dsd + k * 2, kb_ + (c * 4 + k) * (2048 >> 4), idesc_q, (c > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(bar_qe + 8 * st);
          umma_commit(bar_dqf);
        }
      }
      if (ok && elect_one_sync()) umma_commit(bar_fin);
      if (!ok && lane == 0) atomicCAS(args.status, 0, kTimeoutMma);
    }
  } else {
    const int row = threadIdx.x;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    if (args.segment_ids) seg_k[row] = args.segment_ids[b * args.T + kt * kTile + row];
    named_barrier_softmax();
    bool ok = true;
    uint32_t r[32], g[32];
    for (int it = 0; it < n_it && ok; ++it) {
      const int h = hk * group + it / per_head;
      const int qt = qt_lo + it % per_head;
      const int q_idx = qt * kTile + row;
      const long long stat = (static_cast<long long>(b) * args.H + h) * args.T + q_idx;
      const float L = args.lse[stat];
      const float Dq = args.delta[stat];
      const int seg_q = args.segment_ids ? args.segment_ids[b * args.T + q_idx] : 0;
      const bool diag = args.causal && qt == kt;
      if (!mbar_wait(bar_sdp, static_cast<uint32_t>(it & 1), abort_flag)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        tmem_ld_32x32(tmem_s + lane_base + c * 32, r);
        tmem_ld_32x32(tmem_dp + lane_base + c * 32, g);
        tmem_ld_wait();
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p2[2], d2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = c * 32 + i + e;  // key index inside the tile
            const bool keep = (!diag || col <= row) && (!args.segment_ids || seg_k[col] == seg_q);
            const float p = keep ? fast_exp2(__uint_as_float(r[i + e]) * args.scale_log2 - L) : 0.0f;
            p2[e] = p;
            d2[e] = p * (__uint_as_float(g[i + e]) - Dq) * args.scale;
          }
          pp[i >> 1] = pack_bf16(p2[0], p2[1]);
          dd[i >> 1] = pack_bf16(d2[0], d2[1]);
        }
        const uint32_t off = (c >> 1) * (kTile * 128);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t a = swz(row, (c & 1) * 4 + q4);
          st_shared_v4(sm_p + off + a, make_uint4(pp[4 * q4], pp[4 * q4 + 1], pp[4 * q4 + 2], pp[4 * q4 + 3]));
          st_shared_v4(sm_ds + off + a, make_uint4(dd[4 * q4], dd[4 * q4 + 1], dd[4 * q4 + 2], dd[4 * q4 + 3]));
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(bar_pds);
      // dQ_i tile -> fp32 accumulation buffer (other key tiles add to the same rows)
      if (!mbar_wait(bar_dqf, static_cast<uint32_t>(it & 1), abort_flag)) { ok = false; break; }
      tc_fence_after();
      float* dq_row = args.dq_accum + ((static_cast<long long>(b) * args.T + q_idx) * args.H + h) * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        tmem_ld_32x32(tmem_s + lane_base + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          atomicAdd(reinterpret_cast<float4*>(dq_row + c * 32 + i),
                    make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                                __uint_as_float(r[i + 3])));
      }
      tc_fence_before();
      mbar_arrive(bar_dqe);
    }
    if (ok) {
      if (n_it > 0) {
        if (!mbar_wait(bar_fin, 0, abort_flag)) ok = false;
      }
      if (ok) {
        tc_fence_after();
        const long long krow = ((static_cast<long long>(b) * args.T + kt * kTile + row) * args.Hkv + hk) * HD;
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          __nv_bfloat16* dst = (which == 0 ? args.dv : args.dk) + krow;
          const uint32_t src = (which == 0 ? tmem_dv : tmem_dk) + lane_base;
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            if (n_it > 0) {
              tmem_ld_32x32(src + c * 32, r);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = 0u;
            }
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(r[8 * q8]), __uint_as_float(r[8 * q8 + 1]));
              v.y = pack_bf16(__uint_as_float(r[8 * q8 + 2]), __uint_as_float(r[8 * q8 + 3]));
              v.z = pack_bf16(__uint_as_float(r[8 * q8 + 4]), __uint_as_float(r[8 * q8 + 5]));
              v.w = pack_bf16(__uint_as_float(r[8 * q8 + 6]), __uint_as_float(r[8 * q8 + 7]));
              *reinterpret_cast<uint4*>(dst + c * 32 + 8 * q8) = v;
            }
          }
        }
      }
    }
    if (!ok) atomicCAS(args.status, 0, kTimeoutEpilogue);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_s, Plan::kTmemCols);
}

template <int HD>
int launch_fwd(const CUtensorMap& q, const CUtensorMap& k, const CUtensorMap& v, const AttnArgs& a, cudaStream_t st) {
  auto kern = attn_fwd_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdPlan<HD>::kTotal) != cudaSuccess)
      return 300;
    configured = true;
  }
  dim3 grid(a.T / kTile, a.H, a.B);
  kern<<<grid, kFwdThreads, FwdPlan<HD>::kTotal, st>>>(q, k, v, a);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

template <int HD>
int launch_bwd(const CUtensorMap& q, const CUtensorMap& k, const CUtensorMap& v, const CUtensorMap& d_o,
               const AttnArgs& a, cudaStream_t st) {
  auto kern = attn_bwd_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdPlan<HD>::kTotal) != cudaSuccess)
      return 300;
    configured = true;
  }
  dim3 grid(a.T / kTile, a.Hkv, a.B);
  kern<<<grid, kFwdThreads, BwdPlan<HD>::kTotal, st>>>(q, k, v, d_o, a);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

}  // namespace

extern "C" int pd_flash_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                                      const int* segment_ids, int B, int T, int H, int Hkv, int hd, int causal,
                                      int* status, void* stream) {
  if (bad_shape(B, T, H, Hkv, hd) || status == nullptr) return pd::kBadArgument;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = encode_bthd(&tq, q, B, T, H, hd)) != 0) return 1000 + rc;
  if ((rc = encode_bthd(&tk, k, B, T, Hkv, hd)) != 0) return 1000 + rc;
  if ((rc = encode_bthd(&tv, v, B, T, Hkv, hd)) != 0) return 1000 + rc;
  AttnArgs a{};
  a.B = B; a.T = T; a.H = H; a.Hkv = Hkv; a.causal = causal;
  a.scale = 1.0f / sqrtf(static_cast<float>(hd));
  a.scale_log2 = a.scale * kLog2e;
  a.segment_ids = segment_ids;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.lse = lse;
  a.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return hd == 64 ? launch_fwd<64>(tq, tk, tv, a, st) : launch_fwd<128>(tq, tk, tv, a, st);
}

// `delta` [B, H, T] fp32 and `dq_accum` [B, T, H, hd] fp32 are scratch supplied by the caller;
// `dq_accum` must be zero on entry.
extern "C" int pd_flash_attention_bwd(const void* q, const void* k, const void* v, const void* out, const void* d_out,
                                      const float* lse, float* delta, float* dq_accum, void* dq, void* dk, void* dv,
                                      const int* segment_ids, int B, int T, int H, int Hkv, int hd, int causal,
                                      int* status, void* stream) {
  if (bad_shape(B, T, H, Hkv, hd) || status == nullptr) return pd::kBadArgument;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = encode_bthd(&tq, q, B, T, H, hd)) != 0) return 1000 + rc;
  if ((rc = encode_bthd(&tk, k, B, T, Hkv, hd)) != 0) return 1000 + rc;
  if ((rc = encode_bthd(&tv, v, B, T, Hkv, hd)) != 0) return 1000 + rc;
  if ((rc = encode_bthd(&tdo, d_out, B, T, H, hd)) != 0) return 1000 + rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long rows = static_cast<long long>(B) * T * H;
  attn_delta_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(d_out), delta, B, T, H, hd);
  AttnArgs a{};
  a.B = B; a.T = T; a.H = H; a.Hkv = Hkv; a.causal = causal;
  a.scale = 1.0f / sqrtf(static_cast<float>(hd));
  a.scale_log2 = a.scale * kLog2e;
  a.segment_ids = segment_ids;
  a.lse = const_cast<float*>(lse);
  a.delta = delta;
  a.dq_accum = dq_accum;
  a.dk = static_cast<__nv_bfloat16*>(dk);
  a.dv = static_cast<__nv_bfloat16*>(dv);
  a.status = status;
  rc = hd == 64 ? launch_bwd<64>(tq, tk, tv, tdo, a, st) : launch_bwd<128>(tq, tk, tv, tdo, a, st);
  if (rc != 0) return rc;
  const long long n = rows * hd;
  attn_dq_cast_kernel<<<static_cast<unsigned>(std::min<long long>((n / 4 + 255) / 256, 148 * 16)), 256, 0, st>>>(
      dq_accum, static_cast<__nv_bfloat16*>(dq), n);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}
