// Attention-pattern KL on sm_100a: KL(softmax(S_clean) || softmax(S_masked)) per (batch, head, query)
// without ever forming a [T, T] pattern. Both score tiles come from tcgen05 (two TMEM accumulators),
// the statistics are online base-2 softmax sums kept in registers:
//     KL = A / l_c - LSE_c + LSE_m,   A = sum_j exp(s_c_j - m_c) (s_c_j - s_m_j)
// The backward recomputes the tiles: dS_m = g (softmax(S_m) - softmax(S_c)) * scale, then
// dK_m += dS_m^T Q_m (TMEM across the loop) and dQ_m = dS_m K_m (fp32 atomics); the clean stream is
// a constant. Roles, layouts and masks as in the flash-attention kernels (attention_sm100.cu).
//
// Replaces the reference's Pallas-Triton `_forward_kernel`, `_dq_kernel`, `_dk_kernel`
// (param_decomp/attention_kl.py:93-264).
#include "attention_common.cuh"

namespace {

using namespace pd_attn;

struct KlArgs {
  int B, T, H, Hkv;
  int causal;
  float scale_log2, scale;
  const int* segment_ids;
  float* kl;         // [B, H, T] nats
  float* lse_c;      // [B, H, T] base-2
  float* lse_m;
  const float* g;    // backward: upstream gradient per row [B, H, T]
  float* dq_accum;   // [B, T, H, hd] fp32, zero on entry
  __nv_bfloat16* dk; // [B, T, Hkv, hd]
  int* status;
};

template <int HD>
struct KlFwdPlan {
  static constexpr int kTileBytes = kTile * HD * 2;
  static constexpr int kStages = 2;
  static constexpr int kTotal = 2 * kTileBytes + 2 * kStages * kTileBytes + 2048;
};

template <int HD>
__global__ void __launch_bounds__(kFwdThreads, 1) attn_kl_fwd_kernel(const __grid_constant__ CUtensorMap tmQc,
                                                                      const __grid_constant__ CUtensorMap tmKc,
                                                                      const __grid_constant__ CUtensorMap tmQm,
                                                                      const __grid_constant__ CUtensorMap tmKm,
                                                                      const KlArgs args) {
  using Plan = KlFwdPlan<HD>;
  constexpr int kStages = Plan::kStages;
  constexpr int kKB = HD / 64;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sm_qc = base, sm_qm = sm_qc + Plan::kTileBytes;
  const uint32_t sm_kc = sm_qm + Plan::kTileBytes, sm_km = sm_kc + kStages * Plan::kTileBytes;
  const uint32_t sm_bar = sm_km + kStages * Plan::kTileBytes;
  const uint32_t bar_q = sm_bar, bar_kf = bar_q + 8, bar_ke = bar_kf + 16, bar_s = bar_ke + 16, bar_se = bar_s + 8;
  const uint32_t tmem_slot = bar_se + 8;
  uint8_t* gbase = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(gbase + (tmem_slot - base));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gbase + (tmem_slot + 4 - base));
  int* seg_k = reinterpret_cast<int*>(gbase + (sm_bar + 256 - base));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_se, kSoftmaxThreads);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_c = *tmem_slot_ptr;
  const uint32_t tmem_m = tmem_c + 128;

  if (warp == 4) {
    // whole warp walks the loop, one elected lane issues (operands stay in uniform registers)
    if (elect_one_sync()) {
      mbar_expect_tx(bar_q, 2 * Plan::kTileBytes);
      for (int c = 0; c < kKB; ++c) {
        tma_load_3d(sm_qc + c * (kTile * 128), &tmQc, bar_q, h * HD + 64 * c, qt * kTile, b);
        tma_load_3d(sm_qm + c * (kTile * 128), &tmQm, bar_q, h * HD + 64 * c, qt * kTile, b);
      }
    }
    for (int j = 0; j < n_kv; ++j) {
      const int st = j % kStages;
      if (!mbar_wait_warp(bar_ke + 8 * st, static_cast<uint32_t>(((j / kStages) & 1) ^ 1), abort_flag)) {
        if (lane == 0) atomicCAS(args.status, 0, kTimeoutProducer);
        break;
      }
      if (elect_one_sync()) {
        mbar_expect_tx(bar_kf + 8 * st, 2 * Plan::kTileBytes);
        for (int c = 0; c < kKB; ++c) {
          tma_load_3d(sm_kc + st * Plan::kTileBytes + c * (kTile * 128), &tmKc, bar_kf + 8 * st, hk * HD + 64 * c,
                      j * kTile, b);
          tma_load_3d(sm_km + st * Plan::kTileBytes + c * (kTile * 128), &tmKm, bar_kf + 8 * st, hk * HD + 64 * c,
                      j * kTile, b);
        }
      }
    }
  } else if (warp == 5) {
    {
      constexpr uint32_t idesc = make_idesc_bf16(kTile, kTile, 0, 0);
      bool ok = mbar_wait_warp(bar_q, 0, abort_flag);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j % kStages;
        if (!mbar_wait_warp(bar_kf + 8 * st, static_cast<uint32_t>((j / kStages) & 1), abort_flag) ||
            !mbar_wait_warp(bar_se, static_cast<uint32_t>((j & 1) ^ 1), abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (elect_one_sync()) {
#pragma unroll
          for (int c = 0; c < kKB; ++c) {
            const uint64_t qc = make_smem_desc(sm_qc + c * (kTile * 128), 16, 1024);
            const uint64_t qm = make_smem_desc(sm_qm + c * (kTile * 128), 16, 1024);
            const uint64_t kc = make_smem_desc(sm_kc + st * Plan::kTileBytes + c * (kTile * 128), 16, 1024);
            const uint64_t km = make_smem_desc(sm_km + st * Plan::kTileBytes + c * (kTile * 128), 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              umma_bf16(tmem_c, qc + k * 2, kc + k * 2, idesc, (c > 0 || k > 0) ? 1u : 0u);
              umma_bf16(tmem_m, qm + k * 2, km + k * 2, idesc, (c > 0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit(bar_ke + 8 * st);
          umma_commit(bar_s);
        }
      }
      if (!ok && lane == 0) atomicCAS(args.status, 0, kTimeoutMma);
    }
  } else {
    const int row = threadIdx.x;
    const int q_idx = qt * kTile + row;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    const int seg_q = args.segment_ids ? args.segment_ids[b * args.T + q_idx] : 0;
    float m_c = -INFINITY, l_c = 0.0f, A = 0.0f, m_m = -INFINITY, l_m = 0.0f;
    bool ok = true;
    uint32_t rc[32], rm[32];
    for (int j = 0; j < n_kv && ok; ++j) {
      if (args.segment_ids) {
        named_barrier_softmax();
        seg_k[row] = args.segment_ids[b * args.T + j * kTile + row];
        named_barrier_softmax();
      }
      if (!mbar_wait(bar_s, static_cast<uint32_t>(j & 1), abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = args.causal && j == qt;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        tmem_ld_32x32(tmem_c + lane_base + c * 32, rc);
        tmem_ld_32x32(tmem_m + lane_base + c * 32, rm);
        tmem_ld_wait();
        float mc_new = m_c, mm_new = m_m;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int col = c * 32 + i;
          const bool keep = (!diag || col <= row) && (!args.segment_ids || seg_k[col] == seg_q);
          if (keep) {
            mc_new = fmaxf(mc_new, __uint_as_float(rc[i]) * args.scale_log2);
            mm_new = fmaxf(mm_new, __uint_as_float(rm[i]) * args.scale_log2);
          }
        }
        if (mc_new == -INFINITY) continue;  // nothing kept so far in this row
        const float fc = (m_c == -INFINITY) ? 0.0f : fast_exp2(m_c - mc_new);
        const float fm = (m_m == -INFINITY) ? 0.0f : fast_exp2(m_m - mm_new);
        float lc_add = 0.0f, a_add = 0.0f, lm_add = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int col = c * 32 + i;
          const bool keep = (!diag || col <= row) && (!args.segment_ids || seg_k[col] == seg_q);
          if (keep) {
            const float sc = __uint_as_float(rc[i]) * args.scale_log2, sm = __uint_as_float(rm[i]) * args.scale_log2;
            const float e = fast_exp2(sc - mc_new);
            lc_add += e;
            a_add = fmaf(e, sc - sm, a_add);
            lm_add += fast_exp2(sm - mm_new);
          }
        }
        l_c = fmaf(l_c, fc, lc_add);
        A = fmaf(A, fc, a_add);
        l_m = fmaf(l_m, fm, lm_add);
        m_c = mc_new;
        m_m = mm_new;
      }
      tc_fence_before();
      mbar_arrive(bar_se);
    }
    if (ok) {
      const long long o = (static_cast<long long>(b) * args.H + h) * args.T + q_idx;
      const float Lc = m_c + log2f(l_c), Lm = m_m + log2f(l_m);
      args.kl[o] = kLn2 * (A / l_c - Lc + Lm);
      args.lse_c[o] = Lc;
      args.lse_m[o] = Lm;
    } else {
      atomicCAS(args.status, 0, kTimeoutEpilogue);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_c, 256);
}

template <int HD>
struct KlBwdPlan {
  static constexpr int kTileBytes = kTile * HD * 2;
  static constexpr int kStages = HD == 64 ? 2 : 1;
  static constexpr int kDsBytes = kTile * kTile * 2;
  static constexpr int kTotal = 2 * kTileBytes + 2 * kStages * kTileBytes + kDsBytes + 2048;
};

template <int HD>
__global__ void __launch_bounds__(kFwdThreads, 1) attn_kl_bwd_kernel(const __grid_constant__ CUtensorMap tmQc,
                                                                      const __grid_constant__ CUtensorMap tmKc,
                                                                      const __grid_constant__ CUtensorMap tmQm,
                                                                      const __grid_constant__ CUtensorMap tmKm,
                                                                      const KlArgs args) {
  using Plan = KlBwdPlan<HD>;
  constexpr int kStages = Plan::kStages;
  constexpr int kKB = HD / 64;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sm_kc = base, sm_km = sm_kc + Plan::kTileBytes;
  const uint32_t sm_qc = sm_km + Plan::kTileBytes, sm_qm = sm_qc + kStages * Plan::kTileBytes;
  const uint32_t sm_ds = sm_qm + kStages * Plan::kTileBytes;
  const uint32_t sm_bar = sm_ds + Plan::kDsBytes;
  const uint32_t bar_kv = sm_bar, bar_qf = bar_kv + 8, bar_qe = bar_qf + 16;
  const uint32_t bar_s = bar_qe + 16, bar_ds = bar_s + 8, bar_dqf = bar_ds + 8, bar_dqe = bar_dqf + 8;
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
  const int n_it = per_head * group;

  if (threadIdx.x == 0) {
    mbar_init(bar_kv, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_qf + 8 * s, 1);
      mbar_init(bar_qe + 8 * s, 1);
    }
    mbar_init(bar_s, 1);
    mbar_init(bar_ds, kSoftmaxThreads);
    mbar_init(bar_dqf, 1);
    mbar_init(bar_dqe, kSoftmaxThreads);
    mbar_init(bar_fin, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_c = *tmem_slot_ptr;  // S_clean, later dQ
  const uint32_t tmem_m = tmem_c + 128;
  const uint32_t tmem_dk = tmem_c + 256;

  if (warp == 4) {
    if (elect_one_sync()) {
      mbar_expect_tx(bar_kv, 2 * Plan::kTileBytes);
      for (int c = 0; c < kKB; ++c) {
        tma_load_3d(sm_kc + c * (kTile * 128), &tmKc, bar_kv, hk * HD + 64 * c, kt * kTile, b);
        tma_load_3d(sm_km + c * (kTile * 128), &tmKm, bar_kv, hk * HD + 64 * c, kt * kTile, b);
      }
    }
    for (int it = 0; it < n_it; ++it) {
      const int st = it % kStages;
      if (!mbar_wait_warp(bar_qe + 8 * st, static_cast<uint32_t>(((it / kStages) & 1) ^ 1), abort_flag)) {
        if (lane == 0) atomicCAS(args.status, 0, kTimeoutProducer);
        break;
      }
      const int h = hk * group + it / per_head;
      const int qt = qt_lo + it % per_head;
      if (elect_one_sync()) {
        mbar_expect_tx(bar_qf + 8 * st, 2 * Plan::kTileBytes);
        for (int c = 0; c < kKB; ++c) {
          tma_load_3d(sm_qc + st * Plan::kTileBytes + c * (kTile * 128), &tmQc, bar_qf + 8 * st, h * HD + 64 * c,
                      qt * kTile, b);
          tma_load_3d(sm_qm + st * Plan::kTileBytes + c * (kTile * 128), &tmQm, bar_qf + 8 * st, h * HD + 64 * c,
                      qt * kTile, b);
        }
      }
    }
  } else if (warp == 5) {
    {
      constexpr uint32_t idesc_s = make_idesc_bf16(kTile, kTile, 0, 0);
      constexpr uint32_t idesc_t = make_idesc_bf16(kTile, HD, 1, 1);
      constexpr uint32_t idesc_q = make_idesc_bf16(kTile, HD, 0, 1);
      bool ok = mbar_wait_warp(bar_kv, 0, abort_flag);
      for (int it = 0; it < n_it && ok; ++it) {
        const int st = it % kStages;
        if (!mbar_wait_warp(bar_qf + 8 * st, static_cast<uint32_t>((it / kStages) & 1), abort_flag) ||
            !mbar_wait_warp(bar_dqe, static_cast<uint32_t>((it & 1) ^ 1), abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t qc_s = sm_qc + st * Plan::kTileBytes, qm_s = sm_qm + st * Plan::kTileBytes;
        if (elect_one_sync()) {
#pragma unroll
          for (int c = 0; c < kKB; ++c) {
            const uint64_t qc = make_smem_desc(qc_s + c * (kTile * 128), 16, 1024);
            const uint64_t qm = make_smem_desc(qm_s + c * (kTile * 128), 16, 1024);
            const uint64_t kc = make_smem_desc(sm_kc + c * (kTile * 128), 16, 1024);
            const uint64_t km = make_smem_desc(sm_km + c * (kTile * 128), 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              umma_bf16(tmem_c, qc + k * 2, kc + k * 2, idesc_s, (c > 0 || k > 0) ? 1u : 0u);
              umma_bf16(tmem_m, qm + k * 2, km + k * 2, idesc_s, (c > 0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit(bar_s);
        }
        if (!mbar_wait_warp(bar_ds, static_cast<uint32_t>(it & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (elect_one_sync()) {
          const uint64_t dst = make_smem_desc(sm_ds, kTile * 128, 1024);
          const uint64_t qb = make_smem_desc(qm_s, kTile * 128, 1024);
#pragma unroll
          for (int k = 0; k < kTile / 16; ++k)
            umma_bf16(tmem_dk, dst + k * (2048 >> 4), qb + k * (2048 >> 4), idesc_t, (it > 0 || k > 0) ? 1u : 0u);
          const uint64_t kb_ = make_smem_desc(sm_km, kTile * 128, 1024);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const uint64_t dsd = make_smem_desc(sm_ds + c * (kTile * 128), 16, 1024);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16(tmem_c, dsd + k * 2, kb_ + (c * 4 + k) * (2048 >> 4), idesc_q, (c > 0 || k > 0) ? 1u : 0u);
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
    uint32_t rc[32], rm[32];
    for (int it = 0; it < n_it && ok; ++it) {
      const int h = hk * group + it / per_head;
      const int qt = qt_lo + it % per_head;
      const int q_idx = qt * kTile + row;
      const long long stat = (static_cast<long long>(b) * args.H + h) * args.T + q_idx;
      const float Lc = args.lse_c[stat], Lm = args.lse_m[stat];
      const float gs = args.g[stat] * args.scale;
      const int seg_q = args.segment_ids ? args.segment_ids[b * args.T + q_idx] : 0;
      const bool diag = args.causal && qt == kt;
      if (!mbar_wait(bar_s, static_cast<uint32_t>(it & 1), abort_flag)) { ok = false; break; }
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        tmem_ld_32x32(tmem_c + lane_base + c * 32, rc);
        tmem_ld_32x32(tmem_m + lane_base + c * 32, rm);
        tmem_ld_wait();
        uint32_t dd[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float d2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = c * 32 + i + e;
            const bool keep = (!diag || col <= row) && (!args.segment_ids || seg_k[col] == seg_q);
            const float p = fast_exp2(__uint_as_float(rc[i + e]) * args.scale_log2 - Lc);
            const float qq = fast_exp2(__uint_as_float(rm[i + e]) * args.scale_log2 - Lm);
            d2[e] = keep ? gs * (qq - p) : 0.0f;
          }
          dd[i >> 1] = pack_bf16(d2[0], d2[1]);
        }
        const uint32_t off = (c >> 1) * (kTile * 128);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          st_shared_v4(sm_ds + off + swz(row, (c & 1) * 4 + q4),
                       make_uint4(dd[4 * q4], dd[4 * q4 + 1], dd[4 * q4 + 2], dd[4 * q4 + 3]));
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(bar_ds);
      if (!mbar_wait(bar_dqf, static_cast<uint32_t>(it & 1), abort_flag)) { ok = false; break; }
      tc_fence_after();
      float* dq_row = args.dq_accum + ((static_cast<long long>(b) * args.T + q_idx) * args.H + h) * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        tmem_ld_32x32(tmem_c + lane_base + c * 32, rc);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          atomicAdd(reinterpret_cast<float4*>(dq_row + c * 32 + i),
                    make_float4(__uint_as_float(rc[i]), __uint_as_float(rc[i + 1]), __uint_as_float(rc[i + 2]),
                                __uint_as_float(rc[i + 3])));
      }
      tc_fence_before();
      mbar_arrive(bar_dqe);
    }
    if (ok && !mbar_wait(bar_fin, 0, abort_flag)) ok = false;
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dst = args.dk + ((static_cast<long long>(b) * args.T + kt * kTile + row) * args.Hkv + hk) * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        tmem_ld_32x32(tmem_dk + lane_base + c * 32, rc);
        tmem_ld_wait();
#pragma unroll
        for (int q8 = 0; q8 < 4; ++q8) {
          uint4 v;
          v.x = pack_bf16(__uint_as_float(rc[8 * q8]), __uint_as_float(rc[8 * q8 + 1]));
          v.y = pack_bf16(__uint_as_float(rc[8 * q8 + 2]), __uint_as_float(rc[8 * q8 + 3]));
          v.z = pack_bf16(__uint_as_float(rc[8 * q8 + 4]), __uint_as_float(rc[8 * q8 + 5]));
          v.w = pack_bf16(__uint_as_float(rc[8 * q8 + 6]), __uint_as_float(rc[8 * q8 + 7]));
          *reinterpret_cast<uint4*>(dst + c * 32 + 8 * q8) = v;
        }
      }
    } else {
      atomicCAS(args.status, 0, kTimeoutEpilogue);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_c, 512);
}

__global__ void kl_dq_cast_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long n) {
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(acc + i);
    uint2 o;
    o.x = pack_bf16(v.x, v.y);
    o.y = pack_bf16(v.z, v.w);
    *reinterpret_cast<uint2*>(dq + i) = o;
  }
}

template <int HD, bool BWD>
int launch(const CUtensorMap& qc, const CUtensorMap& kc, const CUtensorMap& qm, const CUtensorMap& km,
           const KlArgs& a, cudaStream_t st) {
  constexpr int smem = BWD ? KlBwdPlan<HD>::kTotal : KlFwdPlan<HD>::kTotal;
  auto kern = BWD ? attn_kl_bwd_kernel<HD> : attn_kl_fwd_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return 300;
    configured = true;
  }
  dim3 grid(a.T / kTile, BWD ? a.Hkv : a.H, a.B);
  kern<<<grid, kFwdThreads, smem, st>>>(qc, kc, qm, km, a);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

int encode4(CUtensorMap* t, const void* qc, const void* kc, const void* qm, const void* km, int B, int T, int H,
            int Hkv, int hd) {
  int rc;
  if ((rc = encode_bthd(&t[0], qc, B, T, H, hd)) != 0) return 1000 + rc;
  if ((rc = encode_bthd(&t[1], kc, B, T, Hkv, hd)) != 0) return 1000 + rc;
  if ((rc = encode_bthd(&t[2], qm, B, T, H, hd)) != 0) return 1000 + rc;
  if ((rc = encode_bthd(&t[3], km, B, T, Hkv, hd)) != 0) return 1000 + rc;
  return 0;
}

}  // namespace

// q [B,T,H,hd], k [B,T,Hkv,hd] bf16 (after RoPE); kl, lse_c, lse_m [B,H,T] fp32
extern "C" int pd_attention_kl_fwd(const void* qc, const void* kc, const void* qm, const void* km, float* kl,
                                   float* lse_c, float* lse_m, const int* segment_ids, int B, int T, int H, int Hkv,
                                   int hd, int causal, int* status, void* stream) {
  if (bad_shape(B, T, H, Hkv, hd) || status == nullptr) return pd::kBadArgument;
  CUtensorMap t[4];
  int rc = encode4(t, qc, kc, qm, km, B, T, H, Hkv, hd);
  if (rc != 0) return rc;
  KlArgs a{};
  a.B = B; a.T = T; a.H = H; a.Hkv = Hkv; a.causal = causal;
  a.scale = 1.0f / sqrtf(static_cast<float>(hd));
  a.scale_log2 = a.scale * kLog2e;
  a.segment_ids = segment_ids;
  a.kl = kl; a.lse_c = lse_c; a.lse_m = lse_m; a.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return hd == 64 ? launch<64, false>(t[0], t[1], t[2], t[3], a, st) : launch<128, false>(t[0], t[1], t[2], t[3], a, st);
}

// g [B,H,T] upstream gradient of kl; dq_accum [B,T,H,hd] fp32 zero on entry; dq, dk bf16 outputs (masked stream)
extern "C" int pd_attention_kl_bwd(const void* qc, const void* kc, const void* qm, const void* km, const float* lse_c,
                                   const float* lse_m, const float* g, float* dq_accum, void* dq, void* dk,
                                   const int* segment_ids, int B, int T, int H, int Hkv, int hd, int causal,
                                   int* status, void* stream) {
  if (bad_shape(B, T, H, Hkv, hd) || status == nullptr) return pd::kBadArgument;
  CUtensorMap t[4];
  int rc = encode4(t, qc, kc, qm, km, B, T, H, Hkv, hd);
  if (rc != 0) return rc;
  KlArgs a{};
  a.B = B; a.T = T; a.H = H; a.Hkv = Hkv; a.causal = causal;
  a.scale = 1.0f / sqrtf(static_cast<float>(hd));
  a.scale_log2 = a.scale * kLog2e;
  a.segment_ids = segment_ids;
  a.lse_c = const_cast<float*>(lse_c); a.lse_m = const_cast<float*>(lse_m); a.g = g;
  a.dq_accum = dq_accum; a.dk = static_cast<__nv_bfloat16*>(dk); a.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = hd == 64 ? launch<64, true>(t[0], t[1], t[2], t[3], a, st) : launch<128, true>(t[0], t[1], t[2], t[3], a, st);
  if (rc != 0) return rc;
  const long long n = static_cast<long long>(B) * T * H * hd;
  long long blocks = (n / 4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  kl_dq_cast_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(dq_accum, static_cast<__nv_bfloat16*>(dq), n);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}
