// Persistent, warp-specialised bf16 GEMM for sm_100a built on tcgen05.mma with TMEM accumulators
// and TMA-fed shared-memory operands, plus the fused epilogues the decomposition step needs.
//
//   D[b][M,N] = sum over up to two K-phases of A_p[b] * B_p[b]
//
// Each operand is described by a tensor map and a "major": K-major means the matrix is stored with
// K contiguous ([M,K] or [N,K] row-major); MN-major means it is stored transposed ([K,M] or [K,N]
// row-major). All four combinations run on the same kernel, so forward, input-gradient and
// weight-gradient products all read the tensors exactly as they sit in memory, no transposed copies.
//
// Two K-phases let one accumulator take  (xV .* coef) U  +  (d .* x) W^T  without a second pass:
// phase 0 walks the component axis, phase 1 walks d_in, and the sum never leaves TMEM.
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + single-thread MMA issuer,
// warps 2..9 = epilogue. A warp may only read the TMEM lane quarter warp_id % 4, so two warps share
// each quarter and take alternate output boxes; with short K (d_in = 768) the epilogue is the
// longer half of a tile and needs the issue slots of all four schedulers. Two accumulators of BN
// columns alternate so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Tiles are rasterised in panels of kGroupM row blocks so that one wave of CTAs touches few
// distinct A and B blocks (both stay in L2 while the [M,N]-sized epilogue tensors stream past).
//
// Epilogues:
//   EPI_PLAIN     out0 = act(alpha * acc + bias)          bf16 or fp32, optional reduce-add (split-K
//                                                         and gradient accumulation)
//   EPI_MASK_FWD  out0 = bf16(acc .* coef), out1 = bf16(acc) (optional)
//                 coef = rowscale * (m - delta),  m = ci + (1 - ci) * u,  u ~ Philox(seed, stream, row, col)
//                 or m read from memory when mask_mode == 1
//   EPI_MASK_BWD  acc = dA;  out0 = bf16(acc .* coef);  dci (+)= acc .* H .* rowscale .* dm/dci
//   EPI_FAITH     out0 = bf16(R - acc) with R read from memory, and *sumsq += sum (R - acc)^2:
//                 the faithfulness residual W - (VU)^T and its squared norm without a second pass
//
// The mask epilogues come in two forms. NOUT = 1 / 2: each epilogue thread reads its row's ci / H values with
// plain global loads (row-strided: 32 cache lines per warp request) and writes its mask gradient the same way;
// this form serves row-mapped (routed) products. NOUT = 4, the TMA-fed form for dense sites: ci and H arrive as
// 32-row x 64-column boxes by TMA into a two-slot ring of shared-memory boxes per epilogue warp (issued one
// unit ahead), every thread reads its own 128-byte row of the swizzled box, writes its results IN PLACE
// (ci box -> A or dH, H box -> mask gradient or the H output) and the boxes leave by TMA store. No global
// load or store instruction is left in the epilogue: L1 wavefronts drop from 32 to 4 per 16-byte request.
//
// Every wait is bounded (see common.cuh); on time-out the kernel stores a code to *status and returns.
#include "common.cuh"

namespace pd {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kNumEpiWarps = 8;
constexpr int kNumThreads = 32 * (2 + kNumEpiWarps);
constexpr int kGatherChunk = 16384;  // bytes per bulk copy of the all-gather CTAs
constexpr int kGatherSlotsMax = 12;
constexpr int kMaxPeers = 8;

struct PeerMaps {
  CUtensorMap m[kMaxPeers];
};
constexpr int kGroupM = 16;
constexpr int kStageBytesA = BM * BK * 2;  // 16 KiB
constexpr int kOutBoxBytes = 32 * 128;     // one 32-row x 128-byte staging box

enum Epi : int { EPI_PLAIN = 0, EPI_MASK_FWD = 1, EPI_MASK_BWD = 2, EPI_FAITH = 3 };
enum Act : int { ACT_NONE = 0, ACT_GELU = 1, ACT_SILU = 2, ACT_RELU = 3 };

struct GemmArgs {
  int M, N, batch;
  int kblocks0, kblocks1;
  int split_k;
  int a_mn0, b_mn0, a_mn1, b_mn1;
  int accumulate;
  int out_fp32;
  int has_out1;
  float alpha;
  const float* alpha_dev;  // when set, the plain epilogue scales by alpha * *alpha_dev (a scheduled coefficient in device memory)
  const float* bias;
  long long bias_bs;
  int act;
  const __nv_bfloat16* ci;
  long long ld_ci;
  const __nv_bfloat16* H;
  long long ld_h;
  const float* delta;
  const float* rowscale;
  float* dci;
  long long ld_dci;
  int dci_accumulate;
  int dci_bf16;
  unsigned long long seed;
  // When set, the Philox seed is read from device memory at run time instead of `seed`: a launch recorded
  // once (CUDA graph) then draws a fresh mask stream every replay after the host rewrites that word.
  const unsigned long long* seed_dev;
  unsigned int stream;
  unsigned int row_offset;
  int mask_mode;
  int* status;
  // grouped (ragged) products: see PdGemmCall
  const int* bgroup_of_mblock;
  const int* kblock_range;
  int a_bcast, b_bcast;
  // GEMM -> reduce-scatter: output row block goes to its owner's fp32 buffer by TMA reduce-add
  int rs_world;          // 0/1 = off
  int rs_rows;           // rows per owner (multiple of 128)
  // all-gather -> GEMM: A (phase 0) rows are sharded by rank; remote row blocks are pulled into the
  // local full-size A buffer by the gather warp, each block once per GPU, and released by a flag
  int ag_world, ag_rank; // ag_world 0/1 = off
  int ag_rows;           // rows per rank (multiple of 128)
  const void* ag_src[kMaxPeers];  // each rank's shard [ag_rows, K0] bf16, row pitch ag_ld elements
  void* ag_dst;          // local full buffer [M, K0] (the A0 operand), same row pitch
  long long ag_ld;
  int ag_k;              // K0 in elements
  unsigned int* ag_flags;  // [num_m] local flags, block is ready when flag == ag_seq
  unsigned int ag_seq;
  int ag_gather_ctas;    // trailing CTAs of the grid that only move peers' rows (no tiles)
  int ag_mode;           // 0: A row blocks (activations sharded by rows); 1: B K-slabs (weights sharded by K rows)
  // Mask epilogues on job rows (routed experts): row r of the product reads its CI / mask values, its
  // delta and row scale, draws its uniforms and writes its CI gradient at the SOURCE position
  // rowmap[r] = {source row, first source column, -, -}; source row -1 marks a padding row.
  const int4* rowmap;
  // First global column of this product's mask columns in the Philox counter space (a rank that holds a
  // column slice of a site draws the same uniforms the whole site would); multiple of 8.
  unsigned int philox_col0;
  // panel decode without a hardware divide: quotient by kGroupM * num_n = (umulhi(n, pg_mul) + n) >> pg_shift
  unsigned int pg_mul, pg_shift;
  long long* timeline;  // diagnostic: CTA 0 writes clock64() stamps here (256 slots), nullptr = off
  int probe;        // timing probes (results are garbage): bit 0 = no operand loads, bit 1 = no MMAs, bit 2 (with bit 0) = no operand barriers
  int stage_limit;  // > 0: use only this many of the operand ring's stages (a tuning probe of pipeline depth)
};

template <int BN, int NOUT, int CG = 1>
struct SmemPlan {
  static constexpr int kStageBytesB = BN * BK * 2 / CG;  // a CTA pair splits the B tile
  static constexpr int kStageBytes = kStageBytesA + kStageBytesB;
  static constexpr int kOutBytes = kNumEpiWarps * NOUT * kOutBoxBytes;
  static constexpr int kBarrierBytes = 512;  // pipeline + accumulator barriers, then two operand barriers per epilogue warp
  static constexpr int kBudget = 227 * 1024 - 1024 /*alignment slack*/ - kBarrierBytes;
  static constexpr int kStagesRaw = (kBudget - kOutBytes) / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kTotal = kStages * kStageBytes + kOutBytes + kBarrierBytes + 1024;
  static_assert(16 * kStages + 40 + 8 * kGatherSlotsMax <= 256, "barrier area");
  static_assert(kStages >= 2, "the operand pipeline needs at least two stages");
};

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case ACT_GELU:
      return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    case ACT_SILU:
      return v / (1.0f + __expf(-v));
    case ACT_RELU:
      return fmaxf(v, 0.0f);
    default:
      return v;
  }
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// Packed fp32 pairs (`.f32x2`, one instruction for two lanes of arithmetic): the mask epilogue is bound by
// instruction issue, so its per-element arithmetic runs two columns at a time. Each op rounds exactly like
// its scalar form.
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pk2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ f32x2 pk2u(uint32_t lo, uint32_t hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16_2(f32x2 v) {  // (lo, hi) -> bf16x2 with lo in the low half
  uint32_t r;
  asm("{\n\t.reg .f32 lo, hi;\n\tmov.b64 {lo, hi}, %1;\n\tcvt.rn.bf16x2.f32 %0, hi, lo;\n\t}" : "=r"(r) : "l"(v));
  return r;
}
// bf16x2 word -> the two values as an fp32 pair
__device__ __forceinline__ f32x2 unpack_bf16_2(uint32_t w) { return pk2u(w << 16, w & 0xFFFF0000u); }
// One Philox word -> its two 16-bit uniforms (b + 0.5) / 65536 as an fp32 pair: the bits go to the top of the
// mantissa of a float in [1, 2), and 2^-17 - 1 (exact in fp32) is added - the same values as `bits16_to_unit`.
__device__ __forceinline__ f32x2 philox_word_to_unit2(uint32_t w) {
  const uint32_t lo = 0x3F800000u | ((w & 0xFFFFu) << 7), hi = 0x3F800000u | ((w >> 9) & 0x007FFF80u);
  constexpr float kBias = 0.5f / 65536.0f - 1.0f;
  return add2(pk2u(lo, hi), pk2(kBias, kBias));
}

// Write 32 bf16 values (half of a 64-column box) of this thread's row into the swizzled staging box.
__device__ __forceinline__ void stage_bf16_half(uint32_t box, int lane, int half,
                                                const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int idx = half * 4 + j;
    const uint32_t addr = box + lane * 128 + ((idx ^ (lane & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                 "r"(pack_bf16(v[8 * j + 0], v[8 * j + 1])),
                 "r"(pack_bf16(v[8 * j + 2], v[8 * j + 3])),
                 "r"(pack_bf16(v[8 * j + 4], v[8 * j + 5])),
                 "r"(pack_bf16(v[8 * j + 6], v[8 * j + 7]))
                 : "memory");
  }
}
__device__ __forceinline__ void stage_fp32(uint32_t box, int lane, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t addr = box + lane * 128 + ((j ^ (lane & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                 "r"(__float_as_uint(v[4 * j + 0])), "r"(__float_as_uint(v[4 * j + 1])),
                 "r"(__float_as_uint(v[4 * j + 2])), "r"(__float_as_uint(v[4 * j + 3]))
                 : "memory");
  }
}

template <int BN, int EPI, int NOUT, int CG>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmB0,
            const __grid_constant__ CUtensorMap tmA1, const __grid_constant__ CUtensorMap tmB1,
            const __grid_constant__ CUtensorMap tmOut0, const __grid_constant__ CUtensorMap tmOut1,
            const __grid_constant__ CUtensorMap tmCi, const __grid_constant__ CUtensorMap tmH,
            const __grid_constant__ CUtensorMap tmDci,
            const __grid_constant__ PeerMaps peerOut, const GemmArgs args) {
  using Plan = SmemPlan<BN, NOUT, CG>;
  constexpr int kStages = Plan::kStages;
  const int nstages = (args.stage_limit >= 2 && args.stage_limit < kStages) ? args.stage_limit : kStages;
  constexpr int kStageBytesB = Plan::kStageBytesB;
  constexpr uint32_t kTmemCols = 2 * BN;  // 256 or 512: powers of two as tcgen05.alloc requires
  // CG == 2: two CTAs of a cluster share a 256-row tile; rank 0 issues the MMAs for both.
  const uint32_t cta_rank = CG == 2 ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_a = smem_base;
  const uint32_t smem_b = smem_a + kStages * kStageBytesA;
  const uint32_t smem_out = smem_b + kStages * kStageBytesB;
  const uint32_t smem_bar = smem_out + Plan::kOutBytes;
  // barrier layout: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2], then two words
  const uint32_t bar_full = smem_bar;
  const uint32_t bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_tfull = bar_empty + 8 * kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  const uint32_t tmem_slot = bar_tempty + 16;
  uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(
      generic_base + (tmem_slot - smem_base));
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(generic_base + (tmem_slot + 4 - smem_base));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // Diagnostic timeline (CTA 0 only): slot 0 entry, 1 set-up done, 2 before teardown, 3 exit; MMA issuer
  // 16 + 2i / 17 + 2i = accumulator granted / tile i committed; first epilogue warp 80 + 2i / 81 + 2i =
  // accumulator full seen / tile i drained; producer 144 + i = last load of tile i issued; TMA-fed mask epilogue, first
  // epilogue warp, unit u < 8: 176 + 8u .. 182 + 8u = operands landed, accumulator ready, values in registers,
  // first half done, next operands requested, second half done, stores issued.
  auto stamp = [&](int slot) {
    if (args.timeline != nullptr && blockIdx.x == 0 && slot < 256) args.timeline[slot] = clock64();
  };
  if (threadIdx.x == 0) stamp(0);
  const int num_m = (args.M + BM - 1) / BM;
  const int num_n = (args.N + BN - 1) / BN;
  const int kb_total = args.kblocks0 + args.kblocks1;
  const int split = args.split_k;
  const int kb_per_split = (kb_total + split - 1) / split;
  const int num_m_t = (num_m + CG - 1) / CG;  // row tiles of 128 * CG rows
  const long long num_tiles = static_cast<long long>(num_m_t) * num_n * split * args.batch;
  // All-gather mode: the last `ag_gather_ctas` CTAs own no tiles; they stream peers' row blocks
  // into the local A buffer while the others compute.
  const int n_gather = args.ag_world > 1 ? args.ag_gather_ctas : 0;
  const int n_compute = static_cast<int>(gridDim.x) - n_gather;
  const bool is_gather_cta = static_cast<int>(blockIdx.x) >= n_compute;
  const long long tile0 = is_gather_cta ? num_tiles : static_cast<long long>(blockIdx.x) / CG;
  const long long tstride = n_compute / CG;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, kNumEpiWarps * CG);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA0);
    tma_prefetch_desc(&tmB0);
    tma_prefetch_desc(&tmOut0);
    if (args.kblocks1 > 0) {
      tma_prefetch_desc(&tmA1);
      tma_prefetch_desc(&tmB1);
    }
  }
  if (warp == 1) {
    if constexpr (CG == 2) {
      tmem_alloc_pair(tmem_slot, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  if (threadIdx.x == 0) stamp(1);

  // Tile decode: batch / split outermost, then panels of kGroupM row blocks walked column by column.
  const long long tiles_per_mat = static_cast<long long>(num_m_t) * num_n;
  // One matrix and no K split (every site product of a train step): the tile index is the panel index and fits
  // 32 bits, the panel quotient is a multiply-high, a full panel's row / column split is a shift and a mask.
  // The epilogue warps decode several tiles per unit of work, so this keeps divides off their critical path.
  const bool single_mat = split == 1 && args.batch == 1;
  auto decode = [&](long long t, int& b, int& mb, int& nb, int& sp) {
    uint32_t pid;
    if (single_mat) {
      pid = static_cast<uint32_t>(t);
      sp = 0;
      b = 0;
    } else {
      const long long outer = t / tiles_per_mat;
      pid = static_cast<uint32_t>(t % tiles_per_mat);
      sp = static_cast<int>(outer % split);
      b = static_cast<int>(outer / split);
    }
    const uint32_t per_group = static_cast<uint32_t>(kGroupM * num_n);
    const uint32_t group = (__umulhi(pid, args.pg_mul) + pid) >> args.pg_shift;
    const int first_m = static_cast<int>(group) * kGroupM;
    const int gsz = min(num_m_t - first_m, kGroupM);
    const uint32_t in_group = pid - group * per_group;
    uint32_t r_in, c_in;
    if (gsz == kGroupM) {
      r_in = in_group & static_cast<uint32_t>(kGroupM - 1);
      c_in = in_group / static_cast<uint32_t>(kGroupM);
    } else {
      c_in = in_group / static_cast<uint32_t>(gsz);
      r_in = in_group - c_in * static_cast<uint32_t>(gsz);
    }
    mb = (first_m + static_cast<int>(r_in)) * CG + static_cast<int>(cta_rank);
    nb = static_cast<int>(c_in);
    if (args.ag_world > 1 && args.ag_mode == 0) {  // start with the row blocks this rank already holds
      const int per_rank = args.ag_rows / BM;
      mb = (mb + args.ag_rank * per_rank) % num_m;
    }
  };

  // K-block range of a tile: a split of the whole K extent, or (ragged weight-gradient products) the
  // batch's own range of the shared K axis; an empty range yields an all-zero output tile.
  auto tile_krange = [&](int b, int sp, int& lo, int& hi) {
    if (args.kblock_range) {
      lo = args.kblock_range[2 * b];
      hi = args.kblock_range[2 * b + 1];
    } else {
      lo = sp * kb_per_split;
      hi = min(kb_total, lo + kb_per_split);
    }
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0 && is_gather_cta) {
      // Bulk-copy ring: peer global -> shared (mbarrier) -> local global (bulk group). The pipeline
      // stages are unused in this CTA and serve as the ring; loads run kSlots-2 chunks ahead.
      constexpr int kSlots = (kStages * Plan::kStageBytes / kGatherChunk) < kGatherSlotsMax
                                 ? (kStages * Plan::kStageBytes / kGatherChunk) : kGatherSlotsMax;
      constexpr int kLag = kSlots - 2;
      const uint32_t bar_g = tmem_slot + 8;
      for (int s2 = 0; s2 < kSlots; ++s2) mbar_init(bar_g + 8 * s2, 1);
      mbar_fence_init();
      // a block = 128 rows of A (mode 0) or one 64-row K slab of B (mode 1); both are contiguous
      const int blk_rows = args.ag_mode == 0 ? BM : BK;
      const int n_blocks = args.ag_mode == 0 ? num_m : args.kblocks0;
      const int per_rank = args.ag_rows / blk_rows;
      const int n_remote = n_blocks - per_rank;
      const int gidx = static_cast<int>(blockIdx.x) - n_compute;
      const long long block_bytes = static_cast<long long>(blk_rows) * args.ag_k * 2;
      const int chunks = static_cast<int>((block_bytes + kGatherChunk - 1) / kGatherChunk);
      const int my_blocks = n_remote > gidx ? (n_remote - gidx + n_gather - 1) / n_gather : 0;
      // One cursor for the loads and one for the stores: (block, chunk) advance by increments only,
      // the block's addresses are resolved once per block (no division per chunk in this thread).
      struct Cursor {
        int blk, ch, mb, slot;
        uint32_t parity;
        const char* src;
        char* dst;
      };
      auto open_block = [&](Cursor& c) {
        int i = gidx + c.blk * n_gather;  // remote blocks in the order the raster consumes them
        int mb = (args.ag_rank + 1) * per_rank + i;
        while (mb >= n_blocks) mb -= n_blocks;
        int owner = 0, first = 0;
        while (first + per_rank <= mb) { first += per_rank; ++owner; }
        c.mb = mb;
        c.src = static_cast<const char*>(args.ag_src[owner]) + static_cast<long long>(mb - first) * block_bytes;
        c.dst = static_cast<char*>(args.ag_dst) + static_cast<long long>(mb) * block_bytes;
      };
      auto advance = [&](Cursor& c) {
        if (++c.slot == kSlots) { c.slot = 0; c.parity ^= 1u; }
        if (++c.ch == chunks) { c.ch = 0; ++c.blk; if (c.blk < my_blocks) open_block(c); }
      };
      Cursor ld{0, 0, 0, 0, 0u, nullptr, nullptr}, st{0, 0, 0, 0, 0u, nullptr, nullptr};
      if (my_blocks > 0) { open_block(ld); open_block(st); }
      const int total = my_blocks * chunks;
      bool ok = true;
      for (int it = 0; it < total + kLag && ok; ++it) {
        if (it < total) {
          const long long off = static_cast<long long>(ld.ch) * kGatherChunk;
          const uint32_t bytes = static_cast<uint32_t>(block_bytes - off < kGatherChunk ? block_bytes - off : kGatherChunk);
          // the store that last read this slot was committed kSlots - kLag - 1 = 1 group ago
          asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          mbar_expect_tx(bar_g + 8 * ld.slot, bytes);
          asm volatile(
              "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
              ::"r"(smem_a + ld.slot * kGatherChunk), "l"(ld.src + off), "r"(bytes), "r"(bar_g + 8 * ld.slot) : "memory");
          advance(ld);
        }
        if (it >= kLag) {
          const long long off = static_cast<long long>(st.ch) * kGatherChunk;
          const uint32_t bytes = static_cast<uint32_t>(block_bytes - off < kGatherChunk ? block_bytes - off : kGatherChunk);
          if (!mbar_wait(bar_g + 8 * st.slot, st.parity, abort_flag)) {
            if (args.status) atomicCAS(args.status, 0, kTimeoutPeerFlag);
            ok = false;
            break;
          }
          asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                       ::"l"(st.dst + off), "r"(smem_a + st.slot * kGatherChunk), "r"(bytes) : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          if (st.ch == chunks - 1) {  // the whole block has landed: publish it to the producers of every CTA
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            asm volatile("fence.proxy.async;" ::: "memory");
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(args.ag_flags + st.mb), "r"(args.ag_seq) : "memory");
          }
          advance(st);
        }
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    } else if (!is_gather_cta) {
      // The whole warp walks the loop with identical values, and one elected lane issues the copies: the
      // loop state then lives in uniform registers, which is where the TMA instructions take their operands
      // from. (A loop run by a single diverged lane pays a register-to-uniform move per operand per copy.)
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      unsigned long long landed = 0ull;  // mode 1: K slabs (< 64) already seen complete
      auto wait_block = [&](int idx) {  // lane 0 polls the flag, the warp takes its verdict
        int good = 1;
        if (lane == 0) {
          const unsigned long long t0 = globaltimer_ns();
          while (true) {
            unsigned int f;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(f) : "l"(args.ag_flags + idx) : "memory");
            if (f == args.ag_seq) break;
            if (*abort_flag || globaltimer_ns() - t0 > kWaitLimitNs) {
              *abort_flag = 1;
              if (args.status) atomicCAS(args.status, 0, kTimeoutPeerFlag);
              good = 0;
              break;
            }
          }
          asm volatile("fence.proxy.async.global;" ::: "memory");  // bulk-copy writes -> TMA reads
        }
        return __shfl_sync(0xffffffffu, good, 0) != 0;
      };
      const bool ag_b = args.ag_world > 1 && args.ag_mode == 1;
      const int ag_per_rank = args.ag_world > 1 ? args.ag_rows / (ag_b ? BK : BM) : 1;
      const int ag_lo = args.ag_rank * ag_per_rank, ag_hi = ag_lo + ag_per_rank;  // this rank's own blocks
      int tile_idx = 0;
      for (long long t = tile0; t < num_tiles && ok; t += tstride, ++tile_idx) {
        int b, mb, nb, sp;
        decode(t, b, mb, nb, sp);
        int kb_lo, kb_hi;
        tile_krange(b, sp, kb_lo, kb_hi);
        const int bb = args.bgroup_of_mblock ? args.bgroup_of_mblock[mb] : b;
        if (bb < 0) continue;  // padding row block of a grouped product: no tile
        const int ab = args.a_bcast ? 0 : b;
        const int bbatch = args.b_bcast ? 0 : bb;
        if (args.ag_world > 1 && args.ag_mode == 0 && (mb < ag_lo || mb >= ag_hi)) {
          // remote row block: wait (bounded) until a gather CTA has landed it locally
          if (!wait_block(mb)) {
            ok = false;
            break;
          }
        }
        const int n0 = nb * BN + static_cast<int>(cta_rank) * (BN / CG);  // this CTA's share of the B tile
        for (int kbi = kb_lo; kbi < kb_hi; ++kbi) {
          int kb = kbi;
          if (ag_b) {  // this rank's own K slabs first, then the peers' in the order they arrive
            kb = kbi + ag_lo;
            if (kb >= args.kblocks0) kb -= args.kblocks0;
            if ((kb < ag_lo || kb >= ag_hi) && !(kb < 64 && ((landed >> kb) & 1ull))) {
              if (!wait_block(kb)) {
                ok = false;
                break;
              }
              if (kb < 64) landed |= 1ull << kb;
            }
          }
          if (args.probe & 4) continue;  // MMA-rate probe: no operand handshake at all
          if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag))) {
            if (args.status && lane == 0) atomicCAS(args.status, 0, kTimeoutProducer);
            ok = false;
            break;
          }
          const bool p1 = kb >= args.kblocks0;
          const int k0 = (p1 ? kb - args.kblocks0 : kb) * BK;
          const CUtensorMap* ta = p1 ? &tmA1 : &tmA0;
          const CUtensorMap* tb = p1 ? &tmB1 : &tmB0;
          const int a_mn = p1 ? args.a_mn1 : args.a_mn0;
          const int b_mn = p1 ? args.b_mn1 : args.b_mn0;
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t sa = smem_a + stage * kStageBytesA;
          const uint32_t sb = smem_b + stage * kStageBytesB;
          if (elect_one_sync()) {
            if (args.probe & 1) {
              if (leader) mbar_arrive(full);
            } else {
              // pair: the leader's barrier collects the bytes of both CTAs' copies
              if (leader) mbar_expect_tx(full, (kStageBytesA + kStageBytesB) * CG);
              auto load = [&](uint32_t dst, const CUtensorMap* tm, int c0, int c1, int c2) {
                if constexpr (CG == 2)
                  tma_load_3d_pair(dst, tm, full, c0, c1, c2);
                else
                  tma_load_3d(dst, tm, full, c0, c1, c2);
              };
              if (!a_mn) {
                load(sa, ta, k0, mb * BM, ab);
              } else {
#pragma unroll
                for (int i = 0; i < BM / 64; ++i) load(sa + i * (BK * 128), ta, mb * BM + 64 * i, k0, ab);
              }
              if (!b_mn) {
                load(sb, tb, k0, n0, bbatch);
              } else {
#pragma unroll
                for (int i = 0; i < BN / 64 / CG; ++i) load(sb + i * (BK * 128), tb, n0 + 64 * i, k0, bbatch);
              }
            }
          }
          if (++stage == nstages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (lane == 0) stamp(144 + tile_idx);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (leader) {
      // Warp-uniform loop, one elected lane issues (see the producer): descriptors and barrier addresses
      // stay in uniform registers.
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      // per K phase: instruction descriptor, the descriptor bits above the address, the address step per K = 16.
      // One instruction covers K = 16: 32 B along a K-major swizzle row, or two 8-row groups (2048 B) of an
      // MN-major tile. The address field counts 16-byte units.
      const uint32_t idesc0 = make_idesc_bf16(BM * CG, BN, args.a_mn0, args.b_mn0);
      const uint32_t idesc1 = make_idesc_bf16(BM * CG, BN, args.a_mn1, args.b_mn1);
      const uint64_t a_hi0 = make_smem_desc(0, args.a_mn0 ? BK * 128 : 16, 1024);
      const uint64_t a_hi1 = make_smem_desc(0, args.a_mn1 ? BK * 128 : 16, 1024);
      const uint64_t b_hi0 = make_smem_desc(0, args.b_mn0 ? BK * 128 : 16, 1024);
      const uint64_t b_hi1 = make_smem_desc(0, args.b_mn1 ? BK * 128 : 16, 1024);
      const uint32_t a_step0 = args.a_mn0 ? (2048 >> 4) : (32 >> 4), a_step1 = args.a_mn1 ? (2048 >> 4) : (32 >> 4);
      const uint32_t b_step0 = args.b_mn0 ? (2048 >> 4) : (32 >> 4), b_step1 = args.b_mn1 ? (2048 >> 4) : (32 >> 4);
      int tile_idx = 0;
      for (long long t = tile0; t < num_tiles && ok; t += tstride, ++tile_idx) {
        int b, mb, nb, sp;
        decode(t, b, mb, nb, sp);
        int kb_lo, kb_hi;
        tile_krange(b, sp, kb_lo, kb_hi);
        if (args.bgroup_of_mblock && args.bgroup_of_mblock[mb] < 0) continue;
        if (!__all_sync(0xffffffffu, mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag))) {
          if (args.status && lane == 0) atomicCAS(args.status, 0, kTimeoutMma);
          break;
        }
        tc_fence_after();
        if (lane == 0) stamp(16 + 2 * tile_idx);
        const uint32_t tmem_d = tmem_base + acc * BN;
        uint32_t accumulate = 0u;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!(args.probe & 4) &&
              !__all_sync(0xffffffffu, mbar_wait(bar_full + 8 * stage, phase, abort_flag))) {
            if (args.status && lane == 0) atomicCAS(args.status, 0, kTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after();
          const bool p1 = kb >= args.kblocks0;
          const uint32_t idesc = p1 ? idesc1 : idesc0;
          const uint32_t sa = smem_a + stage * kStageBytesA;
          const uint32_t sb = smem_b + stage * kStageBytesB;
          const uint64_t adesc = (p1 ? a_hi1 : a_hi0) | static_cast<uint64_t>((sa & 0x3FFFF) >> 4);
          const uint64_t bdesc = (p1 ? b_hi1 : b_hi0) | static_cast<uint64_t>((sb & 0x3FFFF) >> 4);
          const uint32_t a_step = p1 ? a_step1 : a_step0;
          const uint32_t b_step = p1 ? b_step1 : b_step0;
          if (elect_one_sync()) {
            if (!(args.probe & 2)) {
#pragma unroll
              for (int k = 0; k < BK / 16; ++k) {
                if constexpr (CG == 2)
                  umma_bf16_pair(tmem_d, adesc + k * a_step, bdesc + k * b_step, idesc, k > 0 ? 1u : accumulate);
                else
                  umma_bf16(tmem_d, adesc + k * a_step, bdesc + k * b_step, idesc, k > 0 ? 1u : accumulate);
              }
            }
            if (!(args.probe & 4)) {
              if constexpr (CG == 2)
                umma_commit_pair(bar_empty + 8 * stage);
              else
                umma_commit(bar_empty + 8 * stage);
            }
          }
          accumulate = 1u;
          if (++stage == nstages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (elect_one_sync()) {
          if constexpr (CG == 2)
            umma_commit_pair(bar_tfull + 8 * acc);
          else
            umma_commit(bar_tfull + 8 * acc);
        }
        if (lane == 0) stamp(17 + 2 * tile_idx);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    if constexpr (NOUT == 4) {
      // TMA-fed mask epilogue (EPI_MASK_FWD / EPI_MASK_BWD on dense sites). Unit = one 64-column box of this
      // warp's 32 rows; ring of two slots, slot = {box_a: ci in, A / dH out; box_b: H in (bwd), dci or H out}.
      static_assert(EPI == EPI_MASK_FWD || EPI == EPI_MASK_BWD, "TMA-fed epilogue is for the mask epilogues");
      const int ew = warp - 2, q = warp & 3, grp = ew >> 2;
      const uint32_t ring = smem_out + ew * (4 * kOutBoxBytes);
      const uint32_t bar_in = smem_bar + 256 + ew * 16;
      constexpr bool kBwd = (EPI == EPI_MASK_BWD);
      const bool want_h = kBwd && args.dci != nullptr;           // H comes in, the mask gradient goes out
      const bool h_out = !kBwd && args.has_out1;                  // forward: H goes out through box_b
      const uint32_t in_bytes = kOutBoxBytes * (want_h ? 2 : 1);
      unsigned long long philox_seed = args.seed;
      if (args.seed_dev != nullptr) philox_seed = *args.seed_dev;
      if (lane == 0) {
        mbar_init(bar_in, 1);
        mbar_init(bar_in + 8, 1);
        mbar_fence_init();
      }
      __syncwarp();
      constexpr int nboxes = BN / 64;
      auto tile_is_real = [&](long long t) {
        if (!args.bgroup_of_mblock) return true;
        int b2, mb2, nb2, sp2;
        decode(t, b2, mb2, nb2, sp2);
        return args.bgroup_of_mblock[mb2] >= 0;
      };
      auto next_real_tile = [&](long long t) {
        while (t < num_tiles && !tile_is_real(t)) t += tstride;
        return t;
      };
      // first unit of this warp at or after tile t (a warp may own no column of a narrow tail tile)
      auto first_unit_from = [&](long long t) {
        t = next_real_tile(t);
        while (t < num_tiles) {
          int b2, mb2, nb2, sp2;
          decode(t, b2, mb2, nb2, sp2);
          if (nb2 * BN + grp * 64 < args.N) break;
          t = next_real_tile(t + tstride);
        }
        return t;
      };
      // Called by the whole warp (coordinates in uniform registers); one elected lane issues. `after_stores`:
      // first wait until the TMA stores that still read the destination slot have finished reading.
      auto issue_load = [&](long long t, int j, int slot, bool after_stores) {
        int b2 = 0, mb2 = 0, nb2 = 0, sp2 = 0;
        const bool real = t < num_tiles;  // past the last tile only the wait remains
        if (real) decode(t, b2, mb2, nb2, sp2);
        const int crow = mb2 * BM + q * 32, col0 = nb2 * BN + j * 64;
        const uint32_t bar = bar_in + 8 * slot, box_a = ring + slot * (2 * kOutBoxBytes);
        if (elect_one_sync()) {
          if (after_stores) tma_store_wait_read<0>();
          if (real) {
            mbar_expect_tx(bar, in_bytes);
            tma_load_3d(box_a, &tmCi, bar, col0, crow, 0);
            if (want_h) tma_load_3d(box_a + kOutBoxBytes, &tmH, bar, col0, crow, 0);
          }
        }
      };
      int acc = 0;
      uint32_t acc_phase = 0;
      uint32_t unit = 0;  // units consumed so far by this warp: slot = unit & 1, parity = (unit >> 1) & 1
      {
        const long long t0u = first_unit_from(tile0);
        issue_load(t0u, grp, 0, false);
      }
      bool failed = false;
      for (long long t = next_real_tile(tile0); t < num_tiles && !failed; t = next_real_tile(t + tstride)) {
        int b, mb, nb, sp;
        decode(t, b, mb, nb, sp);
        int kb_lo_e, kb_hi_e;
        tile_krange(b, sp, kb_lo_e, kb_hi_e);
        const bool empty_k = kb_hi_e <= kb_lo_e;
        const int row = mb * BM + q * 32 + lane;
        const bool row_ok = row < args.M;
        const uint32_t tmem_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
        float delta = 0.0f, rs = 1.0f;
        if (row_ok) {
          if (args.delta) delta = args.delta[row];
          if (args.rowscale) rs = args.rowscale[row];
        }
        bool have_acc = false;
        if (args.timeline != nullptr && warp == 2 && lane == 0 && unit < 16) stamp(240 + static_cast<int>(unit >> 1));
        const long long t_next = first_unit_from(t + tstride);  // the tile whose first unit follows this tile's last
#pragma unroll 1
        for (int j = grp; j < nboxes && !failed; j += 2) {
          const int col0 = nb * BN + j * 64;
          if (col0 >= args.N) break;  // uniform across the warp
          const int slot = unit & 1;
          const uint32_t box_a = ring + slot * (2 * kOutBoxBytes), box_b = box_a + kOutBoxBytes;
          if (!mbar_wait(bar_in + 8 * slot, (unit >> 1) & 1, abort_flag)) {
            if (args.status && lane == 0) atomicCAS(args.status, 0, kTimeoutEpilogue);
            failed = true;
            break;
          }
          const bool tl_on = args.timeline != nullptr && warp == 2 && lane == 0 && unit < 8;  // slots 176 .. 238
          if (tl_on) stamp(176 + 8 * static_cast<int>(unit));  // operands of the unit have landed
          if (!have_acc) {
            if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag)) {
              if (args.status && lane == 0) atomicCAS(args.status, 0, kTimeoutEpilogue);
              failed = true;
              break;
            }
            tc_fence_after();
            have_acc = true;
          }
          if (tl_on) stamp(177 + 8 * static_cast<int>(unit));  // accumulator ready
          const f32x2 rs2 = pk2(rs, rs), ndelta2 = pk2(-delta, -delta), one2 = pk2(1.0f, 1.0f), neg2 = pk2(-1.0f, -1.0f);
          // One half (32 columns) of the unit: all shared-memory loads first, then the arithmetic of the four
          // 8-column groups as plain code (four independent Philox chains the scheduler can interleave), then all
          // stores. The loads and stores are `asm volatile` (they must stay behind the barrier waits), so they
          // are kept in two blocks instead of fencing each group's arithmetic from the next.
          auto do_half = [&](const int half) {
            const int c0 = col0 + 32 * half;
            uint32_t r[32];
            tmem_ld_32x32(tmem_row + j * 64 + 32 * half, r);
            uint4 ciq[4], hq[4];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const uint32_t off = lane * 128 + (((half * 4 + g) ^ (lane & 7)) << 4);
              asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(ciq[g].x), "=r"(ciq[g].y), "=r"(ciq[g].z), "=r"(ciq[g].w) : "r"(box_a + off) : "memory");
              hq[g] = make_uint4(0u, 0u, 0u, 0u);
              if (want_h)
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(hq[g].x), "=r"(hq[g].y), "=r"(hq[g].z), "=r"(hq[g].w) : "r"(box_b + off) : "memory");
            }
            tmem_ld_wait();
            uint32_t out_a[4][4], out_b[4][4];
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const uint32_t ciw[4] = {ciq[g].x, ciq[g].y, ciq[g].z, ciq[g].w}, hw[4] = {hq[g].x, hq[g].y, hq[g].z, hq[g].w};
              f32x2 v2[4], coef2[4], dmdci2[4];
#pragma unroll
              for (int i = 0; i < 4; ++i)
                v2[i] = empty_k ? pk2(0.0f, 0.0f) : pk2u(r[8 * g + 2 * i], r[8 * g + 2 * i + 1]);
              if (args.mask_mode == 0) {
                const uint4 pr = Philox::run(
                    make_uint4(static_cast<uint32_t>((c0 >> 3) + g) + (args.philox_col0 >> 3),
                               static_cast<uint32_t>(row) + args.row_offset, args.stream, 0x5044u),
                    make_uint2(static_cast<uint32_t>(philox_seed), static_cast<uint32_t>(philox_seed >> 32)));
                const uint32_t pw[4] = {pr.x, pr.y, pr.z, pr.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const f32x2 u2 = philox_word_to_unit2(pw[i]);
                  const f32x2 om2 = fma2(u2, neg2, one2);                       // 1 - u
                  const f32x2 m2 = fma2(unpack_bf16_2(ciw[i]), om2, u2);        // ci (1 - u) + u
                  coef2[i] = mul2(rs2, add2(m2, ndelta2));
                  dmdci2[i] = mul2(rs2, om2);
                }
              } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  coef2[i] = mul2(rs2, add2(unpack_bf16_2(ciw[i]), ndelta2));
                  dmdci2[i] = rs2;
                }
              }
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                out_a[g][i] = pack_bf16_2(mul2(v2[i], coef2[i]));  // masked product
                if constexpr (kBwd)
                  out_b[g][i] = pack_bf16_2(mul2(mul2(v2[i], unpack_bf16_2(hw[i])), dmdci2[i]));  // mask gradient
                else
                  out_b[g][i] = pack_bf16_2(v2[i]);  // forward: the unmasked product
              }
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const uint32_t off = lane * 128 + (((half * 4 + g) ^ (lane & 7)) << 4);
              if (kBwd ? want_h : h_out)  // box_b: the mask gradient replaces H (backward), or H goes out (forward)
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(box_b + off), "r"(out_b[g][0]),
                             "r"(out_b[g][1]), "r"(out_b[g][2]), "r"(out_b[g][3]) : "memory");
              // box_a: the masked product replaces this thread's ci values
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(box_a + off), "r"(out_a[g][0]),
                           "r"(out_a[g][1]), "r"(out_a[g][2]), "r"(out_a[g][3]) : "memory");
            }
          };
          do_half(0);
          if (tl_on) stamp(179 + 8 * static_cast<int>(unit));  // first half computed
          {
            // The other slot's boxes were handed to TMA stores one unit ago: once those have been read,
            // request the NEXT unit's operands into it (they land while this unit's second half is computed).
            long long tn = t;
            int jn = j + 2;
            if (!(jn < nboxes && nb * BN + jn * 64 < args.N)) {
              tn = t_next;
              jn = grp;
            }
            issue_load(tn, jn, slot ^ 1, true);
          }
          __syncwarp();
          if (tl_on) stamp(180 + 8 * static_cast<int>(unit));  // previous stores read, next operands requested
          do_half(1);
          if (tl_on) stamp(181 + 8 * static_cast<int>(unit));  // second half computed
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int crow = mb * BM + q * 32;
            if (crow < args.M) {
              tma_store_3d(&tmOut0, box_a, col0, crow, b);
              if (want_h) tma_store_3d(&tmDci, box_b, col0, crow, 0);
              if (h_out) tma_store_3d(&tmOut1, box_b, col0, crow, b);
            }
            tma_store_commit();
          }
          if (tl_on) stamp(182 + 8 * static_cast<int>(unit));  // stores issued
          ++unit;
        }
        if (failed) break;
        if (!have_acc) {  // no column of this tile fell to this warp: still consume the phase
          if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag)) {
            if (args.status && lane == 0) atomicCAS(args.status, 0, kTimeoutEpilogue);
            break;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (CG == 2 && !leader)
            mbar_arrive_cluster(mapa_shared(bar_tempty + 8 * acc, 0));
          else
            mbar_arrive(bar_tempty + 8 * acc);
        }
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
      if (lane == 0) tma_store_wait_all<0>();
    } else {
    // Work unit = a 32-column half of an output box. Global operands of the mask epilogues
    // (ci / W rows, and H rows in the backward) are requested one unit ahead, across box and tile
    // boundaries, so their latency hides behind the math of the previous unit.
    const int ew = warp - 2;   // 0..7
    const int q = warp & 3;    // TMEM lane quarter this warp may read
    const int grp = ew >> 2;   // the two warps of a quarter take alternate boxes
    const uint32_t box0 = smem_out + ew * (NOUT * kOutBoxBytes);
    const uint32_t box1 = box0 + (NOUT - 1) * kOutBoxBytes;
    int acc = 0;
    uint32_t acc_phase = 0;
    float faith_acc = 0.0f;
    const bool out32 = (EPI == EPI_PLAIN) && args.out_fp32;
    const int box_cols = out32 ? 32 : 64;
    const int nboxes = BN / box_cols;
    const int halves = out32 ? 1 : 2;
    const bool plain_fast = (EPI == EPI_PLAIN) && args.bias == nullptr && args.act == ACT_NONE &&
                            args.alpha == 1.0f && args.alpha_dev == nullptr;
    const float alpha_eff = (EPI == EPI_PLAIN && args.alpha_dev != nullptr) ? args.alpha * *args.alpha_dev : args.alpha;
    constexpr bool kWantH = (EPI == EPI_MASK_BWD);
    const bool want_h = kWantH && args.dci != nullptr;
    unsigned long long philox_seed = args.seed;
    if constexpr (EPI == EPI_MASK_FWD || EPI == EPI_MASK_BWD) {
      if (args.seed_dev != nullptr) philox_seed = *args.seed_dev;
    }

    auto tile_is_real = [&](long long t) {
      if (!args.bgroup_of_mblock) return true;
      int b2, mb2, nb2, sp2;
      decode(t, b2, mb2, nb2, sp2);
      return args.bgroup_of_mblock[mb2] >= 0;
    };
    auto next_real_tile = [&](long long t) {
      while (t < num_tiles && !tile_is_real(t)) t += tstride;
      return t;
    };
    uint4 pre_ci[4], pre_h[4];
    // Request the operands of unit (t, j, half); silently does nothing past the end.
    auto issue_prefetch = [&](long long t, int j, int half) {
      if constexpr (EPI != EPI_PLAIN) {
        if (t >= num_tiles) return;
        int b2, mb2, nb2, sp2;
        decode(t, b2, mb2, nb2, sp2);
        const int prow = mb2 * BM + q * 32 + lane;
        const int pcol = nb2 * BN + j * box_cols + 32 * half;
        bool ok_row = prow < args.M;
        long long src = prow;
        int colb = 0;
        if (args.rowmap != nullptr && ok_row) {
          const int4 pm = __ldg(args.rowmap + prow);
          src = pm.x;
          colb = pm.y;
          ok_row = pm.x >= 0;
        }
        const __nv_bfloat16* ci_row = args.ci + src * args.ld_ci + colb + pcol;
#pragma unroll
        for (int g = 0; g < 4; ++g)
          pre_ci[g] = (ok_row && pcol + 8 * g < args.N) ? __ldg(reinterpret_cast<const uint4*>(ci_row + 8 * g))
                                                        : make_uint4(0u, 0u, 0u, 0u);
        if (want_h) {
          const __nv_bfloat16* h_row = args.H + static_cast<long long>(prow) * args.ld_h + pcol;
#pragma unroll
          for (int g = 0; g < 4; ++g)
            pre_h[g] = (ok_row && pcol + 8 * g < args.N) ? __ldg(reinterpret_cast<const uint4*>(h_row + 8 * g))
                                                         : make_uint4(0u, 0u, 0u, 0u);
        }
      }
    };
    // First unit this warp owns at or after tile t (a warp may own no column of a narrow tail tile).
    auto first_unit_from = [&](long long t, long long& t_out, int& j_out) {
      t = next_real_tile(t);
      while (t < num_tiles) {
        int b2, mb2, nb2, sp2;
        decode(t, b2, mb2, nb2, sp2);
        if (nb2 * BN + grp * box_cols < args.N) break;
        t = next_real_tile(t + tstride);
      }
      t_out = t;
      j_out = grp;
    };
    {
      long long tp;
      int jp;
      first_unit_from(tile0, tp, jp);
      issue_prefetch(tp, jp, 0);
    }

    for (long long t = next_real_tile(tile0); t < num_tiles; t = next_real_tile(t + tstride)) {
      int b, mb, nb, sp;
      decode(t, b, mb, nb, sp);
      int kb_lo_e, kb_hi_e;
      tile_krange(b, sp, kb_lo_e, kb_hi_e);
      const bool empty_k = kb_hi_e <= kb_lo_e;
      const int row = mb * BM + q * 32 + lane;
      bool row_ok = row < args.M;
      long long src_row = row;  // where this row's mask inputs live (differs from `row` on job rows)
      int src_col = 0;
      const uint32_t tmem_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      float delta = 0.0f, rs = 1.0f;
      if constexpr (EPI != EPI_PLAIN) {
        if (args.rowmap != nullptr && row_ok) {
          const int4 rm = __ldg(args.rowmap + row);
          src_row = rm.x;
          src_col = rm.y;
          row_ok = rm.x >= 0;
        }
        if (row_ok) {
          if (args.delta) delta = args.delta[src_row];
          if (args.rowscale) rs = args.rowscale[src_row];
        }
      }
      bool have_acc = false;
      bool failed = false;
#pragma unroll 1
      for (int j = grp; j < nboxes && !failed; j += 2) {
        const int col0 = nb * BN + j * box_cols;
        if (col0 >= args.N) break;  // uniform across the warp
#pragma unroll 1
        for (int half = 0; half < halves; ++half) {
          const int c0 = col0 + 32 * half;
          if (c0 >= args.N) break;
          uint4 ciq[4], hq[4];
          if constexpr (EPI != EPI_PLAIN) {
#pragma unroll
            for (int g = 0; g < 4; ++g) ciq[g] = pre_ci[g];
            if constexpr (kWantH) {
#pragma unroll
              for (int g = 0; g < 4; ++g) hq[g] = pre_h[g];
            }
            // the unit after this one: other half, next box of this tile, or first unit of a later tile
            if (half + 1 < halves && c0 + 32 < args.N) {
              issue_prefetch(t, j, half + 1);
            } else if (j + 2 < nboxes && nb * BN + (j + 2) * box_cols < args.N) {
              issue_prefetch(t, j + 2, 0);
            } else {
              long long tn;
              int jn;
              first_unit_from(t + tstride, tn, jn);
              issue_prefetch(tn, jn, 0);
            }
          }
          if (!have_acc) {
            bool got = true;
            if (args.probe & 16) {  // one lane polls; the others park at the warp shuffle
              if (lane == 0) got = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag);
              got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
            } else {
              got = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag);
            }
            if (!got) {
              if (args.status && lane == 0) atomicCAS(args.status, 0, kTimeoutEpilogue);
              failed = true;
              break;
            }
            tc_fence_after();
            have_acc = true;
            if (args.timeline != nullptr && warp == 2 && lane == 0) stamp(80 + 2 * static_cast<int>((t - tile0) / tstride));
          }
          uint32_t r[32];
          tmem_ld_32x32(tmem_row + j * box_cols + 32 * half, r);
          tmem_ld_wait();
          if (half == 0) {
            // The staging boxes were handed to TMA one box ago: make sure they have been read.
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
          }
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = empty_k ? 0.0f : __uint_as_float(r[i]);

          if constexpr (EPI == EPI_PLAIN) {
            if (!plain_fast) {
              const float* bias = args.bias ? args.bias + b * args.bias_bs : nullptr;
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                float x = v[i] * alpha_eff;
                if (bias && c0 + i < args.N) x += bias[c0 + i];
                v[i] = x;
              }
              if (args.act == ACT_GELU) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = apply_act(v[i], ACT_GELU);
              } else if (args.act == ACT_SILU) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = apply_act(v[i], ACT_SILU);
              } else if (args.act == ACT_RELU) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = fmaxf(v[i], 0.0f);
              }
            }
            if (out32)
              stage_fp32(box0, lane, v);
            else
              stage_bf16_half(box0, lane, half, v);
          } else if constexpr (EPI == EPI_FAITH) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float rf[8];
              unpack8(ciq[g], rf);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float dlt = rf[i] - v[8 * g + i];
                v[8 * g + i] = dlt;
                faith_acc += dlt * dlt;
              }
            }
            stage_bf16_half(box0, lane, half, v);
          } else {
            if constexpr (EPI == EPI_MASK_FWD) {
              if (NOUT == 2 && args.has_out1) stage_bf16_half(box1, lane, half, v);
            }
            // eight columns at a time: mask, its derivative, products; nothing wider stays live
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float cf[8], coef[8], dmdci[8];
              unpack8(ciq[g], cf);
              if (args.mask_mode == 0) {
                float u[8];
                philox_uniform8(philox_seed, args.stream, static_cast<uint32_t>(src_row) + args.row_offset,
                                static_cast<uint32_t>(((src_col + c0) >> 3) + g) + (args.philox_col0 >> 3), u);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  const float om = 1.0f - u[i];
                  coef[i] = rs * (fmaf(cf[i], om, u[i]) - delta);  // ci + (1-ci) u - d
                  dmdci[i] = rs * om;
                }
              } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  coef[i] = rs * (cf[i] - delta);
                  dmdci[i] = rs;
                }
              }
              if constexpr (EPI == EPI_MASK_BWD) {
                if (want_h && row_ok && c0 + 8 * g < args.N) {
                  float hf[8], tt[8];
                  unpack8(hq[g], hf);
#pragma unroll
                  for (int i = 0; i < 8; ++i) tt[i] = v[8 * g + i] * hf[i] * dmdci[i];
                  if (args.dci_bf16) {
                    __nv_bfloat16* dstb = reinterpret_cast<__nv_bfloat16*>(args.dci) +
                                          src_row * args.ld_dci + src_col + c0 + 8 * g;
                    if (args.dci_accumulate) {
                      float old8[8];
                      unpack8(*reinterpret_cast<const uint4*>(dstb), old8);
#pragma unroll
                      for (int i = 0; i < 8; ++i) tt[i] += old8[i];
                    }
                    uint4 pk;
                    pk.x = pack_bf16(tt[0], tt[1]); pk.y = pack_bf16(tt[2], tt[3]);
                    pk.z = pack_bf16(tt[4], tt[5]); pk.w = pack_bf16(tt[6], tt[7]);
                    *reinterpret_cast<uint4*>(dstb) = pk;
                  } else {
                    float* dst = args.dci + src_row * args.ld_dci + src_col + c0 + 8 * g;
                    float4 o0 = make_float4(tt[0], tt[1], tt[2], tt[3]), o1 = make_float4(tt[4], tt[5], tt[6], tt[7]);
                    if (args.dci_accumulate) {
                      const float4 p0 = *reinterpret_cast<float4*>(dst), p1 = *reinterpret_cast<float4*>(dst + 4);
                      o0.x += p0.x; o0.y += p0.y; o0.z += p0.z; o0.w += p0.w;
                      o1.x += p1.x; o1.y += p1.y; o1.z += p1.z; o1.w += p1.w;
                    }
                    *reinterpret_cast<float4*>(dst) = o0;
                    *reinterpret_cast<float4*>(dst + 4) = o1;
                  }
                }
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) v[8 * g + i] *= coef[i];
            }
            stage_bf16_half(box0, lane, half, v);
          }
        }
        if (failed) break;

        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int crow = mb * BM + q * 32;
          if (crow < args.M) {
            if (args.rs_world > 1) {
              const int owner = crow / args.rs_rows;
              tma_reduce_add_3d(&peerOut.m[owner], box0, col0, crow - owner * args.rs_rows, b);
            } else if (args.accumulate)
              tma_reduce_add_3d(&tmOut0, box0, col0, crow, b);
            else
              tma_store_3d(&tmOut0, box0, col0, crow, b);
            if constexpr (EPI == EPI_MASK_FWD && NOUT == 2) {
              if (args.has_out1) tma_store_3d(&tmOut1, box1, col0, crow, b);
            }
          }
          tma_store_commit();
        }
      }
      if (failed) break;
      if (!have_acc) {  // no column of this tile fell to this warp: still consume the phase
        if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag)) {
          if (args.status && lane == 0) atomicCAS(args.status, 0, kTimeoutEpilogue);
          break;
        }
      }
      // Accumulator drained by this warp: hand it back to the MMA warp.
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CG == 2 && !leader)
          mbar_arrive_cluster(mapa_shared(bar_tempty + 8 * acc, 0));  // the MMA issuer lives in the leader
        else
          mbar_arrive(bar_tempty + 8 * acc);
        if (args.timeline != nullptr && warp == 2) stamp(81 + 2 * static_cast<int>((t - tile0) / tstride));
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if constexpr (EPI == EPI_FAITH) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) faith_acc += __shfl_xor_sync(0xffffffffu, faith_acc, o);
      if (lane == 0 && args.dci != nullptr) atomicAdd(args.dci, faith_acc);
    }
    if (lane == 0) tma_store_wait_all<0>();
    }  // NOUT != 4
  }

  // Unwind: every role has left its loop (all waits are bounded). A producer that gave up may
  // still have loads in flight; give them a bounded grace period before the CTA's smem goes away.
  if (*abort_flag && warp == 0 && lane == 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) {
    }
  }
  if (threadIdx.x == 0) stamp(2);
  tc_fence_before();
  __syncthreads();
  // pair: neither CTA may retire while its partner can still signal its barriers or read its smem
  if constexpr (CG == 2) cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    if constexpr (CG == 2)
      tmem_dealloc_pair(tmem_base, kTmemCols);
    else
      tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) stamp(3);
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct OperandDesc {
  const void* ptr;      // bf16
  long long ld;         // elements between rows of the stored matrix
  long long batch_stride;
  int mn_major;         // 0: stored [rows=M|N, K]; 1: stored [rows=K, M|N]
};

static int g_num_sms = 0;
static long long* g_timeline = nullptr;  // pd_gemm_set_timeline(ptr): see GemmArgs::timeline
static int g_probe = 0;             // pd_gemm_set_probe(bits): timing probes, see GemmArgs::probe
static int g_stage_limit = 0;       // pd_gemm_set_stage_limit(n): probe of pipeline depth, 0 = all stages
static bool g_pair_default = true;  // pd_gemm_set_pair_default(0) turns automatic pairing off

static int encode_operand(CUtensorMap* tm, const OperandDesc& op, int mn_extent, int k_extent,
                          int batch, int box_rows_k_major) {
  if (!op.mn_major) {
    return encode_tmap(tm, op.ptr, 2, false, k_extent, mn_extent, op.ld, batch,
                       op.batch_stride, 64, box_rows_k_major);
  }
  return encode_tmap(tm, op.ptr, 2, false, mn_extent, k_extent, op.ld, batch, op.batch_stride, 64,
                     BK);
}

template <int BN, int EPI, int NOUT, int CG>
static int launch_gemm(const CUtensorMap& a0, const CUtensorMap& b0, const CUtensorMap& a1,
                       const CUtensorMap& b1, const CUtensorMap& o0, const CUtensorMap& o1,
                       const CUtensorMap& mci, const CUtensorMap& mh, const CUtensorMap& mdci,
                       const PeerMaps& peers, const GemmArgs& args, int max_ctas, cudaStream_t stream) {
  using Plan = SmemPlan<BN, NOUT, CG>;
  auto kern = gemm_kernel<BN, EPI, NOUT, CG>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Plan::kTotal);
    if (e != cudaSuccess) return 300 + static_cast<int>(e);
    configured = true;
  }
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const long long tiles = static_cast<long long>((args.M + BM * CG - 1) / (BM * CG)) *
                          ((args.N + BN - 1) / BN) * args.split_k * args.batch * CG;
  int grid = static_cast<int>(tiles < g_num_sms ? tiles : g_num_sms);
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  grid -= grid % CG;
  if (grid <= 0) return 0;
  GemmArgs launch_args = args;
  {  // magic numbers of the panel quotient (valid for dividends below 2^31)
    const unsigned long long d = static_cast<unsigned long long>(kGroupM) * ((args.N + BN - 1) / BN);
    unsigned int sh = 0;
    while ((1ull << sh) < d) ++sh;
    launch_args.pg_shift = sh;
    launch_args.pg_mul = static_cast<unsigned int>(((1ull << 32) * ((1ull << sh) - d)) / d + 1);
  }
  if (args.ag_world > 1) {
    // every CTA must be resident (producers wait on blocks that gather CTAs deliver): one per SM
    if (max_ctas > 0 && max_ctas < g_num_sms) return kBadArgument;
    grid = g_num_sms;
    int g = args.ag_gather_ctas > 0 ? args.ag_gather_ctas : (args.ag_mode == 1 ? 8 : 16);
    if (g > grid / 2) g = grid / 2;
    launch_args.ag_gather_ctas = g;
  }
  if constexpr (CG == 2) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kNumThreads);
    cfg.dynamicSmemBytes = Plan::kTotal;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, kern, a0, b0, a1, b1, o0, o1, mci, mh, mdci, peers, launch_args);
    return le == cudaSuccess ? 0 : 400 + static_cast<int>(le);
  }
  kern<<<grid, kNumThreads, Plan::kTotal, stream>>>(a0, b0, a1, b1, o0, o1, mci, mh, mdci, peers, launch_args);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + static_cast<int>(e);
}

}  // namespace pd

using namespace pd;

// C ABI -----------------------------------------------------------------------------------------
// All pointers are device pointers; `stream` is a cudaStream_t. Return value 0 = launched.
struct PdGemmCall {
  // problem
  int M, N, batch;
  int K0, K1;
  // operands of phase 0 and (if K1 > 0) phase 1
  const void* A0; long long lda0; long long bsa0; int a_mn0;
  const void* B0; long long ldb0; long long bsb0; int b_mn0;
  const void* A1; long long lda1; long long bsa1; int a_mn1;
  const void* B1; long long ldb1; long long bsb1; int b_mn1;
  // outputs
  void* out0; long long ldo0; long long bso0; int out_fp32; int accumulate;
  void* out1; long long ldo1; long long bso1;
  // plain epilogue
  float alpha; const float* bias; long long bias_bs; int act;
  // mask epilogues
  int epi;
  const void* ci; long long ld_ci;
  const void* H; long long ld_h;
  const float* delta; const float* rowscale;
  float* dci; long long ld_dci; int dci_accumulate; int dci_bf16;
  unsigned long long seed; unsigned int rng_stream; unsigned int rng_row_offset; int mask_mode;
  // control
  int split_k; int bn; int max_ctas;
  int* status;
  // Grouped products. bgroup_of_mblock[mb] (device, one int per 128-row block of the output):
  // batch index of the B operand for that row block (A and out are one ragged [rows, *] matrix whose
  // rows are sorted by group and padded to 128 per group); -1 = padding block, skipped.
  // kblock_range[2*b], [2*b+1] (device): 64-wide K-block range of batch b on a K axis shared by all
  // batches (ragged weight gradients: A/B are broadcast, a_bcast/b_bcast = 1).
  const int* bgroup_of_mblock; const int* kblock_range; int a_bcast; int b_bcast; int b_groups;
  // GEMM -> reduce-scatter over peer memory: rs_out[r] = rank r's fp32 [rs_rows, N] buffer (pitch ldo0)
  int rs_world; int rs_rows; void* rs_out[8];
  // all-gather -> GEMM: ag_src[r] = rank r's A shard [ag_rows, K0]; A0 is the local full buffer
  int ag_world; int ag_rank; int ag_rows; const void* ag_src[8]; unsigned int* ag_flags; unsigned int ag_seq;
  // ag_mode 1: ag_src[r] = rank r's K slab [ag_rows, N] of the MN-major B operand; B0 is the local full buffer
  int ag_mode; int ag_gather_ctas;
  int cta_group;  // 0 = automatic, 1 = single CTA tiles, 2 = CTA pairs where the call allows them
  const void* rowmap;  // [M] int4 {source row, first source column, 0, 0} for the mask epilogues, or null
  unsigned int philox_col0;  // global index of mask column 0 in the Philox counter space (multiple of 8)
  const unsigned long long* seed_dev;  // when set, overrides `seed` with the value in device memory at run time
  const float* alpha_dev;              // when set, the plain epilogue's scale is alpha * *alpha_dev
  int epi_tma;  // mask epilogues: 0 = TMA-fed form where the call allows it and K is short, 1 = never, 2 = whenever allowed
};

extern "C" int pd_gemm(const PdGemmCall* c, void* stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (c->M <= 0 || c->N <= 0 || c->batch <= 0 || c->K0 <= 0) return kBadArgument;
  if (c->epi != EPI_PLAIN && (c->batch != 1 || c->accumulate || c->out_fp32)) return kBadArgument;
  if (c->accumulate && !c->out_fp32) return kBadArgument;
  const int bn = c->bn == 128 ? 128 : 256;
  const int nout = (c->epi == EPI_MASK_FWD && c->out1 != nullptr) ? 2 : 1;

  GemmArgs a{};
  a.M = c->M; a.N = c->N; a.batch = c->batch;
  a.kblocks0 = (c->K0 + BK - 1) / BK;
  a.kblocks1 = c->K1 > 0 ? (c->K1 + BK - 1) / BK : 0;
  a.split_k = c->split_k > 0 ? c->split_k : 1;
  if (a.split_k > 1 && !(c->accumulate && c->epi == EPI_PLAIN && c->act == ACT_NONE &&
                         c->bias == nullptr))
    return kBadArgument;
  if (a.split_k > a.kblocks0 + a.kblocks1) a.split_k = a.kblocks0 + a.kblocks1;
  a.a_mn0 = c->a_mn0; a.b_mn0 = c->b_mn0; a.a_mn1 = c->a_mn1; a.b_mn1 = c->b_mn1;
  a.accumulate = c->accumulate; a.out_fp32 = c->out_fp32; a.has_out1 = c->out1 != nullptr;
  a.alpha = c->alpha; a.alpha_dev = c->alpha_dev; a.bias = c->bias; a.bias_bs = c->bias_bs; a.act = c->act;
  a.ci = static_cast<const __nv_bfloat16*>(c->ci); a.ld_ci = c->ld_ci;
  a.H = static_cast<const __nv_bfloat16*>(c->H); a.ld_h = c->ld_h;
  a.delta = c->delta; a.rowscale = c->rowscale;
  a.dci = c->dci; a.ld_dci = c->ld_dci; a.dci_accumulate = c->dci_accumulate; a.dci_bf16 = c->dci_bf16;
  a.seed = c->seed; a.seed_dev = c->seed_dev; a.stream = c->rng_stream; a.row_offset = c->rng_row_offset; a.mask_mode = c->mask_mode;
  a.status = c->status;
  a.bgroup_of_mblock = c->bgroup_of_mblock; a.kblock_range = c->kblock_range;
  a.a_bcast = c->a_bcast; a.b_bcast = c->b_bcast;
  a.rs_world = c->rs_world; a.rs_rows = c->rs_rows;
  a.ag_world = c->ag_world; a.ag_rank = c->ag_rank; a.ag_rows = c->ag_rows;
  a.ag_dst = const_cast<void*>(c->A0); a.ag_ld = c->lda0; a.ag_k = c->K0; a.ag_flags = c->ag_flags; a.ag_seq = c->ag_seq;
  for (int r = 0; r < kMaxPeers; ++r) a.ag_src[r] = c->ag_src[r];
  a.ag_gather_ctas = c->ag_gather_ctas;
  a.ag_mode = c->ag_mode;
  a.rowmap = static_cast<const int4*>(c->rowmap);
  a.philox_col0 = c->philox_col0;
  a.stage_limit = g_stage_limit;
  a.probe = g_probe;
  a.timeline = g_timeline;
  if (c->philox_col0 % 8 != 0) return kBadArgument;
  if (c->ag_world > 1 && c->ag_mode == 1) {
    a.ag_dst = const_cast<void*>(c->B0); a.ag_ld = c->ldb0; a.ag_k = c->N;
  }
  if (c->rs_world > 1) {
    if (c->rs_world > kMaxPeers || !c->out_fp32 || c->epi != EPI_PLAIN || c->batch != 1 || (c->rs_rows % BM) != 0 ||
        c->rs_rows * c->rs_world < c->M)
      return kBadArgument;
  }
  if (c->ag_world > 1 && c->ag_mode == 0) {
    if (c->ag_world > kMaxPeers || c->a_mn0 || c->batch != 1 || (c->ag_rows % BM) != 0 || (c->K0 % 8) != 0 ||
        c->ag_rows * c->ag_world != c->M || c->ag_flags == nullptr || a.split_k != 1 || c->lda0 != c->K0)
      return kBadArgument;
  } else if (c->ag_world > 1) {
    if (c->ag_world > kMaxPeers || c->ag_mode != 1 || !c->b_mn0 || c->batch != 1 || c->K1 != 0 ||
        (c->ag_rows % BK) != 0 || (c->N % 8) != 0 || c->ag_rows * c->ag_world != c->K0 || c->ag_flags == nullptr ||
        a.split_k != 1 || c->ldb0 != c->N || c->bgroup_of_mblock != nullptr || c->kblock_range != nullptr)
      return kBadArgument;
  }
  if (c->epi == EPI_FAITH) {
    if (c->ci == nullptr || (c->ld_ci % 8) != 0 || (reinterpret_cast<uintptr_t>(c->ci) & 15) || c->N % 8 != 0)
      return kBadArgument;
  } else if (c->epi != EPI_PLAIN) {
    if (c->ci == nullptr || (c->ld_ci % 8) != 0 || (reinterpret_cast<uintptr_t>(c->ci) & 15))
      return kBadArgument;
    if (c->epi == EPI_MASK_BWD && c->dci != nullptr) {
      if (c->H == nullptr || (c->ld_h % 8) != 0 || (c->ld_dci % (c->dci_bf16 ? 8 : 4)) != 0 ||
          (reinterpret_cast<uintptr_t>(c->H) & 15) || (reinterpret_cast<uintptr_t>(c->dci) & 15))
        return kBadArgument;
    }
    if (c->N % 8 != 0) return kBadArgument;
  }

  CUtensorMap ta0, tb0, ta1, tb1, to0, to1;
  PeerMaps peers;
  int rc;
  OperandDesc A0{c->A0, c->lda0, c->bsa0, c->a_mn0}, B0{c->B0, c->ldb0, c->bsb0, c->b_mn0};
  const int a_batch = c->a_bcast ? 1 : c->batch;
  const int b_batch = c->b_bcast ? 1 : (c->bgroup_of_mblock ? c->b_groups : c->batch);
  // CTA pairs (one MMA over two CTAs, each staging half of B): dense, ungrouped products whose row
  // count fills at least one 256-row tile; `cta_group` = 1 / 2 forces the choice, 0 = automatic.
  // A grouped product may pair only on request (`cta_group` = 2): the caller then guarantees that row groups
  // start on 256-row boundaries, so both CTAs of a pair read the same group's B.
  const bool grouped_pair = c->bgroup_of_mblock == nullptr || (c->cta_group == 2 && c->M % (2 * BM) == 0);
  const bool pair_ok = bn == 256 && grouped_pair && c->ag_world <= 1 && c->rs_world <= 1 &&
                       c->M >= 2 * BM && (c->max_ctas == 0 || c->max_ctas >= 2);
  // Pairs halve each CTA's share of the B tile (less shared-memory fill per MMA) and win on every flagship
  // shape measured, K-major or MN-major operands alike.
  const bool pair = pair_ok && c->cta_group != 1 && (c->cta_group == 2 || g_pair_default);
  const int b_box = pair ? bn / 2 : bn;
  if ((rc = encode_operand(&ta0, A0, c->M, c->K0, a_batch, BM))) return 1000 + rc;
  if ((rc = encode_operand(&tb0, B0, c->N, c->K0, b_batch, b_box))) return 2000 + rc;
  if (c->K1 > 0) {
    OperandDesc A1{c->A1, c->lda1, c->bsa1, c->a_mn1}, B1{c->B1, c->ldb1, c->bsb1, c->b_mn1};
    if ((rc = encode_operand(&ta1, A1, c->M, c->K1, a_batch, BM))) return 3000 + rc;
    if ((rc = encode_operand(&tb1, B1, c->N, c->K1, b_batch, b_box))) return 4000 + rc;
  } else {
    ta1 = ta0;
    tb1 = tb0;
  }
  const int oes = c->out_fp32 ? 4 : 2;
  if ((rc = encode_tmap(&to0, c->out0, oes, true, c->N, c->M, c->ldo0, c->batch, c->bso0,
                        c->out_fp32 ? 32 : 64, 32)))
    return 5000 + rc;
  if (nout == 2) {
    if ((rc = encode_tmap(&to1, c->out1, 2, false, c->N, c->M, c->ldo1, 1, 0, 64, 32)))
      return 6000 + rc;
  } else {
    to1 = to0;
  }

  // TMA-fed mask epilogue: dense (no row map), bf16 mask gradient written (not accumulated), real row pitches.
  // With a long K loop the main loop is the longer half of a tile and wants the pipeline stages the operand
  // ring would take, so the automatic choice keeps it to short K.
  CUtensorMap tci = to0, th = to0, tdci = to0;
  bool epi_tma = false;
  if ((c->epi == EPI_MASK_FWD || c->epi == EPI_MASK_BWD) && c->epi_tma != 1 && bn == 256 && c->rowmap == nullptr &&
      c->bgroup_of_mblock == nullptr && c->ag_world <= 1 && c->rs_world <= 1 && c->ld_ci >= c->N &&
      (c->epi_tma == 2 || c->K0 + c->K1 <= 1536)) {
    const bool want_h = c->epi == EPI_MASK_BWD && c->dci != nullptr;
    epi_tma = !(want_h && (!c->dci_bf16 || c->dci_accumulate || c->ld_h < c->N || c->ld_dci < c->N));
    if (epi_tma) {
      if ((rc = encode_tmap(&tci, c->ci, 2, false, c->N, c->M, c->ld_ci, 1, 0, 64, 32))) return 8000 + rc;
      if (want_h) {
        if ((rc = encode_tmap(&th, c->H, 2, false, c->N, c->M, c->ld_h, 1, 0, 64, 32))) return 8100 + rc;
        if ((rc = encode_tmap(&tdci, c->dci, 2, false, c->N, c->M, c->ld_dci, 1, 0, 64, 32))) return 8200 + rc;
      }
      if (c->epi == EPI_MASK_FWD && nout != 2) to1 = to0;
    }
  }
  for (int r = 0; r < kMaxPeers; ++r) peers.m[r] = to0;
  if (c->rs_world > 1) {
    for (int r = 0; r < c->rs_world; ++r)
      if ((rc = encode_tmap(&peers.m[r], c->rs_out[r], 4, true, c->N, c->rs_rows, c->ldo0, 1, 0, 32, 32)))
        return 7000 + rc;
  }
#define PD_LAUNCH(BN_, EPI_, NOUT_) \
  launch_gemm<BN_, EPI_, NOUT_, 1>(ta0, tb0, ta1, tb1, to0, to1, tci, th, tdci, peers, a, c->max_ctas, stream)
#define PD_LAUNCH2(EPI_, NOUT_) \
  launch_gemm<256, EPI_, NOUT_, 2>(ta0, tb0, ta1, tb1, to0, to1, tci, th, tdci, peers, a, c->max_ctas, stream)
  if (epi_tma) {
    if (c->epi == EPI_MASK_FWD) return pair ? PD_LAUNCH2(EPI_MASK_FWD, 4) : PD_LAUNCH(256, EPI_MASK_FWD, 4);
    return pair ? PD_LAUNCH2(EPI_MASK_BWD, 4) : PD_LAUNCH(256, EPI_MASK_BWD, 4);
  }
  if (pair) {
    if (c->epi == EPI_PLAIN) return PD_LAUNCH2(EPI_PLAIN, 1);
    if (c->epi == EPI_MASK_FWD) return nout == 2 ? PD_LAUNCH2(EPI_MASK_FWD, 2) : PD_LAUNCH2(EPI_MASK_FWD, 1);
    if (c->epi == EPI_MASK_BWD) return PD_LAUNCH2(EPI_MASK_BWD, 1);
    if (c->epi == EPI_FAITH) return PD_LAUNCH2(EPI_FAITH, 1);
  }
  if (c->epi == EPI_PLAIN) return bn == 256 ? PD_LAUNCH(256, EPI_PLAIN, 1) : PD_LAUNCH(128, EPI_PLAIN, 1);
  if (c->epi == EPI_MASK_FWD) {
    if (nout == 2) return bn == 256 ? PD_LAUNCH(256, EPI_MASK_FWD, 2) : PD_LAUNCH(128, EPI_MASK_FWD, 2);
    return bn == 256 ? PD_LAUNCH(256, EPI_MASK_FWD, 1) : PD_LAUNCH(128, EPI_MASK_FWD, 1);
  }
  if (c->epi == EPI_MASK_BWD) return bn == 256 ? PD_LAUNCH(256, EPI_MASK_BWD, 1) : PD_LAUNCH(128, EPI_MASK_BWD, 1);
  if (c->epi == EPI_FAITH) return bn == 256 ? PD_LAUNCH(256, EPI_FAITH, 1) : PD_LAUNCH(128, EPI_FAITH, 1);
#undef PD_LAUNCH2
#undef PD_LAUNCH
  return kBadArgument;
}

extern "C" void pd_gemm_set_timeline(void* dev_ptr) { g_timeline = static_cast<long long*>(dev_ptr); }

extern "C" void pd_gemm_set_probe(int bits) { g_probe = bits; }

extern "C" void pd_gemm_set_stage_limit(int n) { g_stage_limit = n; }

extern "C" void pd_gemm_set_pair_default(int on) { g_pair_default = on != 0; }

extern "C" int pd_gemm_call_size() { return static_cast<int>(sizeof(PdGemmCall)); }
