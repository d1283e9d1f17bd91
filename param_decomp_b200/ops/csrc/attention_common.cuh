// Helpers shared by the attention kernels (flash attention, attention-pattern KL): tile constants,
// swizzled shared-memory addressing, packing, and the [B, T, heads * hd] tensor-map encoder.
#pragma once

#include "common.cuh"

namespace pd_attn {

using namespace pd;

constexpr int kTile = 128;        // query rows and key rows per tile
constexpr int kSoftmaxThreads = 128;
constexpr int kFwdThreads = 192;  // 4 softmax warps + producer + MMA
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of 16-byte chunk `chunk16` (0..7) of row `row` inside a [rows x 64 bf16] block laid out
// the way TMA's 128-byte swizzle (and the tcgen05 descriptors) expect.
__device__ __forceinline__ uint32_t swz(int row, int chunk16) {
  return static_cast<uint32_t>(row) * 128u + static_cast<uint32_t>((chunk16 ^ (row & 7)) << 4);
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void named_barrier_softmax() {
  asm volatile("bar.sync 1, 128;" ::: "memory");
}


inline int encode_bthd(CUtensorMap* tm, const void* p, int B, int T, int heads, int hd) {
  // [B, T, heads * hd] bf16 viewed as (inner = heads*hd, rows = T, batch = B); box = 64 columns x 128 rows
  return encode_tmap(tm, p, 2, false, static_cast<uint64_t>(heads) * hd, T, static_cast<uint64_t>(heads) * hd, B,
                     static_cast<uint64_t>(T) * heads * hd, 64, kTile);
}

inline bool bad_shape(int B, int T, int H, int Hkv, int hd) {
  return B < 1 || T < kTile || (T % kTile) != 0 || H < 1 || Hkv < 1 || (H % Hkv) != 0 || (hd != 64 && hd != 128) ||
         B > 65535 || H > 65535;
}

}  // namespace pd_attn
