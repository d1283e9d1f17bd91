// Bandwidth-bound kernels of the step: fused AdamW with device-side global-norm clipping,
// fp32 -> bf16 casts, RMSNorm forward/backward, rotary embedding, SwiGLU forward/backward,
// per-row scaling, leaky-hard sigmoids. All are plain grid-stride / row-per-warp kernels with
// 16-byte vector accesses; none of them waits on anything, so none needs a status word.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

inline int blocks_for(long long n, int per_block, int cap = 148 * 16) {
  long long b = (n + per_block - 1) / per_block;
  if (b < 1) b = 1;
  return static_cast<int>(b < cap ? b : cap);
}

// ---- optimizer ------------------------------------------------------------------------------
__global__ void sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  float acc = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += stride) {
    if (i + 3 < n) {
      const float4 v = *reinterpret_cast<const float4*>(g + i);
      acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    } else {
      for (long long j = i; j < n; ++j) acc += g[j] * g[j];
    }
  }
  acc = warp_sum(acc);
  __shared__ float part[kThreads / 32];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kThreads / 32 ? part[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) atomicAdd(out, v);
  }
}

// scale = min(max_norm / (sqrt(sumsq) + 1e-6), 1); max_norm <= 0 means no clipping.
__global__ void clip_scale_kernel(const float* __restrict__ sumsq, float max_norm,
                                  float* __restrict__ scale, float* __restrict__ norm_out) {
  const float norm = sqrtf(*sumsq);
  *norm_out = norm;
  *scale = max_norm > 0.f ? fminf(max_norm / (norm + 1e-6f), 1.f) : 1.f;
}

__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v, long long n, float lr,
                             float b1, float b2, float eps, float wd, float inv_bc1, float inv_bc2,
                             const float* __restrict__ grad_scale) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < n;
       i += stride) {
    if (i + 3 < n) {
      float4 pp = *reinterpret_cast<float4*>(p + i);
      const float4 gg = *reinterpret_cast<const float4*>(g + i);
      float4 mm = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      float* pa = &pp.x; const float* ga = &gg.x; float* ma = &mm.x; float* va = &vv.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gk = ga[k] * gs;
        ma[k] = b1 * ma[k] + (1.f - b1) * gk;
        va[k] = b2 * va[k] + (1.f - b2) * gk * gk;
        const float upd = (ma[k] * inv_bc1) / (sqrtf(va[k] * inv_bc2) + eps) + wd * pa[k];
        pa[k] -= lr * upd;
      }
      *reinterpret_cast<float4*>(p + i) = pp;
      *reinterpret_cast<float4*>(m + i) = mm;
      *reinterpret_cast<float4*>(v + i) = vv;
    } else {
      for (long long j = i; j < n; ++j) {
        const float gk = g[j] * gs;
        m[j] = b1 * m[j] + (1.f - b1) * gk;
        v[j] = b2 * v[j] + (1.f - b2) * gk * gk;
        p[j] -= lr * ((m[j] * inv_bc1) / (sqrtf(v[j] * inv_bc2) + eps) + wd * p[j]);
      }
    }
  }
}

__global__ void cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                 long long n) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < n;
       i += stride) {
    if (i + 7 < n) {
      const float4 a = *reinterpret_cast<const float4*>(src + i);
      const float4 b = *reinterpret_cast<const float4*>(src + i + 4);
      __nv_bfloat162 o[4] = {__floats2bfloat162_rn(a.x, a.y), __floats2bfloat162_rn(a.z, a.w),
                             __floats2bfloat162_rn(b.x, b.y), __floats2bfloat162_rn(b.z, b.w)};
      *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<uint4*>(o);
    } else {
      for (long long j = i; j < n; ++j) dst[j] = __float2bfloat16(src[j]);
    }
  }
}

// ---- RMSNorm: one warp per row, bf16 in/out, fp32 statistics -----------------------------------
// forward also stores rstd[row] for the backward.
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                   long long rows, int d, float eps) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (long long row = static_cast<long long>(blockIdx.x) * warps + (threadIdx.x >> 5); row < rows;
       row += static_cast<long long>(gridDim.x) * warps) {
    const __nv_bfloat16* xr = x + row * d;
    float ss = 0.f;
    for (int i = lane * 8; i < d; i += 256) {
      const uint4 q = *reinterpret_cast<const uint4*>(xr + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / d + eps);
    if (lane == 0 && rstd) rstd[row] = r;
    __nv_bfloat16* yr = y + row * d;
    for (int i = lane * 8; i < d; i += 256) {
      const uint4 q = *reinterpret_cast<const uint4*>(xr + i);
      const uint4 wq = w ? *reinterpret_cast<const uint4*>(w + i) : make_uint4(0, 0, 0, 0);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
      const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wq);
      __nv_bfloat162 o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float2 f = __bfloat1622float2(h[k]);
        const float2 g = w ? __bfloat1622float2(wh[k]) : make_float2(1.f, 1.f);
        o[k] = __floats2bfloat162_rn(f.x * r * g.x, f.y * r * g.y);
      }
      *reinterpret_cast<uint4*>(yr + i) = *reinterpret_cast<uint4*>(o);
    }
  }
}

// dx = rstd * (g*w - xhat * mean(g*w*xhat)), xhat = x*rstd. The weight is frozen: no dw.
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w,
                                   const __nv_bfloat16* __restrict__ dy,
                                   const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
                                   long long rows, int d) {
  const int warps = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (long long row = static_cast<long long>(blockIdx.x) * warps + (threadIdx.x >> 5); row < rows;
       row += static_cast<long long>(gridDim.x) * warps) {
    const __nv_bfloat16* xr = x + row * d;
    const __nv_bfloat16* gr = dy + row * d;
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = lane * 8; i < d; i += 256) {
      const uint4 q = *reinterpret_cast<const uint4*>(xr + i);
      const uint4 gq = *reinterpret_cast<const uint4*>(gr + i);
      const uint4 wq = w ? *reinterpret_cast<const uint4*>(w + i) : make_uint4(0, 0, 0, 0);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gq);
      const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wq);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]), g = __bfloat1622float2(gh[k]);
        const float2 ww = w ? __bfloat1622float2(wh[k]) : make_float2(1.f, 1.f);
        dot += g.x * ww.x * f.x * r + g.y * ww.y * f.y * r;
      }
    }
    dot = warp_sum(dot) / d;
    __nv_bfloat16* dr = dx + row * d;
    for (int i = lane * 8; i < d; i += 256) {
      const uint4 q = *reinterpret_cast<const uint4*>(xr + i);
      const uint4 gq = *reinterpret_cast<const uint4*>(gr + i);
      const uint4 wq = w ? *reinterpret_cast<const uint4*>(w + i) : make_uint4(0, 0, 0, 0);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gq);
      const __nv_bfloat162* wh = reinterpret_cast<const __nv_bfloat162*>(&wq);
      __nv_bfloat162 o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]), g = __bfloat1622float2(gh[k]);
        const float2 ww = w ? __bfloat1622float2(wh[k]) : make_float2(1.f, 1.f);
        o[k] = __floats2bfloat162_rn(r * (g.x * ww.x - f.x * r * dot), r * (g.y * ww.y - f.y * r * dot));
      }
      *reinterpret_cast<uint4*>(dr + i) = *reinterpret_cast<uint4*>(o);
    }
  }
}

// ---- rotary embedding (rotate-half form), in place on [rows = B*T, heads, hd] -------------------
// cos/sin [T, hd/2] fp32; `inverse` applies the transpose rotation (the backward).
// `src` may equal `dst` (in place): every thread reads its pair before it writes it.
__global__ void rope_kernel(const __nv_bfloat16* src, __nv_bfloat16* dst, const float* __restrict__ cs,
                            const float* __restrict__ sn, long long rows, int T, int heads, int hd,
                            int inverse) {
  const int half = hd >> 1;
  const long long total = rows * heads * half;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(i % half);
    const long long rh = i / half;
    const long long row = rh / heads;
    const int t = static_cast<int>(row % T);
    const float c = cs[t * half + j];
    const float s = inverse ? -sn[t * half + j] : sn[t * half + j];
    const __nv_bfloat16* q = src + rh * hd;
    __nv_bfloat16* p = dst + rh * hd;
    const float a = __bfloat162float(q[j]), b = __bfloat162float(q[j + half]);
    p[j] = __float2bfloat16(a * c - b * s);
    p[j + half] = __float2bfloat16(b * c + a * s);
  }
}

// eight rotation pairs per thread (16-byte loads of the low and the high half); needs hd % 16 == 0
__global__ void rope_vec_kernel(const __nv_bfloat16* src, __nv_bfloat16* dst, const float* __restrict__ cs,
                                const float* __restrict__ sn, long long rows, int T, int heads, int hd,
                                int inverse) {
  const int half = hd >> 1, groups = half >> 3;
  const long long total = rows * heads * groups;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int g = static_cast<int>(i % groups);
    const long long rh = i / groups;
    const int t = static_cast<int>((rh / heads) % T);
    const __nv_bfloat16* q = src + rh * hd + 8 * g;
    __nv_bfloat16* p = dst + rh * hd + 8 * g;
    const uint4 lo = *reinterpret_cast<const uint4*>(q), hi = *reinterpret_cast<const uint4*>(q + half);
    const __nv_bfloat162* l2 = reinterpret_cast<const __nv_bfloat162*>(&lo);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&hi);
    const float4* c4 = reinterpret_cast<const float4*>(cs + static_cast<long long>(t) * half + 8 * g);
    const float4* s4 = reinterpret_cast<const float4*>(sn + static_cast<long long>(t) * half + 8 * g);
    const float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
    const float c[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
    const float sv[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
    __nv_bfloat162 ol[4], oh[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = __bfloat1622float2(l2[k]), b = __bfloat1622float2(h2[k]);
      const float s0 = inverse ? -sv[2 * k] : sv[2 * k], s1 = inverse ? -sv[2 * k + 1] : sv[2 * k + 1];
      ol[k] = __floats2bfloat162_rn(a.x * c[2 * k] - b.x * s0, a.y * c[2 * k + 1] - b.y * s1);
      oh[k] = __floats2bfloat162_rn(b.x * c[2 * k] + a.x * s0, b.y * c[2 * k + 1] + a.y * s1);
    }
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<uint4*>(ol);
    *reinterpret_cast<uint4*>(p + half) = *reinterpret_cast<uint4*>(oh);
  }
}

// ---- SwiGLU ---------------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gate,
                                  const __nv_bfloat16* __restrict__ up,
                                  __nv_bfloat16* __restrict__ out, long long n) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < n;
       i += stride) {
    const uint4 gq = *reinterpret_cast<const uint4*>(gate + i);
    const uint4 uq = *reinterpret_cast<const uint4*>(up + i);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gq);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uq);
    __nv_bfloat162 o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(gh[k]), u = __bfloat1622float2(uh[k]);
      o[k] = __floats2bfloat162_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
    }
    *reinterpret_cast<uint4*>(out + i) = *reinterpret_cast<uint4*>(o);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gate,
                                  const __nv_bfloat16* __restrict__ up,
                                  const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgate, __nv_bfloat16* __restrict__ dup,
                                  long long n) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < n;
       i += stride) {
    const uint4 gq = *reinterpret_cast<const uint4*>(gate + i);
    const uint4 uq = *reinterpret_cast<const uint4*>(up + i);
    const uint4 dq = *reinterpret_cast<const uint4*>(dout + i);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gq);
    const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uq);
    const __nv_bfloat162* dh = reinterpret_cast<const __nv_bfloat162*>(&dq);
    __nv_bfloat162 og[4], ou[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 g = __bfloat1622float2(gh[k]), u = __bfloat1622float2(uh[k]),
                   d = __bfloat1622float2(dh[k]);
      const float sx = 1.f / (1.f + __expf(-g.x)), sy = 1.f / (1.f + __expf(-g.y));
      ou[k] = __floats2bfloat162_rn(d.x * g.x * sx, d.y * g.y * sy);
      og[k] = __floats2bfloat162_rn(d.x * u.x * sx * (1.f + g.x * (1.f - sx)),
                                    d.y * u.y * sy * (1.f + g.y * (1.f - sy)));
    }
    *reinterpret_cast<uint4*>(dgate + i) = *reinterpret_cast<uint4*>(og);
    *reinterpret_cast<uint4*>(dup + i) = *reinterpret_cast<uint4*>(ou);
  }
}

// y[row, :] = x[row, :] * s[row]
__global__ void rowscale_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ s,
                                __nv_bfloat16* __restrict__ y, long long rows, int d) {
  const long long total = rows * (d / 8);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / (d / 8);
    const float sc = s[row];
    const uint4 q = *reinterpret_cast<const uint4*>(x + i * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
    __nv_bfloat162 o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      o[k] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
    }
    *reinterpret_cast<uint4*>(y + i * 8) = *reinterpret_cast<uint4*>(o);
  }
}

// ---- routed rows: tokens <-> padded sorted job rows -----------------------------------------------
// `rowmap[r] = (token, slot, -, -)` of padded row r (token -1 on padding rows); `pos[token * k + slot]`
// is the inverse. Both directions move whole rows in 16-byte pieces; no row is written twice, so
// neither direction needs atomics or a cleared destination.
//
// out[r, :] = w[src] * x[src, :],  src = token * rep + slot * use_slot;  zero rows on padding.
__global__ void rows_expand_kernel(const __nv_bfloat16* __restrict__ x, const int4* __restrict__ rowmap,
                                   const float* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                   long long n_rows, int d, int k_sel, int rep, int use_slot) {
  const int segs = d / 8;
  const long long total = n_rows * segs;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / segs;
    const int seg = static_cast<int>(i - r * segs);
    const int4 rm = __ldg(rowmap + r);
    uint4 q = make_uint4(0, 0, 0, 0);
    if (rm.x >= 0) {
      const long long src = static_cast<long long>(rm.x) * rep + (use_slot ? rm.y : 0);
      q = *reinterpret_cast<const uint4*>(x + src * d + seg * 8);
      if (w != nullptr) {
        const float sc = w[static_cast<long long>(rm.x) * k_sel + rm.y];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          h[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
      }
    }
    *reinterpret_cast<uint4*>(out + i * 8) = q;
  }
}

// y[n, :] = sum_s w[n, s] * padded[pos[n * k + s], :]   (fp32 accumulation)
// With `bgroup` (owner of every 128-row block, -1 = rows no product wrote) jobs in unowned blocks are left out.
__global__ void rows_combine_kernel(const __nv_bfloat16* __restrict__ padded, const long long* __restrict__ pos,
                                    const float* __restrict__ w, const int* __restrict__ bgroup,
                                    __nv_bfloat16* __restrict__ y, long long tokens, int d, int k_sel) {
  const int segs = d / 8;
  const long long total = tokens * segs;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long n = i / segs;
    const int seg = static_cast<int>(i - n * segs);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int s = 0; s < k_sel; ++s) {
      const long long r = __ldg(pos + n * k_sel + s);
      if (bgroup != nullptr && __ldg(bgroup + (r >> 7)) < 0) continue;
      const float sc = w != nullptr ? __ldg(w + n * k_sel + s) : 1.0f;
      const uint4 q = *reinterpret_cast<const uint4*>(padded + r * d + seg * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] = fmaf(f.x, sc, acc[2 * j]);
        acc[2 * j + 1] = fmaf(f.y, sc, acc[2 * j + 1]);
      }
    }
    __nv_bfloat162 o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(y + i * 8) = *reinterpret_cast<uint4*>(o);
  }
}

// lower (bf16, masks) and upper (fp32-accurate bf16, minimality) leaky-hard sigmoids of fp32/bf16
// pre-activations in one pass.
__global__ void ci_squash_kernel(const __nv_bfloat16* __restrict__ pre,
                                 __nv_bfloat16* __restrict__ lower,
                                 __nv_bfloat16* __restrict__ upper, long long n, float alpha) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 8;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < n;
       i += stride) {
    const uint4 q = *reinterpret_cast<const uint4*>(pre + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
    __nv_bfloat162 lo[4], hi[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]);
      const float lx = fminf(fmaxf(f.x, 0.f), 1.f), ly = fminf(fmaxf(f.y, 0.f), 1.f);
      lo[k] = __floats2bfloat162_rn(lx, ly);
      hi[k] = __floats2bfloat162_rn(f.x > 1.f ? 1.f + alpha * (f.x - 1.f) : lx,
                                    f.y > 1.f ? 1.f + alpha * (f.y - 1.f) : ly);
    }
    *reinterpret_cast<uint4*>(lower + i) = *reinterpret_cast<uint4*>(lo);
    *reinterpret_cast<uint4*>(upper + i) = *reinterpret_cast<uint4*>(hi);
  }
}


// ---- fused CI squash + smooth-L0 activity ------------------------------------------------------
// One pass over the pre-activations [rows, C] (bf16):
//   lower = clamp(pre, 0, 1)                                   (bf16, feeds the masks)
//   colsum[c] += sum_rows psi(upper(pre)),  psi(u) = u^2 / (u^2 + gamma^2) (* (1 + gamma^2))
// Block = 32 column groups of 8 columns x 8 row lanes; grid = (C / 256, row chunks).
__global__ void ci_squash_activity_kernel(const __nv_bfloat16* __restrict__ pre,
                                          __nv_bfloat16* __restrict__ lower,
                                          float* __restrict__ colsum, long long rows, int C,
                                          float gamma2, float norm, float alpha, const float* __restrict__ gamma_dev, int normalize) {
  if (gamma_dev != nullptr) {  // the schedule's current value lives in device memory (recorded launches)
    const float gm = *gamma_dev;
    gamma2 = gm * gm;
    norm = normalize ? 1.f + gamma2 : 1.f;
  }
  const int cg = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + cg) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < C) {
    for (long long r = static_cast<long long>(blockIdx.y) * 8 + rl; r < rows;
         r += static_cast<long long>(gridDim.y) * 8) {
      const uint4 q = *reinterpret_cast<const uint4*>(pre + r * C + col);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
      __nv_bfloat162 lo[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        const float lx = fminf(fmaxf(f.x, 0.f), 1.f), ly = fminf(fmaxf(f.y, 0.f), 1.f);
        lo[k] = __floats2bfloat162_rn(lx, ly);
        const float ux = f.x > 1.f ? 1.f + alpha * (f.x - 1.f) : lx;
        const float uy = f.y > 1.f ? 1.f + alpha * (f.y - 1.f) : ly;
        acc[2 * k] += norm * __fdividef(ux * ux, ux * ux + gamma2);
        acc[2 * k + 1] += norm * __fdividef(uy * uy, uy * uy + gamma2);
      }
      *reinterpret_cast<uint4*>(lower + r * C + col) = *reinterpret_cast<uint4*>(lo);
    }
  }
  __shared__ float red[8][32][8];
#pragma unroll
  for (int k = 0; k < 8; ++k) red[rl][cg][k] = acc[k];
  __syncthreads();
  if (rl == 0 && col < C) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float v = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) v += red[j][cg][k];
      atomicAdd(colsum + col + k, v);
    }
  }
}

// dpre = lower'(pre; dlower) + dcol[c] * psi'(upper) * upper'(pre)
//   lower': pre in (0,1] -> g;  pre <= 0 -> (g < 0 ? alpha g : 0);  pre > 1 -> 0
__global__ void ci_squash_activity_bwd_kernel(const __nv_bfloat16* __restrict__ pre,
                                              const __nv_bfloat16* __restrict__ dlower,
                                              const float* __restrict__ dcol,
                                              __nv_bfloat16* __restrict__ dpre, long long rows, int C,
                                              float gamma2, float norm, float alpha, const float* __restrict__ gamma_dev, int normalize) {
  if (gamma_dev != nullptr) {  // the schedule's current value lives in device memory (recorded launches)
    const float gm = *gamma_dev;
    gamma2 = gm * gm;
    norm = normalize ? 1.f + gamma2 : 1.f;
  }
  // Same tiling as the forward: a thread owns 8 columns (its dcol values stay in registers) and walks
  // rows with the grid's row stride, four rows in flight per iteration.
  const int cg = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + cg) * 8;
  if (col >= C) return;
  const float4 d0 = *reinterpret_cast<const float4*>(dcol + col);
  const float4 d1 = *reinterpret_cast<const float4*>(dcol + col + 4);
  const float dc[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
  const float k2 = norm * 2.f * gamma2;
  const long long stride = static_cast<long long>(gridDim.y) * 8;
  // Branch-free per element (the three regimes of the leaky clamp are selects, not divergent paths).
  auto one = [&](long long r, const uint4 q, const uint4 gq) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gq);
    __nv_bfloat162 o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]), g = __bfloat1622float2(gh[k]);
      float out[2];
      const float x[2] = {f.x, f.y}, gg[2] = {g.x, g.y};
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float xv = x[e];
        const bool above = xv > 1.f, inside = xv > 0.f;
        const float u = above ? fmaf(alpha, xv - 1.f, 1.f) : fmaxf(xv, 0.f);
        const float du = above ? alpha : (inside ? 1.f : 0.f);
        const float lg = above ? 0.f : (inside ? gg[e] : alpha * fminf(gg[e], 0.f));
        const float den = fmaf(u, u, gamma2);
        out[e] = fmaf(dc[2 * k + e] * du, __fdividef(k2 * u, den * den), lg);
      }
      o[k] = __floats2bfloat162_rn(out[0], out[1]);
    }
    *reinterpret_cast<uint4*>(dpre + r * C + col) = *reinterpret_cast<uint4*>(o);
  };
  const uint4 zero = make_uint4(0, 0, 0, 0);
  long long r = static_cast<long long>(blockIdx.y) * 8 + rl;
  // four rows in flight per thread: eight 16-byte loads issued before the first is consumed
  for (; r + 3 * stride < rows; r += 4 * stride) {
    uint4 q[4], g[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = *reinterpret_cast<const uint4*>(pre + (r + j * stride) * C + col);
#pragma unroll
    for (int j = 0; j < 4; ++j) g[j] = dlower ? *reinterpret_cast<const uint4*>(dlower + (r + j * stride) * C + col) : zero;
#pragma unroll
    for (int j = 0; j < 4; ++j) one(r + j * stride, q[j], g[j]);
  }
  for (; r < rows; r += stride) {
    const uint4 qa = *reinterpret_cast<const uint4*>(pre + r * C + col);
    const uint4 ga = dlower ? *reinterpret_cast<const uint4*>(dlower + r * C + col) : zero;
    one(r, qa, ga);
  }
}

// ---- the same pair for narrow CI of an expert-blocked site ---------------------------------------
// `pre [tokens, k * c]` holds one c-wide slot per selected expert of each token. The rows of the
// padded sorted job layout map to (token, slot) through `rowmap`, and every 128-row block belongs
// to one expert (`bgroup`), so a block sums its rows in registers and issues one atomic per column
// into `colsum [n_experts * c]`. `lower` is written back in token order.
__global__ void ci_squash_activity_jobs_kernel(const __nv_bfloat16* __restrict__ pre,
                                               __nv_bfloat16* __restrict__ lower,
                                               float* __restrict__ colsum,
                                               const int4* __restrict__ rowmap,
                                               const int* __restrict__ bgroup, int c, long long pitch,
                                               float gamma2, float norm, float alpha, const float* __restrict__ gamma_dev, int normalize) {
  if (gamma_dev != nullptr) {  // the schedule's current value lives in device memory (recorded launches)
    const float gm = *gamma_dev;
    gamma2 = gm * gm;
    norm = normalize ? 1.f + gamma2 : 1.f;
  }
  const int e = bgroup[blockIdx.y];
  if (e < 0) return;
  const int cg = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + cg) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < c) {
#pragma unroll 4
    for (int i = 0; i < 16; ++i) {
      const int4 rm = rowmap[static_cast<long long>(blockIdx.y) * 128 + rl + 8 * i];
      if (rm.x < 0) continue;
      const long long at = static_cast<long long>(rm.x) * pitch + rm.y + col;
      const uint4 q = *reinterpret_cast<const uint4*>(pre + at);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
      __nv_bfloat162 lo[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        const float lx = fminf(fmaxf(f.x, 0.f), 1.f), ly = fminf(fmaxf(f.y, 0.f), 1.f);
        lo[k] = __floats2bfloat162_rn(lx, ly);
        const float ux = f.x > 1.f ? 1.f + alpha * (f.x - 1.f) : lx;
        const float uy = f.y > 1.f ? 1.f + alpha * (f.y - 1.f) : ly;
        acc[2 * k] += norm * __fdividef(ux * ux, ux * ux + gamma2);
        acc[2 * k + 1] += norm * __fdividef(uy * uy, uy * uy + gamma2);
      }
      *reinterpret_cast<uint4*>(lower + at) = *reinterpret_cast<uint4*>(lo);
    }
  }
  __shared__ float red[8][32][8];
#pragma unroll
  for (int k = 0; k < 8; ++k) red[rl][cg][k] = acc[k];
  __syncthreads();
  if (rl == 0 && col < c) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float v = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) v += red[j][cg][k];
      atomicAdd(colsum + static_cast<long long>(e) * c + col + k, v);
    }
  }
}

// Backward in token order: the expert of a slot comes from `experts [tokens, k]`.
__global__ void ci_squash_activity_jobs_bwd_kernel(const __nv_bfloat16* __restrict__ pre,
                                                   const __nv_bfloat16* __restrict__ dlower,
                                                   const float* __restrict__ dcol,
                                                   const long long* __restrict__ experts,
                                                   __nv_bfloat16* __restrict__ dpre, long long tokens,
                                                   int k_sel, int c, float gamma2, float norm,
                                                   float alpha, const float* __restrict__ gamma_dev, int normalize) {
  if (gamma_dev != nullptr) {  // the schedule's current value lives in device memory (recorded launches)
    const float gm = *gamma_dev;
    gamma2 = gm * gm;
    norm = normalize ? 1.f + gamma2 : 1.f;
  }
  const int groups = c / 8;
  const long long total = tokens * k_sel * groups;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long job = i / groups;
    const int col = static_cast<int>(i - job * groups) * 8;
    const long long e = experts[job];
    const uint4 q = *reinterpret_cast<const uint4*>(pre + i * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
    uint4 gq = make_uint4(0, 0, 0, 0);
    if (dlower) gq = *reinterpret_cast<const uint4*>(dlower + i * 8);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gq);
    const float4 d0 = *reinterpret_cast<const float4*>(dcol + e * c + col);
    const float4 d1 = *reinterpret_cast<const float4*>(dcol + e * c + col + 4);
    const float dc[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
    __nv_bfloat162 o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(h[k]), g = __bfloat1622float2(gh[k]);
      float out[2];
      const float x[2] = {f.x, f.y}, gg[2] = {g.x, g.y};
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const float xv = x[t];
        float lg = 0.f, u, du;
        if (xv > 1.f) { u = 1.f + alpha * (xv - 1.f); du = alpha; }
        else if (xv > 0.f) { u = xv; du = 1.f; lg = gg[t]; }
        else { u = 0.f; du = 0.f; lg = gg[t] < 0.f ? alpha * gg[t] : 0.f; }
        const float den = u * u + gamma2;
        const float dpsi = __fdividef(norm * 2.f * u * gamma2, den * den);
        out[t] = lg + dc[2 * k + t] * dpsi * du;
      }
      o[k] = __floats2bfloat162_rn(out[0], out[1]);
    }
    *reinterpret_cast<uint4*>(dpre + i * 8) = *reinterpret_cast<uint4*>(o);
  }
}

// ---- vocabulary KL: one block per position ------------------------------------------------------
// kl[row] = KL(softmax(lc[row]) || softmax(lm[row]));  dlm[row] = softmax(lm) - softmax(lc)
// (the caller scales by the upstream gradient / number of positions inside the next GEMM).
// Rows are `ld` elements apart (padded to a multiple of 8); V valid columns.
__global__ void vocab_kl_kernel(const __nv_bfloat16* __restrict__ lc, const __nv_bfloat16* __restrict__ lm,
                                __nv_bfloat16* __restrict__ dlm, float* __restrict__ kl, int V, long long ld) {
  const long long row = blockIdx.x;
  const __nv_bfloat16* a = lc + row * ld;
  const __nv_bfloat16* b = lm + row * ld;
  __shared__ float red[4][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  // pass 1: row maxima
  float ma = -INFINITY, mb = -INFINITY;
  for (int i = threadIdx.x * 8; i < V; i += blockDim.x * 8) {
    const uint4 qa = *reinterpret_cast<const uint4*>(a + i), qb = *reinterpret_cast<const uint4*>(b + i);
    const __nv_bfloat16* ha = reinterpret_cast<const __nv_bfloat16*>(&qa);
    const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(&qb);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (i + k < V) { ma = fmaxf(ma, __bfloat162float(ha[k])); mb = fmaxf(mb, __bfloat162float(hb[k])); }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ma = fmaxf(ma, __shfl_xor_sync(0xffffffffu, ma, o));
    mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, o));
  }
  if (lane == 0) { red[0][warp] = ma; red[1][warp] = mb; }
  __syncthreads();
  ma = red[0][0]; mb = red[1][0];
  for (int w = 1; w < nw; ++w) { ma = fmaxf(ma, red[0][w]); mb = fmaxf(mb, red[1][w]); }
  __syncthreads();
  // pass 2: partition functions and the cross term sum exp(a - ma) * (a - b)
  float sa = 0.f, sb = 0.f, cross = 0.f;
  for (int i = threadIdx.x * 8; i < V; i += blockDim.x * 8) {
    const uint4 qa = *reinterpret_cast<const uint4*>(a + i), qb = *reinterpret_cast<const uint4*>(b + i);
    const __nv_bfloat16* ha = reinterpret_cast<const __nv_bfloat16*>(&qa);
    const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(&qb);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (i + k < V) {
        const float x = __bfloat162float(ha[k]), y = __bfloat162float(hb[k]);
        const float ea = __expf(x - ma);
        sa += ea; sb += __expf(y - mb); cross += ea * (x - y);
      }
    }
  }
  sa = warp_sum(sa); sb = warp_sum(sb); cross = warp_sum(cross);
  if (lane == 0) { red[0][warp] = sa; red[1][warp] = sb; red[2][warp] = cross; }
  __syncthreads();
  sa = 0.f; sb = 0.f; cross = 0.f;
  for (int w = 0; w < nw; ++w) { sa += red[0][w]; sb += red[1][w]; cross += red[2][w]; }
  const float lsa = ma + __logf(sa), lsb = mb + __logf(sb);
  // KL = sum p_a (a - lsa - b + lsb) = cross / sa - lsa + lsb
  if (threadIdx.x == 0) kl[row] = cross / sa - lsa + lsb;
  // pass 3: gradient wrt the masked logits
  if (dlm != nullptr) {
    __nv_bfloat16* d = dlm + row * ld;
    const float ia = 1.f / sa, ib = 1.f / sb;
    for (int i = threadIdx.x * 8; i < V; i += blockDim.x * 8) {
      const uint4 qa = *reinterpret_cast<const uint4*>(a + i), qb = *reinterpret_cast<const uint4*>(b + i);
      const __nv_bfloat16* ha = reinterpret_cast<const __nv_bfloat16*>(&qa);
      const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(&qb);
      __nv_bfloat16 o[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float x = __bfloat162float(ha[k]), y = __bfloat162float(hb[k]);
        o[k] = __float2bfloat16(i + k < V ? __expf(y - mb) * ib - __expf(x - ma) * ia : 0.f);
      }
      *reinterpret_cast<uint4*>(d + i) = *reinterpret_cast<uint4*>(o);
    }
  }
}


// out[row, 8g .. 8g+7] = the Philox uniforms the GEMM epilogues draw for (seed, stream, row, g).
__global__ void philox_uniform_kernel(float* __restrict__ out, long long rows, int groups, int cols,
                                      unsigned long long seed, unsigned int stream, unsigned int row_offset,
                                      const unsigned long long* __restrict__ seed_dev) {
  if (seed_dev != nullptr) seed = *seed_dev;
  const long long total = rows * groups;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / groups;
    const int g = static_cast<int>(i % groups);
    float u[8];
    pd::philox_uniform8(seed, stream, static_cast<uint32_t>(row) + row_offset, static_cast<uint32_t>(g), u);
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (8 * g + k < cols) out[row * cols + 8 * g + k] = u[k];
  }
}

struct TensorRef {
  float* p;
  const float* g;
  float* m;
  float* v;
  long long n;
};

__global__ void sumsq_multi_kernel(const TensorRef* __restrict__ refs, float* __restrict__ out) {
  const TensorRef t = refs[blockIdx.y];
  float acc = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < t.n; i += stride) {
    if (i + 3 < t.n) {
      const float4 v = *reinterpret_cast<const float4*>(t.g + i);
      acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    } else {
      for (long long j = i; j < t.n; ++j) acc += t.g[j] * t.g[j];
    }
  }
  acc = warp_sum(acc);
  __shared__ float part[kThreads / 32];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kThreads / 32 ? part[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0 && v != 0.f) atomicAdd(out, v);
  }
}

__global__ void adamw_multi_kernel(const TensorRef* __restrict__ refs, float lr, float b1, float b2, float eps,
                                   float wd, float inv_bc1, float inv_bc2, const float* __restrict__ hyper,
                                   const float* __restrict__ grad_scale) {
  const TensorRef t = refs[blockIdx.y];
  if (hyper != nullptr) {
    lr = hyper[0];
    inv_bc1 = hyper[1];
    inv_bc2 = hyper[2];
  }
  const float gs = grad_scale ? *grad_scale : 1.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x * 4;
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < t.n; i += stride) {
    if (i + 3 < t.n) {
      float4 pp = *reinterpret_cast<float4*>(t.p + i);
      const float4 gg = *reinterpret_cast<const float4*>(t.g + i);
      float4 mm = *reinterpret_cast<float4*>(t.m + i);
      float4 vv = *reinterpret_cast<float4*>(t.v + i);
      float* pa = &pp.x; const float* ga = &gg.x; float* ma = &mm.x; float* va = &vv.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gk = ga[k] * gs;
        ma[k] = b1 * ma[k] + (1.f - b1) * gk;
        va[k] = b2 * va[k] + (1.f - b2) * gk * gk;
        pa[k] -= lr * ((ma[k] * inv_bc1) / (sqrtf(va[k] * inv_bc2) + eps) + wd * pa[k]);
      }
      *reinterpret_cast<float4*>(t.p + i) = pp;
      *reinterpret_cast<float4*>(t.m + i) = mm;
      *reinterpret_cast<float4*>(t.v + i) = vv;
    } else {
      for (long long j = i; j < t.n; ++j) {
        const float gk = t.g[j] * gs;
        t.m[j] = b1 * t.m[j] + (1.f - b1) * gk;
        t.v[j] = b2 * t.v[j] + (1.f - b2) * gk * gk;
        t.p[j] -= lr * ((t.m[j] * inv_bc1) / (sqrtf(t.v[j] * inv_bc2) + eps) + wd * t.p[j]);
      }
    }
  }
}

// hi = bf16(x), lo = bf16(x - hi): x ~= hi + lo to ~16 mantissa bits, for split-precision products.
__global__ void split_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ hi,
                                  __nv_bfloat16* __restrict__ lo, long long n) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float v = x[i];
    const __nv_bfloat16 h = __float2bfloat16(v);
    hi[i] = h;
    lo[i] = __float2bfloat16(v - __bfloat162float(h));
  }
}

// Split-precision operands of the faithfulness product, written straight in the layouts the product reads
// (three K-phases side by side): x [g, rows, cols] fp32 ->
//   along_cols = 1: out [g, rows, 3 cols] = [hi | hi | lo] per row   (V: K runs along the columns)
//   along_cols = 0: out [g, 3 rows, cols] = [hi ; lo ; hi]           (U: K runs along the rows)
__global__ void split3_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out, long long g,
                                   long long rows, long long cols, int along_cols) {
  const long long quads = cols / 4, per = rows * quads, total = g * per;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long b = i / per, rem = i - b * per, r = rem / quads, c = (rem - r * quads) * 4;
    const float4 v = *reinterpret_cast<const float4*>(x + (b * rows + r) * cols + c);
    const __nv_bfloat162 h0 = __floats2bfloat162_rn(v.x, v.y), h1 = __floats2bfloat162_rn(v.z, v.w);
    const float2 f0 = __bfloat1622float2(h0), f1 = __bfloat1622float2(h1);
    const __nv_bfloat162 l0 = __floats2bfloat162_rn(v.x - f0.x, v.y - f0.y);
    const __nv_bfloat162 l1 = __floats2bfloat162_rn(v.z - f1.x, v.w - f1.y);
    uint2 hi, lo;
    hi.x = *reinterpret_cast<const uint32_t*>(&h0); hi.y = *reinterpret_cast<const uint32_t*>(&h1);
    lo.x = *reinterpret_cast<const uint32_t*>(&l0); lo.y = *reinterpret_cast<const uint32_t*>(&l1);
    if (along_cols) {
      __nv_bfloat16* o = out + (b * rows + r) * 3 * cols + c;
      *reinterpret_cast<uint2*>(o) = hi;
      *reinterpret_cast<uint2*>(o + cols) = hi;
      *reinterpret_cast<uint2*>(o + 2 * cols) = lo;
    } else {
      __nv_bfloat16* o = out + (b * 3 * rows + r) * cols + c;
      *reinterpret_cast<uint2*>(o) = hi;
      *reinterpret_cast<uint2*>(o + rows * cols) = lo;
      *reinterpret_cast<uint2*>(o + 2 * rows * cols) = hi;
    }
  }
}

// out[c] += sum over rows of x[row, c] (bf16 in, fp32 out). Same tiling as the activity kernel.
__global__ void colsum_bf16_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ out, long long rows,
                                   int C) {
  const int cg = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + cg) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (col < C) {
    for (long long r = static_cast<long long>(blockIdx.y) * 8 + rl; r < rows;
         r += static_cast<long long>(gridDim.y) * 8) {
      const uint4 q = *reinterpret_cast<const uint4*>(x + r * C + col);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
      }
    }
  }
  __shared__ float red[8][32][8];
#pragma unroll
  for (int k = 0; k < 8; ++k) red[rl][cg][k] = acc[k];
  __syncthreads();
  if (rl == 0 && col < C) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float v = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) v += red[j][cg][k];
      atomicAdd(out + col + k, v);
    }
  }
}

}  // namespace

#define PD_CHECK_LAUNCH() (cudaGetLastError() == cudaSuccess ? 0 : 1)

extern "C" int pd_sumsq(const float* g, long long n, float* out, void* stream) {
  sumsq_kernel<<<blocks_for(n, kThreads * 4), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(g, n, out);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_clip_scale(const float* sumsq, float max_norm, float* scale, float* norm, void* stream) {
  clip_scale_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(sumsq, max_norm, scale, norm);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_adamw(float* p, const float* g, float* m, float* v, long long n, float lr, float b1,
                        float b2, float eps, float wd, float bc1, float bc2, const float* grad_scale,
                        void* stream) {
  adamw_kernel<<<blocks_for(n, kThreads * 4), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      p, g, m, v, n, lr, b1, b2, eps, wd, 1.f / bc1, 1.f / bc2, grad_scale);
  return PD_CHECK_LAUNCH();
}
// Multi-tensor forms: one launch covers every leaf of an optimizer group. `refs` is a device array
// of {p, g, m, v, n}; blockIdx.y picks the leaf, blockIdx.x strides over it. `hyper` (device, may be
// null) holds {lr, 1 / bias_correction1, 1 / bias_correction2}: a recorded launch (CUDA graph) then
// follows the schedule without being re-recorded.
extern "C" int pd_sumsq_multi(const void* refs, int count, float* out, void* stream) {
  if (count <= 0) return 0;
  sumsq_multi_kernel<<<dim3(96, count), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const TensorRef*>(refs), out);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_adamw_multi(const void* refs, int count, float lr, float b1, float b2, float eps, float wd,
                              float bc1, float bc2, const float* hyper, const float* grad_scale, void* stream) {
  if (count <= 0) return 0;
  adamw_multi_kernel<<<dim3(96, count), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const TensorRef*>(refs), lr, b1, b2, eps, wd, 1.f / bc1, 1.f / bc2, hyper, grad_scale);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_cast_bf16(const float* src, void* dst, long long n, void* stream) {
  cast_bf16_kernel<<<blocks_for(n, kThreads * 8), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<__nv_bfloat16*>(dst), n);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int d,
                              float eps, void* stream) {
  if (d % 8 != 0) return 5;
  rmsnorm_fwd_kernel<<<blocks_for(rows, kThreads / 32), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<__nv_bfloat16*>(y), rstd, rows, d, eps);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                              long long rows, int d, void* stream) {
  if (d % 8 != 0) return 5;
  rmsnorm_bwd_kernel<<<blocks_for(rows, kThreads / 32), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(dy), rstd, static_cast<__nv_bfloat16*>(dx), rows, d);
  return PD_CHECK_LAUNCH();
}
// Rotary embedding from `src` into `dst` (the same pointer rotates in place).
extern "C" int pd_rope_to(const void* src, void* dst, const float* cs, const float* sn, long long rows, int T,
                          int heads, int hd, int inverse, void* stream) {
  if (hd % 16 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(cs) & 15) == 0 && (reinterpret_cast<uintptr_t>(sn) & 15) == 0) {
    rope_vec_kernel<<<blocks_for(rows * heads * (hd / 16), kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), cs, sn, rows, T, heads, hd, inverse);
    return PD_CHECK_LAUNCH();
  }
  rope_kernel<<<blocks_for(rows * heads * (hd / 2), kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), cs, sn, rows, T, heads, hd, inverse);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_rope(void* x, const float* cs, const float* sn, long long rows, int T, int heads, int hd,
                       int inverse, void* stream) {
  return pd_rope_to(x, x, cs, sn, rows, T, heads, hd, inverse, stream);
}
extern "C" int pd_swiglu_fwd(const void* gate, const void* up, void* out, long long n, void* stream) {
  if (n % 8 != 0) return 5;
  swiglu_fwd_kernel<<<blocks_for(n, kThreads * 8), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
      static_cast<__nv_bfloat16*>(out), n);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_swiglu_bwd(const void* gate, const void* up, const void* dout, void* dgate, void* dup,
                             long long n, void* stream) {
  if (n % 8 != 0) return 5;
  swiglu_bwd_kernel<<<blocks_for(n, kThreads * 8), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(gate), static_cast<const __nv_bfloat16*>(up),
      static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(dgate),
      static_cast<__nv_bfloat16*>(dup), n);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_rowscale(const void* x, const float* s, void* y, long long rows, int d, void* stream) {
  if (d % 8 != 0) return 5;
  rowscale_kernel<<<blocks_for(rows * (d / 8), kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), s, static_cast<__nv_bfloat16*>(y), rows, d);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_rows_expand(const void* x, const void* rowmap, const float* w, void* out, long long n_rows,
                              int d, int k_sel, int rep, int use_slot, void* stream) {
  if (d % 8 != 0 || n_rows <= 0) return 5;
  rows_expand_kernel<<<blocks_for(n_rows * (d / 8), kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const int4*>(rowmap), w,
      static_cast<__nv_bfloat16*>(out), n_rows, d, k_sel, rep, use_slot);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_rows_combine(const void* padded, const long long* pos, const float* w, const int* bgroup,
                               void* y, long long tokens, int d, int k_sel, void* stream) {
  if (d % 8 != 0 || tokens <= 0) return 5;
  rows_combine_kernel<<<blocks_for(tokens * (d / 8), kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(padded), pos, w, bgroup, static_cast<__nv_bfloat16*>(y), tokens, d, k_sel);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_ci_squash(const void* pre, void* lower, void* upper, long long n, float alpha, void* stream) {
  if (n % 8 != 0) return 5;
  ci_squash_kernel<<<blocks_for(n, kThreads * 8), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(pre), static_cast<__nv_bfloat16*>(lower),
      static_cast<__nv_bfloat16*>(upper), n, alpha);
  return PD_CHECK_LAUNCH();
}

extern "C" int pd_ci_squash_activity(const void* pre, void* lower, float* colsum, long long rows, int C,
                                     float gamma, int normalize_at_one, float alpha, const float* gamma_dev,
                                     void* stream) {
  if (C % 8 != 0) return 5;
  const int gx = (C + 255) / 256;
  int gy = (148 * 4 + gx - 1) / gx;
  if (gy > (rows + 7) / 8) gy = static_cast<int>((rows + 7) / 8);
  if (gy < 1) gy = 1;
  const float g2 = gamma * gamma;
  ci_squash_activity_kernel<<<dim3(gx, gy), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(pre), static_cast<__nv_bfloat16*>(lower), colsum, rows, C, g2,
      normalize_at_one ? 1.f + g2 : 1.f, alpha, gamma_dev, normalize_at_one);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_ci_squash_activity_bwd(const void* pre, const void* dlower, const float* dcol, void* dpre,
                                         long long rows, int C, float gamma, int normalize_at_one, float alpha,
                                         const float* gamma_dev, void* stream) {
  if (C % 8 != 0) return 5;
  const float g2 = gamma * gamma;
  const int gx = (C + 255) / 256;
  long long gy = (148 * 8 + gx - 1) / gx;
  if (gy > (rows + 7) / 8) gy = (rows + 7) / 8;
  if (gy < 1) gy = 1;
  ci_squash_activity_bwd_kernel<<<dim3(gx, static_cast<unsigned>(gy)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(pre), static_cast<const __nv_bfloat16*>(dlower), dcol,
      static_cast<__nv_bfloat16*>(dpre), rows, C, g2, normalize_at_one ? 1.f + g2 : 1.f, alpha, gamma_dev,
      normalize_at_one);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_ci_squash_activity_jobs(const void* pre, void* lower, float* colsum, const void* rowmap,
                                          const int* bgroup, long long n_rows, int c, long long pitch,
                                          float gamma, int normalize_at_one, float alpha, const float* gamma_dev,
                                          void* stream) {
  if (c % 8 != 0 || pitch % 8 != 0 || n_rows % 128 != 0 || n_rows <= 0) return 5;
  const float g2 = gamma * gamma;
  ci_squash_activity_jobs_kernel<<<dim3((c + 255) / 256, static_cast<unsigned>(n_rows / 128)), 256, 0,
                                   static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(pre), static_cast<__nv_bfloat16*>(lower), colsum,
      static_cast<const int4*>(rowmap), bgroup, c, pitch, g2, normalize_at_one ? 1.f + g2 : 1.f, alpha, gamma_dev,
      normalize_at_one);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_ci_squash_activity_jobs_bwd(const void* pre, const void* dlower, const float* dcol,
                                              const long long* experts, void* dpre, long long tokens, int k_sel,
                                              int c, float gamma, int normalize_at_one, float alpha,
                                              const float* gamma_dev, void* stream) {
  if (c % 8 != 0 || tokens <= 0) return 5;
  const float g2 = gamma * gamma;
  ci_squash_activity_jobs_bwd_kernel<<<blocks_for(tokens * k_sel * (c / 8), kThreads), kThreads, 0,
                                       static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(pre), static_cast<const __nv_bfloat16*>(dlower), dcol, experts,
      static_cast<__nv_bfloat16*>(dpre), tokens, k_sel, c, g2, normalize_at_one ? 1.f + g2 : 1.f, alpha, gamma_dev,
      normalize_at_one);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_vocab_kl(const void* lc, const void* lm, void* dlm, float* kl, long long rows, int V,
                           long long ld, void* stream) {
  if (ld % 8 != 0 || rows <= 0) return 5;
  // 512 threads per row: four rows in flight per SM keep the rows being re-read (passes 2 and 3)
  // within L2 while different rows' load-bound and exp-bound passes still overlap on the SM
  vocab_kl_kernel<<<static_cast<unsigned>(rows), 512, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(lc), static_cast<const __nv_bfloat16*>(lm),
      static_cast<__nv_bfloat16*>(dlm), kl, V, ld);
  return PD_CHECK_LAUNCH();
}

extern "C" int pd_philox_uniform(float* out, long long rows, int cols, unsigned long long seed, unsigned int stream,
                                 unsigned int row_offset, const unsigned long long* seed_dev, void* stream_v) {
  const int groups = (cols + 7) / 8;
  philox_uniform_kernel<<<blocks_for(rows * groups, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream_v)>>>(
      out, rows, groups, cols, seed, stream, row_offset, seed_dev);
  return PD_CHECK_LAUNCH();
}
extern "C" int pd_split_bf16(const float* x, void* hi, void* lo, long long n, void* stream) {
  split_bf16_kernel<<<blocks_for(n, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      x, static_cast<__nv_bfloat16*>(hi), static_cast<__nv_bfloat16*>(lo), n);
  return PD_CHECK_LAUNCH();
}

extern "C" int pd_split3_bf16(const float* x, void* out, long long g, long long rows, long long cols,
                              int along_cols, void* stream) {
  if (cols % 4 != 0 || g <= 0 || rows <= 0) return 5;
  split3_bf16_kernel<<<blocks_for(g * rows * (cols / 4), kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      x, static_cast<__nv_bfloat16*>(out), g, rows, cols, along_cols);
  return PD_CHECK_LAUNCH();
}

extern "C" int pd_colsum_bf16(const void* x, float* out, long long rows, int C, void* stream) {
  if (C % 8 != 0) return 5;
  const int gx = (C + 255) / 256;
  int gy = (148 * 4 + gx - 1) / gx;
  if (gy > (rows + 7) / 8) gy = static_cast<int>((rows + 7) / 8);
  if (gy < 1) gy = 1;
  colsum_bf16_kernel<<<dim3(gx, gy), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), out, rows, C);
  return PD_CHECK_LAUNCH();
}
