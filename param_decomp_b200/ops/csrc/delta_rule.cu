// Gated delta rule (linear-attention recurrence of the Qwen3.5 DeltaNet layers) and the causal
// depthwise conv1d + SiLU in front of it, forward and backward.
//
//   S_t = exp(g_t) S_{t-1};  delta_t = beta_t (v_t - S_t^T k_t);  S_t += k_t delta_t^T;  o_t = S_t^T q_t
//
// One CTA per (batch, head). The state S [DK, DV] stays on chip for the whole sequence: in the
// forward each thread owns one column of S in registers, so a step is three passes over DK registers
// and nothing is exchanged between threads but the k/q vectors (shared memory, double-buffered).
// The state at the start of every 64-token chunk is written out for the backward, which walks the
// chunks in reverse: it replays a chunk from its checkpoint, saving the pre-step state of each token
// to a scratch area, then runs the adjoint recurrence with the state's cotangent G and the current
// state in shared memory (rows padded by one float so both column-wise and row-wise passes are
// conflict-free).
//
// Replaces the XLA einsum + scan lowering of param_decomp/target_ports/qwen3_5_moe.py:89-158,187-293;
// the torch restatement of the same recurrence (`models/ports.py`) is the oracle.
#include "common.cuh"

namespace {

constexpr int kChunk = 64;

template <int DK, int DV>
__global__ void __launch_bounds__(DV) delta_fwd_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                       const float* __restrict__ v, const float* __restrict__ g,
                                                       const float* __restrict__ beta, float* __restrict__ o,
                                                       float* __restrict__ ckpt, int T, int H) {
  __shared__ float sk[2][DK], sq[2][DK];
  const int b = blockIdx.x / H, h = blockIdx.x % H, j = threadIdx.x;
  const long long row0 = (static_cast<long long>(b) * T) * H + h;  // (b, t=0, h)
  const int n_chunks = (T + kChunk - 1) / kChunk;
  float S[DK];
#pragma unroll
  for (int i = 0; i < DK; ++i) S[i] = 0.0f;
  auto load_kq = [&](int t, int buf) {
    const long long r = (row0 + static_cast<long long>(t) * H) * DK;
    for (int i = j; i < DK; i += DV) {
      sk[buf][i] = k[r + i];
      sq[buf][i] = q[r + i];
    }
  };
  load_kq(0, 0);
  __syncthreads();
  for (int t = 0; t < T; ++t) {
    const int buf = t & 1;
    if (t + 1 < T) load_kq(t + 1, buf ^ 1);
    if (ckpt != nullptr && (t % kChunk) == 0) {
      float* c = ckpt + ((static_cast<long long>(blockIdx.x) * n_chunks + t / kChunk) * DK) * DV;
#pragma unroll
      for (int i = 0; i < DK; ++i) c[i * DV + j] = S[i];
    }
    const long long r = row0 + static_cast<long long>(t) * H;
    const float a = __expf(g[r]), bt = beta[r];
    float mem = 0.0f;
#pragma unroll
    for (int i = 0; i < DK; ++i) {
      S[i] *= a;
      mem = fmaf(S[i], sk[buf][i], mem);
    }
    const float delta = (v[r * DV + j] - mem) * bt;
    float out = 0.0f;
#pragma unroll
    for (int i = 0; i < DK; ++i) {
      S[i] = fmaf(sk[buf][i], delta, S[i]);
      out = fmaf(S[i], sq[buf][i], out);
    }
    o[r * DV + j] = out;
    __syncthreads();
  }
}

template <int N>
__device__ __forceinline__ float block_sum(float x, float* red) {
  // N threads (a multiple of 32, at most 128); every thread gets the total
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) x += __shfl_xor_sync(0xffffffffu, x, s);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = x;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int w = 0; w < N / 32; ++w) tot += red[w];
  return tot;
}

template <int DK, int DV>
__global__ void __launch_bounds__((DK > DV ? DK : DV)) delta_bwd_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ g,
    const float* __restrict__ beta, const float* __restrict__ d_o, const float* __restrict__ ckpt,
    float* __restrict__ scratch, float* __restrict__ dq, float* __restrict__ dk, float* __restrict__ dv,
    float* __restrict__ dg, float* __restrict__ dbeta, int T, int H) {
  constexpr int NT = DK > DV ? DK : DV;
  constexpr int LD = DV + 1;
  extern __shared__ float smem[];
  float* sP = smem;                 // [DK][LD] state before the step (S_{t-1})
  float* sG = sP + DK * LD;         // [DK][LD] cotangent of the state after the step
  float* s_k = sG + DK * LD;        // [DK]
  float* s_q = s_k + DK;            // [DK]
  float* s_do = s_q + DK;           // [DV]
  float* s_delta = s_do + DV;       // [DV]
  float* s_dm = s_delta + DV;       // [DV]
  float* red = s_dm + DV;           // [4]
  const int b = blockIdx.x / H, h = blockIdx.x % H, tid = threadIdx.x;
  const long long row0 = (static_cast<long long>(b) * T) * H + h;
  const int n_chunks = (T + kChunk - 1) / kChunk;
  float* my_scratch = scratch + static_cast<long long>(blockIdx.x) * kChunk * DK * DV;
  for (int i = tid; i < DK * LD; i += NT) sG[i] = 0.0f;
  __syncthreads();

  for (int c = n_chunks - 1; c >= 0; --c) {
    const int t_lo = c * kChunk, t_hi = min(T, t_lo + kChunk);
    // ---- replay the chunk from its checkpoint, saving S_{t-1} for every t ----
    if (tid < DV) {
      const int j = tid;
      float S[DK];
      const float* cp = ckpt + ((static_cast<long long>(blockIdx.x) * n_chunks + c) * DK) * DV;
#pragma unroll
      for (int i = 0; i < DK; ++i) S[i] = cp[i * DV + j];
      for (int t = t_lo; t < t_hi; ++t) {
        float* sp = my_scratch + static_cast<long long>(t - t_lo) * DK * DV;
#pragma unroll
        for (int i = 0; i < DK; ++i) sp[i * DV + j] = S[i];
        if (t + 1 == t_hi) break;
        const long long r = row0 + static_cast<long long>(t) * H;
        const float a = __expf(g[r]), bt = beta[r];
        const float* kr = k + r * DK;
        float mem = 0.0f;
#pragma unroll
        for (int i = 0; i < DK; ++i) {
          S[i] *= a;
          mem = fmaf(S[i], __ldg(kr + i), mem);
        }
        const float delta = (v[r * DV + j] - mem) * bt;
#pragma unroll
        for (int i = 0; i < DK; ++i) S[i] = fmaf(__ldg(kr + i), delta, S[i]);
      }
    }
    __syncthreads();
    // ---- adjoint recurrence over the chunk, last token first ----
    for (int t = t_hi - 1; t >= t_lo; --t) {
      const long long r = row0 + static_cast<long long>(t) * H;
      const float a = __expf(g[r]), bt = beta[r];
      const float* sp = my_scratch + static_cast<long long>(t - t_lo) * DK * DV;
      if (tid < DK) {
        s_k[tid] = k[r * DK + tid];
        s_q[tid] = q[r * DK + tid];
      }
      if (tid < DV) {
        s_do[tid] = d_o[r * DV + tid];
        for (int i = 0; i < DK; ++i) sP[i * LD + tid] = sp[i * DV + tid];
      }
      __syncthreads();
      float dbeta_part = 0.0f;
      if (tid < DV) {  // column pass: G += q do^T; m, delta; d delta = G^T k
        const int j = tid;
        const float doj = s_do[j];
        float m = 0.0f, dd = 0.0f;
        for (int i = 0; i < DK; ++i) {
          const float gij = fmaf(s_q[i], doj, sG[i * LD + j]);
          sG[i * LD + j] = gij;
          m = fmaf(a * sP[i * LD + j], s_k[i], m);
          dd = fmaf(gij, s_k[i], dd);
        }
        const float resid = v[r * DV + j] - m;
        s_delta[j] = bt * resid;
        s_dm[j] = -bt * dd;
        dv[r * DV + j] = bt * dd;
        dbeta_part = dd * resid;
      }
      const float dbeta_t = block_sum<NT>(dbeta_part, red);  // also orders the column pass before the row pass
      float da_part = 0.0f;
      if (tid < DK) {  // row pass: sums over the value index
        const int i = tid;
        const float ki = s_k[i];
        float ddo = 0.0f;  // delta . do
        for (int j = 0; j < DV; ++j) ddo = fmaf(s_delta[j], s_do[j], ddo);
        float acc_q = 0.0f, acc_k = 0.0f;
        for (int j = 0; j < DV; ++j) {
          const float p = sP[i * LD + j], gij = sG[i * LD + j];
          const float sd = a * p;
          acc_q = fmaf(sd, s_do[j], acc_q);
          acc_k = fmaf(gij, s_delta[j], acc_k);
          acc_k = fmaf(sd, s_dm[j], acc_k);
          da_part = fmaf(fmaf(ki, s_dm[j], gij), p, da_part);
        }
        dq[r * DK + i] = fmaf(ki, ddo, acc_q);
        dk[r * DK + i] = acc_k;
      }
      const float da = block_sum<NT>(da_part, red);
      if (tid == 0) {
        dg[r] = da * a;
        dbeta[r] = dbeta_t;
      }
      if (tid < DV) {  // G_{t-1} = a (G + k dm^T)
        const int j = tid;
        const float dmj = s_dm[j];
        for (int i = 0; i < DK; ++i) sG[i * LD + j] = a * fmaf(s_k[i], dmj, sG[i * LD + j]);
      }
      __syncthreads();
    }
  }
}

// ---- causal depthwise conv1d + SiLU: y[b,t,c] = silu(sum_j w[c,j] x[b,t-(K-1)+j,c]) ----
__global__ void conv1d_silu_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                       __nv_bfloat16* __restrict__ y, int B, int T, int D, int K) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(B) * T * D;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % D);
  const int t = static_cast<int>((idx / D) % T);
  float acc = 0.0f;
  for (int j = 0; j < K; ++j) {
    const int ts = t - (K - 1) + j;
    if (ts >= 0) acc = fmaf(__bfloat162float(w[c * K + j]), __bfloat162float(x[idx + static_cast<long long>(ts - t) * D]), acc);
  }
  y[idx] = __float2bfloat16(acc / (1.0f + __expf(-acc)));
}

// dx[b,s,c] = sum_j w[c,j] dpre[b,s+(K-1)-j,c];  dw[c,j] += sum_{b,t} dpre[b,t,c] x[b,t-(K-1)+j,c]
__global__ void conv1d_silu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                       const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx,
                                       float* __restrict__ dw, int B, int T, int D, int K) {
  // one thread per (b, c), walking t: keeps a K-deep window of dpre and x in registers (K <= 8)
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= D) return;
  float wk[8], dwk[8], win_x[8];
  for (int j = 0; j < 8; ++j) {
    wk[j] = j < K ? __bfloat162float(w[c * K + j]) : 0.0f;
    dwk[j] = 0.0f;
    win_x[j] = 0.0f;  // x[t-(K-1)+j]
  }
  const long long base = static_cast<long long>(b) * T * D + c;
  // pass 1 (forward in t): dpre and dw
  for (int t = 0; t < T; ++t) {
    for (int j = 0; j + 1 < K; ++j) win_x[j] = win_x[j + 1];
    win_x[K - 1] = __bfloat162float(x[base + static_cast<long long>(t) * D]);
    float pre = 0.0f;
    for (int j = 0; j < K; ++j) pre = fmaf(wk[j], win_x[j], pre);
    const float sg = 1.0f / (1.0f + __expf(-pre));
    const float dpre = __bfloat162float(dy[base + static_cast<long long>(t) * D]) * sg * (1.0f + pre * (1.0f - sg));
    for (int j = 0; j < K; ++j) dwk[j] = fmaf(dpre, win_x[j], dwk[j]);
  }
  for (int j = 0; j < K; ++j) atomicAdd(dw + c * K + j, dwk[j]);
  // pass 2 (backward in t): dx[s] needs dpre[s .. s+K-1]; recompute dpre on the fly with a second window
  // window of x for recomputing pre at tokens s..s+K-1 would need 2K-1 values: simpler to recompute per token
  for (int s = T - 1; s >= 0; --s) {
    float acc = 0.0f;
    for (int j = 0; j < K; ++j) {
      const int t = s + (K - 1) - j;  // token whose window position j reads x[s]
      if (t >= T) continue;
      float pre = 0.0f;
      for (int jj = 0; jj < K; ++jj) {
        const int ts = t - (K - 1) + jj;
        if (ts >= 0) pre = fmaf(wk[jj], __bfloat162float(x[base + static_cast<long long>(ts) * D]), pre);
      }
      const float sg = 1.0f / (1.0f + __expf(-pre));
      const float dpre = __bfloat162float(dy[base + static_cast<long long>(t) * D]) * sg * (1.0f + pre * (1.0f - sg));
      acc = fmaf(wk[j], dpre, acc);
    }
    dx[base + static_cast<long long>(s) * D] = __float2bfloat16(acc);
  }
}

template <int DK, int DV>
int launch_fwd(const float* q, const float* k, const float* v, const float* g, const float* beta, float* o,
               float* ckpt, int B, int T, int H, cudaStream_t st) {
  delta_fwd_kernel<DK, DV><<<B * H, DV, 0, st>>>(q, k, v, g, beta, o, ckpt, T, H);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

template <int DK, int DV>
int launch_bwd(const float* q, const float* k, const float* v, const float* g, const float* beta, const float* d_o,
               const float* ckpt, float* scratch, float* dq, float* dk, float* dv, float* dg, float* dbeta, int B,
               int T, int H, cudaStream_t st) {
  constexpr int NT = DK > DV ? DK : DV;
  const int smem = (2 * DK * (DV + 1) + 2 * DK + 3 * DV + 4) * 4;
  auto kern = delta_bwd_kernel<DK, DV>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return 300;
    configured = true;
  }
  kern<<<B * H, NT, smem, st>>>(q, k, v, g, beta, d_o, ckpt, scratch, dq, dk, dv, dg, dbeta, T, H);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

}  // namespace

#define PD_DELTA_DISPATCH(FN, ...)                                  \
  if (dk == 64 && dv == 64) return FN<64, 64>(__VA_ARGS__);         \
  if (dk == 128 && dv == 128) return FN<128, 128>(__VA_ARGS__);     \
  if (dk == 64 && dv == 128) return FN<64, 128>(__VA_ARGS__);       \
  if (dk == 32 && dv == 32) return FN<32, 32>(__VA_ARGS__);         \
  return pd::kBadArgument;

// q, k [B,T,H,dk], v, o [B,T,H,dv], g, beta [B,T,H] fp32 contiguous; ckpt [B*H, ceil(T/64), dk, dv] or null
extern "C" int pd_delta_rule_fwd(const float* q, const float* k, const float* v, const float* g, const float* beta,
                                 float* o, float* ckpt, int B, int T, int H, int dk, int dv, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PD_DELTA_DISPATCH(launch_fwd, q, k, v, g, beta, o, ckpt, B, T, H, st)
}

// scratch: [B*H, 64, dk, dv] fp32
extern "C" int pd_delta_rule_bwd(const float* q, const float* k, const float* v, const float* g, const float* beta,
                                 const float* d_o, const float* ckpt, float* scratch, float* dq, float* dk_, float* dv_,
                                 float* dg, float* dbeta, int B, int T, int H, int dk, int dv, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  PD_DELTA_DISPATCH(launch_bwd, q, k, v, g, beta, d_o, ckpt, scratch, dq, dk_, dv_, dg, dbeta, B, T, H, st)
}

extern "C" int pd_conv1d_silu_fwd(const void* x, const void* w, void* y, int B, int T, int D, int K, void* stream) {
  if (K < 1 || K > 8) return pd::kBadArgument;
  const long long total = static_cast<long long>(B) * T * D;
  conv1d_silu_fwd_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), B, T,
      D, K);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// dw [D, K] fp32 must be zero on entry
extern "C" int pd_conv1d_silu_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw, int B, int T,
                                  int D, int K, void* stream) {
  if (K < 1 || K > 8) return pd::kBadArgument;
  dim3 grid((D + 127) / 128, B);
  conv1d_silu_bwd_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(dy), static_cast<__nv_bfloat16*>(dx), dw, B, T, D, K);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}
