// Allocation-free global-norm clip factor (see noalloc.h for the contract and who it is for).
//
// Two launches on the caller's stream: (1) every block writes the sum of squares of its grid-stride
// share of `g` into its own slot of the static scratch array; (2) one block adds the slots in a
// fixed order and writes norm and scale. No atomics, so the result is bit-reproducible, and no slot
// is read that this call did not write.
#include <cuda_runtime.h>

#include <mutex>

#include "noalloc.h"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxDevices = 64;

// The scratch itself. In host code this name is only a handle for cudaGetSymbolAddress, never a
// device pointer; kernels receive the resolved address as an argument.
static __device__ __align__(256) float g_clip_scratch[PD_NOALLOC_CLIP_SCRATCH_SLOTS];

float* g_scratch_addr[kMaxDevices] = {};  // resolved once per device
std::mutex g_scratch_mutex;               // two host threads may make the first call on a device together

__global__ void partial_sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ slots) {
  float acc = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float v = g[i];
    acc += v * v;
  }
  __shared__ float part[kThreads];
  part[threadIdx.x] = acc;
  __syncthreads();
  for (int s = kThreads / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) part[threadIdx.x] += part[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) slots[blockIdx.x] = part[0];
}

__global__ void finish_clip_kernel(const float* __restrict__ slots, int n_slots, float max_norm,
                                   float* __restrict__ scale_out, float* __restrict__ norm_out) {
  __shared__ float part[kThreads];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n_slots; i += kThreads) acc += slots[i];
  part[threadIdx.x] = acc;
  __syncthreads();
  for (int s = kThreads / 2; s > 0; s >>= 1) {
    if (threadIdx.x < s) part[threadIdx.x] += part[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float norm = sqrtf(part[0]);
    *norm_out = norm;
    *scale_out = max_norm > 0.f ? fminf(max_norm / (norm + 1e-6f), 1.f) : 1.f;
  }
}

// Set-up, once per device, with that device current: turn the symbol into a device address.
int resolve_scratch(float** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return PD_NOALLOC_SETUP_FAILED;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);  // (locking a std::mutex allocates nothing)
  if (g_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_clip_scratch) != cudaSuccess || ptr == nullptr)
      return PD_NOALLOC_SETUP_FAILED;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return PD_NOALLOC_OK;
}

}  // namespace

extern "C" int pd_clip_scale_noalloc(const float* g, long long n, float max_norm, float* scale_out,
                                     float* norm_out, void* stream_v) {
  if (g == nullptr || scale_out == nullptr || norm_out == nullptr || n <= 0) return PD_NOALLOC_BAD_ARGUMENT;
  if (n > PD_NOALLOC_CLIP_MAX_ELEMS) return PD_NOALLOC_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = resolve_scratch(&scratch);
  if (rc != PD_NOALLOC_OK) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  long long want = (n + kThreads - 1) / kThreads;
  const int blocks = static_cast<int>(want < PD_NOALLOC_CLIP_SCRATCH_SLOTS ? want : PD_NOALLOC_CLIP_SCRATCH_SLOTS);
  partial_sumsq_kernel<<<blocks, kThreads, 0, stream>>>(g, n, scratch);
  finish_clip_kernel<<<1, kThreads, 0, stream>>>(scratch, blocks, max_norm, scale_out, norm_out);
  return cudaGetLastError() == cudaSuccess ? PD_NOALLOC_OK : PD_NOALLOC_LAUNCH_FAILED;
}

extern "C" const char* pd_noalloc_strerror(int status) {
  switch (status) {
    case PD_NOALLOC_OK: return "ok";
    case PD_NOALLOC_TOO_LARGE:
      return "input larger than PD_NOALLOC_CLIP_MAX_ELEMS (2^31 elements): split the tensor and combine the norms";
    case PD_NOALLOC_BAD_ARGUMENT: return "null pointer or non-positive element count";
    case PD_NOALLOC_SETUP_FAILED: return "could not resolve the device address of the static scratch array";
    case PD_NOALLOC_LAUNCH_FAILED: return "kernel launch failed";
    default: return "unknown status";
  }
}
