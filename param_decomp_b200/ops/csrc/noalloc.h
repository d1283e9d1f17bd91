// Entry points of libpdb200 that never allocate memory.
//
// This interface has no counterpart in the reference implementation.
//
// Who needs it: code that runs where cudaMalloc is off limits. Examples are a host thread that
// drives a step from inside a region where the CUDA allocator must not be touched (a stream being
// captured into a graph, a real-time control loop with a fixed memory budget, a plugin loaded into
// a process whose allocator is owned by someone else), and embedders who hand this library
// pre-sized buffers and forbid it to grow the process's device footprint behind their back.
// Such callers pass their own inputs and outputs; any scratch the computation needs lives in a
// fixed array inside the library image, so nothing is allocated or freed by the call.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest gradient tensor the allocation-free clip accepts, in elements.
#define PD_NOALLOC_CLIP_MAX_ELEMS (1ll << 31)
// Slots of per-block partial sums kept in the library's static device array (4 KiB per device).
#define PD_NOALLOC_CLIP_SCRATCH_SLOTS 1024

enum PdNoAllocStatus {
  PD_NOALLOC_OK = 0,
  PD_NOALLOC_TOO_LARGE = 1,      // n exceeds PD_NOALLOC_CLIP_MAX_ELEMS
  PD_NOALLOC_BAD_ARGUMENT = 2,   // null pointer or n <= 0
  PD_NOALLOC_SETUP_FAILED = 3,   // the static scratch array's device address could not be resolved
  PD_NOALLOC_LAUNCH_FAILED = 4,
};

// Global-norm clipping factor of one fp32 gradient tensor, computed without allocating:
//   *norm_out  = sqrt(sum g[i]^2)
//   *scale_out = max_norm > 0 ? min(max_norm / (*norm_out + 1e-6), 1) : 1
// It is the allocation-free twin of pd_sumsq + pd_clip_scale (those need a caller-zeroed
// accumulator; this one needs none). `g`, `scale_out`, `norm_out` are device pointers owned by the
// caller; `stream` is a cudaStream_t.
//
// Scratch: per-block partial sums go to a file-scope static device array of
// PD_NOALLOC_CLIP_SCRATCH_SLOTS floats. Every GPU that loads the library holds that array until
// the process exits. Every call overwrites exactly the slots it later reads, so nothing has to be
// cleared between calls, but the array is shared by all calls on a device: two calls whose
// kernels overlap on the GPU (different streams, no ordering between them) race on it. Order such
// calls on one stream or with events.
//
// The first call on each device resolves the array's device address (one
// cudaGetSymbolAddress with that device current) and caches it. Make that first call outside any
// stream capture. The cache is guarded by a mutex, so host threads may make their first calls
// concurrently; that guards the address only, not the array's contents (see above).
//
// Returns a PdNoAllocStatus; pd_noalloc_strerror turns it into text. Sizes beyond
// PD_NOALLOC_CLIP_MAX_ELEMS are refused with PD_NOALLOC_TOO_LARGE and nothing is launched.
int pd_clip_scale_noalloc(const float* g, long long n, float max_norm, float* scale_out, float* norm_out,
                          void* stream);

const char* pd_noalloc_strerror(int status);

#ifdef __cplusplus
}
#endif
