// Column sum of a bf16 matrix (the bias-gradient reduction) for callers that must not allocate.
//
// This entry point has no counterpart in the reference: it exists for hosts of this library that cannot
// call cudaMalloc around a kernel launch.  Typical cases: a robot-side control loop or serving thread with a
// hard latency budget (an allocation may synchronise the whole device and can fail under memory pressure), a
// process that was handed a fixed memory budget at start-up and may not grow it, and C/C++ callers that link
// the shared library directly and have no tensor allocator at hand.  The regular entry points
// (otb_colsum_bf16 + otb_colsum_partials) expect the caller to supply an fp32 scratch buffer for the partial
// sums; here that scratch is a fixed array inside the library's device image.
//
// Limits and rules
//   * H (columns) must be a multiple of 8 and at most OTB_NOALLOC_COLSUM_MAX_H; rows >= 1; lda >= H and a
//     multiple of 8; `a` and `out` 16-byte aligned.  Anything else is refused with a negative code and
//     nothing is launched (otb_noalloc_strerror turns the code into text).
//   * The scratch holds OTB_NOALLOC_COLSUM_MAX_BLOCKS x OTB_NOALLOC_COLSUM_MAX_H floats (2 MiB).  Every GPU
//     that loads the library keeps this array resident until the process exits.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, once per device,
//     with that device current).  Make that first call outside of any stream capture.
//   * All calls on a device share the one array and it keeps the previous call's contents.  Nothing in it has
//     to start at zero: each launch overwrites every element it later reads.  Two calls whose kernels overlap
//     in time on the same GPU (different streams) race on the scratch; serialise them.
//   * `a`, `out` and `stream` must belong to the device that is current in the calling thread: the scratch
//     address is looked up for the current device and nothing checks the pointers against it.  A pointer of
//     another GPU would be combined with this GPU's scratch.
//   * The per-device address cache is filled without a lock.  Two host threads that make the very first call
//     on a device at the same moment both store the same value, which is harmless, but the cache is not
//     otherwise thread-safe: make the first call per device from one thread before sharing the entry point.
//   * No cudaMalloc, cudaFree or other allocating routine is called, on any path.
#pragma once
#include <cuda_runtime.h>

#define OTB_NOALLOC_COLSUM_MAX_H 8192
#define OTB_NOALLOC_COLSUM_MAX_BLOCKS 64

#ifdef __cplusplus
extern "C" {
#endif

// out[c] = sum_r a[r * lda + c]  for c in [0, H), accumulated in fp32, written as bf16.
// a: bf16 [rows, H] with row stride lda (elements); out: bf16 [H].  Returns 0, a negative argument code, or a
// positive cudaError_t.
int otb_colsum_bf16_noalloc(const void* a, long long rows, int H, long long lda, void* out, cudaStream_t stream);

// Text for the codes returned by otb_colsum_bf16_noalloc.
const char* otb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
