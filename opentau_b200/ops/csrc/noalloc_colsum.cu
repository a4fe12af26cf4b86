// Allocation-free column sum: see noalloc_colsum.h for who needs it and for the rules of use.
#include "noalloc_colsum.h"

#include <cuda_bf16.h>
#include <stdint.h>

namespace {

// Scratch for the per-block partial sums.  In host code this name is only a stand-in for the symbol: its
// device address has to be asked for (cudaGetSymbolAddress) before it can be given to a kernel.
static __device__ __align__(256) float g_colsum_scratch[OTB_NOALLOC_COLSUM_MAX_BLOCKS * OTB_NOALLOC_COLSUM_MAX_H];

constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {nullptr};

enum {
  ERR_NULL = -1,
  ERR_ROWS = -2,
  ERR_H = -3,
  ERR_H_TOO_LARGE = -4,
  ERR_LDA = -5,
  ERR_ALIGN = -6,
  ERR_DEVICE = -7,
};

__device__ __forceinline__ void unpack8(const __nv_bfloat16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
    float2 f = __bfloat1622float2(b);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// Stage 1: block (x, y) sums rows [y * rows_per_block, ...) of 8 columns per thread into partial[y][c].
__global__ void colsum_stage1(const __nv_bfloat16* __restrict__ a, long long rows, int H, long long lda,
                              float* __restrict__ partial, int rows_per_block) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= H) return;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  const long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (long long r = r0; r < r1; ++r) {
    float v[8];
    unpack8(a + r * lda + c, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += v[e];
  }
  float* o = partial + (long long)blockIdx.y * H + c;
#pragma unroll
  for (int e = 0; e < 8; ++e) o[e] = acc[e];
}

// Stage 2: fixed-order sum over the partial rows (deterministic), bf16 result.
__global__ void colsum_stage2(const float* __restrict__ partial, int nrows, int H, __nv_bfloat16* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int r = 0; r < nrows; ++r) s += partial[(long long)r * H + c];
  out[c] = __float2bfloat16(s);
}

}  // namespace

extern "C" const char* otb_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case ERR_NULL: return "null input or output pointer";
    case ERR_ROWS: return "rows must be >= 1";
    case ERR_H: return "H must be a positive multiple of 8";
    case ERR_H_TOO_LARGE: return "H exceeds OTB_NOALLOC_COLSUM_MAX_H (8192): the built-in scratch is too small";
    case ERR_LDA: return "lda must be >= H and a multiple of 8";
    case ERR_ALIGN: return "input and output must be 16-byte aligned";
    case ERR_DEVICE: return "current device index is outside the supported range";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown code";
  }
}

extern "C" int otb_colsum_bf16_noalloc(const void* a, long long rows, int H, long long lda, void* out,
                                       cudaStream_t stream) {
  if (a == nullptr || out == nullptr) return ERR_NULL;
  if (rows < 1) return ERR_ROWS;
  if (H < 8 || (H % 8)) return ERR_H;
  if (H > OTB_NOALLOC_COLSUM_MAX_H) return ERR_H_TOO_LARGE;
  if (lda < H || (lda % 8)) return ERR_LDA;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out)) & 15) return ERR_ALIGN;

  // One-time set-up per device (done by the first call on that device, with it current): resolve the device
  // address of the scratch symbol.  Keep this first call out of stream capture.
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= MAX_DEVICES) return ERR_DEVICE;
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_colsum_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_scratch_addr[dev] = p;
  }
  float* scratch = g_scratch_addr[dev];

  long long rpb = (rows + OTB_NOALLOC_COLSUM_MAX_BLOCKS - 1) / OTB_NOALLOC_COLSUM_MAX_BLOCKS;
  if (rpb < 1) rpb = 1;
  const int nblocks = static_cast<int>((rows + rpb - 1) / rpb);   // <= MAX_BLOCKS
  const dim3 grid1((H / 8 + 127) / 128, nblocks);
  colsum_stage1<<<grid1, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(a), rows, H, lda, scratch,
                                           static_cast<int>(rpb));
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  colsum_stage2<<<(H + 255) / 256, 256, 0, stream>>>(scratch, nblocks, H, static_cast<__nv_bfloat16*>(out));
  return static_cast<int>(cudaGetLastError());
}
