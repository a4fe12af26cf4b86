// Peer-memory communication runtime and the fused data-parallel step kernels.
//
// Every rank owns buffers allocated with cudaMalloc and exported through CUDA IPC; each rank maps all
// peers' buffers, so a kernel can read or write any rank's memory over NVLink / NVSwitch with plain
// loads and stores.  On top of that:
//
//   barrier           flag exchange with release/acquire at system scope
//   reduce_scatter    this rank's shard of the gradient = sum over ranks (peer LOADS), bf16 -> fp32,
//                     plus block partials of the squared norm
//   norm_exchange     all-gather of the per-rank squared norms through peer STORES, clip coefficient
//   adamw_allgather   fused AdamW on the fp32 master shard, result written as bf16 into EVERY rank's
//                     parameter buffer (peer stores) -- the all-gather costs no extra pass
//
// All waits are bounded (clock budget passed by the host); on expiry the kernel records
// {kernel, stage, peer} in the status word and returns.  No TMA, no multicast loads.
#include "common.cuh"

namespace otb {

constexpr int MAX_RANKS = 8;
constexpr unsigned KID_BARRIER = 10, KID_NORMX = 11;

struct PeerTable {
  void* ptr[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// flags: each rank has int flags[MAX_RANKS * slots]; slot s, source r at flags[s * MAX_RANKS + r].
// Thread i signals peer i (writes `epoch` into peer i's flags[slot][rank]) and waits for peer i's signal.
__global__ void barrier_kernel(PeerTable flags, int rank, int world, int slot, int epoch, long long budget,
                               KernelStatus* status) {
  const int i = threadIdx.x;
  if (i >= world) return;
  __threadfence_system();
  int* remote = static_cast<int*>(flags.ptr[i]) + slot * MAX_RANKS + rank;
  st_release_sys(remote, epoch);
  const int* mine = static_cast<const int*>(flags.ptr[rank]) + slot * MAX_RANKS + i;
  const long long t0 = clock64();
  while (ld_acquire_sys(mine) < epoch) {
    if (clock64() - t0 > budget) {
      report_timeout(status, KID_BARRIER, (unsigned)slot, (unsigned)i);
      return;
    }
  }
}

// out32[i] = sum_r grad_r[lo + i]; partial[blockIdx.x] = sum of squares of this block's outputs.
__global__ void reduce_scatter_kernel(PeerTable grads, int world, long long lo, long long n,
                                      float* __restrict__ out32, float* __restrict__ partial) {
  __shared__ float red[32];
  float ss = 0.f;
  const long long nvec = n >> 3;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec;
       t += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < world; ++r) {
      const uint4 u = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(grads.ptr[r]) + lo + t * 8);
      float2 f;
      f = unpack_bf16(u.x); acc[0] += f.x; acc[1] += f.y;
      f = unpack_bf16(u.y); acc[2] += f.x; acc[3] += f.y;
      f = unpack_bf16(u.z); acc[4] += f.x; acc[5] += f.y;
      f = unpack_bf16(u.w); acc[6] += f.x; acc[7] += f.y;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += acc[e] * acc[e];
    float4* o = reinterpret_cast<float4*>(out32 + t * 8);
    o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
  // block reduction of ss
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) red[w] = ss;
  __syncthreads();
  if (w == 0) {
    float t = l < nw ? red[l] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (l == 0) partial[blockIdx.x] = t;
  }
}

// One block.  Sums this rank's partials, publishes the total to every rank's norms[rank] (peer store),
// signals, waits for every peer's total, then writes scale[0] = grad_scale * clip coefficient and
// scale[1] = global gradient norm (of the rank-mean gradient).
__global__ void norm_exchange_kernel(const float* __restrict__ partial, int n_partial, PeerTable norms,
                                     PeerTable flags, int rank, int world, int slot, int epoch, float grad_scale,
                                     float max_norm, float* __restrict__ scale_out, long long budget,
                                     KernelStatus* status) {
  __shared__ float red[32];
  __shared__ float total_s;
  float s = 0.f;
  for (int i = threadIdx.x; i < n_partial; i += blockDim.x) s += partial[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) red[w] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < nw; ++i) t += red[i];
    total_s = t;
  }
  __syncthreads();
  if (threadIdx.x < world) {
    const int i = threadIdx.x;
    float* rn = static_cast<float*>(norms.ptr[i]) + rank;
    *reinterpret_cast<volatile float*>(rn) = total_s;
    __threadfence_system();
    st_release_sys(static_cast<int*>(flags.ptr[i]) + slot * MAX_RANKS + rank, epoch);
    const int* mine = static_cast<const int*>(flags.ptr[rank]) + slot * MAX_RANKS + i;
    const long long t0 = clock64();
    while (ld_acquire_sys(mine) < epoch) {
      if (clock64() - t0 > budget) {
        report_timeout(status, KID_NORMX, (unsigned)slot, (unsigned)i);
        break;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const volatile float* my_norms = static_cast<const volatile float*>(norms.ptr[rank]);
    float tot = 0.f;
    for (int i = 0; i < world; ++i) tot += my_norms[i];
    const float norm = sqrtf(tot) * grad_scale;
    const float coef = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
    scale_out[0] = grad_scale * coef;
    scale_out[1] = norm;
  }
}

// AdamW on the shard, then the new bf16 values are stored into every rank's parameter buffer.
__global__ void adamw_allgather_kernel(float* __restrict__ p32, const float* __restrict__ g32, float* __restrict__ m,
                                       float* __restrict__ v, PeerTable params, int world, long long lo, long long n,
                                       float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                                       const float* __restrict__ scale_ptr) {
  const float gs = scale_ptr[0];
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  const long long nvec = n >> 3;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec;
       t += (long long)gridDim.x * blockDim.x) {
    float pn[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const long long i = t * 8 + h * 4;
      float4 p4 = *reinterpret_cast<float4*>(p32 + i);
      const float4 g4 = *reinterpret_cast<const float4*>(g32 + i);
      float4 m4 = *reinterpret_cast<float4*>(m + i);
      float4 v4 = *reinterpret_cast<float4*>(v + i);
      float pp[4] = {p4.x, p4.y, p4.z, p4.w}, gg[4] = {g4.x, g4.y, g4.z, g4.w};
      float mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float gr = gg[e] * gs;
        float pe = pp[e] * (1.f - lr * wd);
        mm[e] = beta1 * mm[e] + (1.f - beta1) * gr;
        vv[e] = beta2 * vv[e] + (1.f - beta2) * gr * gr;
        pe -= lr * inv_bc1 * mm[e] / (sqrtf(vv[e]) * inv_sqrt_bc2 + eps);
        pp[e] = pe;
        pn[h * 4 + e] = pe;
      }
      *reinterpret_cast<float4*>(p32 + i) = make_float4(pp[0], pp[1], pp[2], pp[3]);
      *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    }
    uint4 o;
    o.x = pack_bf16(pn[0], pn[1]);
    o.y = pack_bf16(pn[2], pn[3]);
    o.z = pack_bf16(pn[4], pn[5]);
    o.w = pack_bf16(pn[6], pn[7]);
    for (int r = 0; r < world; ++r)
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(params.ptr[r]) + lo + t * 8) = o;
  }
}

}  // namespace otb

using namespace otb;

extern "C" int otb_comm_alloc(unsigned long long bytes, void** out) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*out, 0, bytes);
}
extern "C" int otb_comm_free(void* p) { return (int)cudaFree(p); }
extern "C" int otb_comm_get_handle(void* p, unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int otb_comm_open_handle(const unsigned char* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int otb_comm_close_handle(void* p) { return (int)cudaIpcCloseMemHandle(p); }

static PeerTable table_from(void* const* ptrs, int world) {
  PeerTable t;
  for (int i = 0; i < MAX_RANKS; ++i) t.ptr[i] = i < world ? ptrs[i] : nullptr;
  return t;
}

extern "C" int otb_comm_barrier(void* const* flag_ptrs, int rank, int world, int slot, int epoch, long long budget,
                                void* status, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS) return -1;
  barrier_kernel<<<1, 32, 0, stream>>>(table_from(flag_ptrs, world), rank, world, slot, epoch, budget,
                                       static_cast<KernelStatus*>(status));
  return (int)cudaGetLastError();
}

extern "C" int otb_comm_reduce_scatter(void* const* grad_ptrs, int world, long long lo, long long n, float* out32,
                                       float* partial, int nblocks, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || (n % 8) || (lo % 8)) return -1;
  reduce_scatter_kernel<<<nblocks, 512, 0, stream>>>(table_from(grad_ptrs, world), world, lo, n, out32, partial);
  return (int)cudaGetLastError();
}

extern "C" int otb_comm_norm_exchange(const float* partial, int n_partial, void* const* norm_ptrs,
                                      void* const* flag_ptrs, int rank, int world, int slot, int epoch,
                                      float grad_scale, float max_norm, float* scale_out, long long budget,
                                      void* status, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS) return -1;
  norm_exchange_kernel<<<1, 256, 0, stream>>>(partial, n_partial, table_from(norm_ptrs, world),
                                              table_from(flag_ptrs, world), rank, world, slot, epoch, grad_scale,
                                              max_norm, scale_out, budget, static_cast<KernelStatus*>(status));
  return (int)cudaGetLastError();
}

extern "C" int otb_comm_adamw_allgather(float* p32, const float* g32, float* m, float* v, void* const* param_ptrs,
                                        int world, long long lo, long long n, float lr, float beta1, float beta2,
                                        float eps, float wd, float bc1, float bc2, const float* scale_ptr,
                                        int nblocks, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || (n % 8) || (lo % 8)) return -1;
  adamw_allgather_kernel<<<nblocks, 512, 0, stream>>>(p32, g32, m, v, table_from(param_ptrs, world), world, lo, n, lr,
                                                      beta1, beta2, eps, wd, bc1, bc2, scale_ptr);
  return (int)cudaGetLastError();
}
