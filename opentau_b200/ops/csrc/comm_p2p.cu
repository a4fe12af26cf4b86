// Peer-memory communication runtime and the fused data-parallel step kernels.
//
// Every rank owns buffers allocated with cudaMalloc and exported through CUDA IPC; each rank maps all
// peers' buffers, so a kernel can read or write any rank's memory over NVLink / NVSwitch with plain
// loads and stores.  On top of that:
//
//   barrier           flag exchange with release/acquire at system scope
//   reduce_scatter    this rank's slice of one gradient bucket = sum over ranks (peer LOADS), bf16 / fp32 -> fp32,
//                     plus block partials of the squared norm; launched per bucket on a side stream as soon as the
//                     bucket's last weight-gradient product has been issued, so it runs under the rest of backward
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

// Eight consecutive elements of a bf16 / fp32 buffer as floats (16-byte loads).
template <typename T> __device__ __forceinline__ void load8(const T* p, float* f);
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 t;
  t = unpack_bf16(u.x); f[0] = t.x; f[1] = t.y;
  t = unpack_bf16(u.y); f[2] = t.x; f[3] = t.y;
  t = unpack_bf16(u.z); f[4] = t.x; f[5] = t.y;
  t = unpack_bf16(u.w); f[6] = t.x; f[7] = t.y;
}
template <> __device__ __forceinline__ void load8<float>(const float* p, float* f) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float* f);
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float* f) {
  uint4 o;
  o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]); o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = o;
}
template <> __device__ __forceinline__ void store8<float>(float* p, const float* f) {
  reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}

// One rank's 8 elements as they come off the wire: 16 bytes (bf16) stay packed in 4 registers until they are summed,
// so that a thread can keep eight ranks' loads in flight with 32 registers; fp32 pieces (8 registers) go 4 at a time.
template <typename T> struct Piece8;
template <> struct Piece8<__nv_bfloat16> {
  static constexpr int BATCH = 8;
  uint4 v;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void add_to(float* acc) const {
    float2 t;
    t = unpack_bf16(v.x); acc[0] += t.x; acc[1] += t.y;
    t = unpack_bf16(v.y); acc[2] += t.x; acc[3] += t.y;
    t = unpack_bf16(v.z); acc[4] += t.x; acc[5] += t.y;
    t = unpack_bf16(v.w); acc[6] += t.x; acc[7] += t.y;
  }
};
template <> struct Piece8<float> {
  static constexpr int BATCH = 4;
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = reinterpret_cast<const float4*>(p)[0];
    b = reinterpret_cast<const float4*>(p)[1];
  }
  __device__ __forceinline__ void add_to(float* acc) const {
    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
    acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
  }
};

// acc[0..8) = sum over ranks (in rank order) of the 8 elements at `offset` of every rank's buffer.  The loads of a
// batch of ranks are all issued before the first is consumed.
template <typename T>
__device__ __forceinline__ void sum_ranks8(const PeerTable& bufs, int world, long long offset, float* acc) {
  constexpr int G = Piece8<T>::BATCH;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
  for (int r0 = 0; r0 < MAX_RANKS; r0 += G) {
    if (r0 < world) {                                      // uniform over the grid
      Piece8<T> piece[G];
#pragma unroll
      for (int g = 0; g < G; ++g)
        if (r0 + g < world) piece[g].load(static_cast<const T*>(bufs.ptr[r0 + g]) + offset);
#pragma unroll
      for (int g = 0; g < G; ++g)
        if (r0 + g < world) piece[g].add_to(acc);
    }
  }
}

// out32[i] = sum_r grad_r[lo + i]; partial[blockIdx.x] = sum of squares of this block's outputs.
// A wait that gave up earlier in this step left a record in `status`: the peers' buffers cannot be trusted then, so
// the kernel writes nothing (the optimizer kernel behind it does the same and the parameters stay as they were).
// Two 512-thread blocks per SM (at most 64 registers): the loads in flight per SM are what hides the latency of peer
// reads, and they are the product of resident threads and loads per thread.
template <typename T>
__global__ void __launch_bounds__(512, 2) reduce_scatter_kernel(PeerTable grads, int world, long long lo, long long n,
                                                                float* __restrict__ out32, float* __restrict__ partial,
                                                                const KernelStatus* status) {
  __shared__ float red[32];
  if (status != nullptr && *reinterpret_cast<const volatile unsigned*>(&status->code) != 0u) return;
  float ss = 0.f;
  const long long nvec = n >> 3;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec;
       t += (long long)gridDim.x * blockDim.x) {
    float acc[8];
    sum_ranks8<T>(grads, world, lo + t * 8, acc);
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

// out[r * n + i] = src_r[i]: all-gather of every rank's n-element (16-byte multiple) buffer by peer LOADS, in rank
// order.  Writes nothing when a wait gave up earlier (the buffers it would read cannot be trusted).
__global__ void allgather_pull_kernel(PeerTable src, int world, long long n_vec16, uint4* __restrict__ out,
                                      const KernelStatus* status) {
  if (status != nullptr && *reinterpret_cast<const volatile unsigned*>(&status->code) != 0u) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int r = 0; r < world; ++r) {
    const uint4* s = static_cast<const uint4*>(src.ptr[r]);
    uint4* o = out + (long long)r * n_vec16;
    long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    // four independent 16-byte peer loads in flight per thread: with one, a grid of 64 K threads keeps 1 MB on the
    // link, about half of what its bandwidth-delay product needs
    for (; t + 3 * stride < n_vec16; t += 4 * stride) {
      const uint4 a = s[t], b = s[t + stride], c = s[t + 2 * stride], d = s[t + 3 * stride];
      o[t] = a;
      o[t + stride] = b;
      o[t + 2 * stride] = c;
      o[t + 3 * stride] = d;
    }
    for (; t < n_vec16; t += stride) o[t] = s[t];
  }
}

// out[i] = sum_r src_r[lo + i] for bf16 buffers, summed in fp32 in rank order, stored as bf16: the reduce-scatter of
// partial results (context-parallel dK / dV) back to the rank that owns the slice.
__global__ void __launch_bounds__(512, 2) reduce_scatter_bf16_kernel(PeerTable src, int world, long long lo, long long n,
                                                                     __nv_bfloat16* __restrict__ out,
                                                                     const KernelStatus* status) {
  if (status != nullptr && *reinterpret_cast<const volatile unsigned*>(&status->code) != 0u) return;
  const long long nvec = n >> 3;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec;
       t += (long long)gridDim.x * blockDim.x) {
    float acc[8];
    sum_ranks8<__nv_bfloat16>(src, world, lo + t * 8, acc);
    store8<__nv_bfloat16>(out + t * 8, acc);
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
  // a wait already gave up in this step: do not start another full-length wait on the same peers
  if (status != nullptr && *reinterpret_cast<const volatile unsigned*>(&status->code) != 0u) return;
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

// AdamW on the shard, then the new values are stored (in the parameters' own dtype) into every rank's parameter
// buffer.  Writes nothing when a wait gave up earlier in this step (see reduce_scatter_kernel).
template <typename T>
__global__ void __launch_bounds__(512, 2) adamw_allgather_kernel(
    float* __restrict__ p32, const float* __restrict__ g32, float* __restrict__ m, float* __restrict__ v,
    PeerTable params, int world, long long lo, long long n, float lr, float beta1, float beta2, float eps, float wd,
    float bc1, float bc2, const float* __restrict__ scale_ptr, const KernelStatus* status) {
  if (status != nullptr && *reinterpret_cast<const volatile unsigned*>(&status->code) != 0u) return;
  const float gs = scale_ptr[0];
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  const float decay = 1.f - lr * wd, c1 = 1.f - beta1, c2 = 1.f - beta2;
  const long long nvec = n >> 3;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec;
       t += (long long)gridDim.x * blockDim.x) {
    const long long i = t * 8;
    // the eight 16-byte loads of this vector are requested before any is used
    float4 p4[2], g4[2], m4[2], v4[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      p4[h] = *reinterpret_cast<const float4*>(p32 + i + h * 4);
      g4[h] = *reinterpret_cast<const float4*>(g32 + i + h * 4);
      m4[h] = *reinterpret_cast<const float4*>(m + i + h * 4);
      v4[h] = *reinterpret_cast<const float4*>(v + i + h * 4);
    }
    float pn[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float pp[4] = {p4[h].x, p4[h].y, p4[h].z, p4[h].w}, gg[4] = {g4[h].x, g4[h].y, g4[h].z, g4[h].w};
      float mm[4] = {m4[h].x, m4[h].y, m4[h].z, m4[h].w}, vv[4] = {v4[h].x, v4[h].y, v4[h].z, v4[h].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float gr = gg[e] * gs;
        float pe = pp[e] * decay;
        mm[e] = beta1 * mm[e] + c1 * gr;
        vv[e] = beta2 * vv[e] + c2 * gr * gr;
        pe -= lr * inv_bc1 * mm[e] / (sqrtf(vv[e]) * inv_sqrt_bc2 + eps);
        pp[e] = pe;
        pn[h * 4 + e] = pe;
      }
      *reinterpret_cast<float4*>(p32 + i + h * 4) = make_float4(pp[0], pp[1], pp[2], pp[3]);
      *reinterpret_cast<float4*>(m + i + h * 4) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(v + i + h * 4) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    }
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r)
      if (r < world) store8<T>(static_cast<T*>(params.ptr[r]) + lo + i, pn);
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

// elem_bytes: 2 = bf16 gradients, 4 = fp32 gradients.
extern "C" int otb_comm_reduce_scatter(void* const* grad_ptrs, int world, long long lo, long long n, float* out32,
                                       float* partial, int nblocks, int elem_bytes, void* status,
                                       cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || (n % 8) || (lo % 8) || nblocks < 1) return -1;
  const KernelStatus* st = static_cast<const KernelStatus*>(status);
  if (elem_bytes == 2)
    reduce_scatter_kernel<__nv_bfloat16><<<nblocks, 512, 0, stream>>>(table_from(grad_ptrs, world), world, lo, n,
                                                                       out32, partial, st);
  else if (elem_bytes == 4)
    reduce_scatter_kernel<float><<<nblocks, 512, 0, stream>>>(table_from(grad_ptrs, world), world, lo, n, out32,
                                                               partial, st);
  else
    return -1;
  return (int)cudaGetLastError();
}

// src_ptrs[r]: rank r's buffer of `bytes` bytes (multiple of 16); out: world * bytes bytes, local.
extern "C" int otb_comm_allgather_pull(void* const* src_ptrs, int world, long long bytes, void* out, int nblocks,
                                       void* status, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || (bytes % 16) || nblocks < 1) return -1;
  allgather_pull_kernel<<<nblocks, 512, 0, stream>>>(table_from(src_ptrs, world), world, bytes / 16,
                                                     static_cast<uint4*>(out),
                                                     static_cast<const KernelStatus*>(status));
  return (int)cudaGetLastError();
}

extern "C" int otb_comm_reduce_scatter_bf16(void* const* src_ptrs, int world, long long lo, long long n, void* out,
                                            int nblocks, void* status, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || (n % 8) || (lo % 8) || nblocks < 1) return -1;
  reduce_scatter_bf16_kernel<<<nblocks, 512, 0, stream>>>(table_from(src_ptrs, world), world, lo, n,
                                                          static_cast<__nv_bfloat16*>(out),
                                                          static_cast<const KernelStatus*>(status));
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
                                        int nblocks, int elem_bytes, void* status, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || (n % 8) || (lo % 8) || nblocks < 1) return -1;
  const KernelStatus* st = static_cast<const KernelStatus*>(status);
  if (elem_bytes == 2)
    adamw_allgather_kernel<__nv_bfloat16><<<nblocks, 512, 0, stream>>>(p32, g32, m, v, table_from(param_ptrs, world),
                                                                        world, lo, n, lr, beta1, beta2, eps, wd, bc1,
                                                                        bc2, scale_ptr, st);
  else if (elem_bytes == 4)
    adamw_allgather_kernel<float><<<nblocks, 512, 0, stream>>>(p32, g32, m, v, table_from(param_ptrs, world), world,
                                                                lo, n, lr, beta1, beta2, eps, wd, bc1, bc2, scale_ptr,
                                                                st);
  else
    return -1;
  return (int)cudaGetLastError();
}
