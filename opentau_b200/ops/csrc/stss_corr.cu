// Space-time self-similarity: local inner products between every patch feature and the features inside an
// (L frames) x (k x k patches) window around it, straight from the token-major feature matrix.
//
//   out[b, t, p, l, u, v] = < x[b, t, p, :],  x[b, tt(t, l), p + (u - k/2, v - k/2), : ] >      (0 outside the image)
//   tt(t, l) = clamp(t + l - L/2, 0, T - 1) for L > 1;  max(t - 1, 0) for L == 1
//
// The dense formulation (unfold the zero-padded target frame, expand the source over L, einsum) materialises
// L * k * k copies of the features; here a warp owns one (b, t, p, l) and reads the k * k neighbour vectors from L2.
// Features are read in 16-byte chunks (chunk c of a row belongs to lane c % 32), products accumulate in fp32.
//
// Backward, gather form (no atomics, fixed order): the gradient of x[b, t, p, :] collects
//   (as a source)  sum_{l, uv}  g[b, t, p, l, uv]        * x[b, tt(t, l), p + uv, :]
//   (as a target)  sum_{t', l : tt(t', l) = t} sum_uv  g[b, t', p - uv, l, uv] * x[b, t', p - uv, :]
// with one warp per (b, t, p).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace otb {

constexpr int STSS_MAX_CHUNKS = 8;   // 16-byte chunks per lane: C <= 2048 (bf16) / 1024 (fp32)

template <typename T>
struct Chunk;
template <>
struct Chunk<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float f[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(h[i]);
      f[2 * i] = x.x;
      f[2 * i + 1] = x.y;
    }
  }
  __device__ static void store(__nv_bfloat16* p, const float f[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
  __device__ static float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
  __device__ static __nv_bfloat16 from_float(float x) { return __float2bfloat16(x); }
};
template <>
struct Chunk<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float f[4]) {
    const float4 u = *reinterpret_cast<const float4*>(p);
    f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
  }
  __device__ static void store(float* p, const float f[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
  __device__ static float to_float(float x) { return x; }
  __device__ static float from_float(float x) { return x; }
};

__device__ __forceinline__ int stss_target_frame(int t, int l, int L, int T) {
  if (L > 1) {
    const int tt = t + l - L / 2;
    return tt < 0 ? 0 : (tt > T - 1 ? T - 1 : tt);
  }
  return t > 0 ? t - 1 : 0;
}

__device__ __forceinline__ float stss_warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

template <typename T>
__global__ void __launch_bounds__(256) stss_corr_fwd_kernel(const T* __restrict__ x, T* __restrict__ out, int B, int Tn,
                                                            int H, int W, int C, int L, int k) {
  using CH = Chunk<T>;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * Tn * H * W * L;
  if (warp >= total) return;
  const int l = int(warp % L);
  long long r = warp / L;
  const int pw = int(r % W); r /= W;
  const int ph = int(r % H); r /= H;
  const int t = int(r % Tn);
  const int b = int(r / Tn);
  const int HW = H * W, kk = k * k, d = k / 2;
  const int nch = C / CH::N;
  const T* src = x + (((long long)b * Tn + t) * HW + ph * W + pw) * C;
  const T* tgt = x + ((long long)b * Tn + stss_target_frame(t, l, L, Tn)) * HW * C;
  float s[STSS_MAX_CHUNKS][CH::N];
#pragma unroll
  for (int i = 0; i < STSS_MAX_CHUNKS; ++i) {
    const int c = lane + 32 * i;
    if (c < nch) CH::load(src + c * CH::N, s[i]);
  }
  T* orow = out + warp * kk;
  for (int base = 0; base < kk; base += 32) {
    float mine = 0.f;
    for (int j = 0; j < 32 && base + j < kk; ++j) {
      const int uv = base + j;
      const int hh = ph + uv / k - d, ww = pw + uv % k - d;
      float acc = 0.f;
      if (hh >= 0 && hh < H && ww >= 0 && ww < W) {          // uniform over the warp
        const T* nb = tgt + (long long)(hh * W + ww) * C;
#pragma unroll
        for (int i = 0; i < STSS_MAX_CHUNKS; ++i) {
          const int c = lane + 32 * i;
          if (c < nch) {
            float f[CH::N];
            CH::load(nb + c * CH::N, f);
#pragma unroll
            for (int e = 0; e < CH::N; ++e) acc = fmaf(s[i][e], f[e], acc);
          }
        }
        acc = stss_warp_sum(acc);
      }
      if (lane == j) mine = acc;
    }
    if (base + lane < kk) orow[base + lane] = CH::from_float(mine);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) stss_corr_bwd_kernel(const T* __restrict__ x, const T* __restrict__ g,
                                                            T* __restrict__ dx, int B, int Tn, int H, int W, int C,
                                                            int L, int k) {
  using CH = Chunk<T>;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * Tn * H * W;
  if (warp >= total) return;
  long long r = warp;
  const int pw = int(r % W); r /= W;
  const int ph = int(r % H); r /= H;
  const int t = int(r % Tn);
  const int b = int(r / Tn);
  const int HW = H * W, kk = k * k, d = k / 2;
  const int nch = C / CH::N;
  float acc[STSS_MAX_CHUNKS][CH::N];
#pragma unroll
  for (int i = 0; i < STSS_MAX_CHUNKS; ++i)
#pragma unroll
    for (int e = 0; e < CH::N; ++e) acc[i][e] = 0.f;
  const T* xb = x + (long long)b * Tn * HW * C;
  const T* gb = g + (long long)b * Tn * HW * L * kk;

  auto add = [&](float gv, const T* vec) {
#pragma unroll
    for (int i = 0; i < STSS_MAX_CHUNKS; ++i) {
      const int c = lane + 32 * i;
      if (c < nch) {
        float f[CH::N];
        CH::load(vec + c * CH::N, f);
#pragma unroll
        for (int e = 0; e < CH::N; ++e) acc[i][e] = fmaf(gv, f[e], acc[i][e]);
      }
    }
  };

  // as a source: this position's own rows of g, neighbours of the target frames
  for (int l = 0; l < L; ++l) {
    const T* tgt = xb + (long long)stss_target_frame(t, l, L, Tn) * HW * C;
    const T* grow = gb + (((long long)t * HW + ph * W + pw) * L + l) * kk;
    for (int uv = 0; uv < kk; ++uv) {
      const int hh = ph + uv / k - d, ww = pw + uv % k - d;
      if (hh < 0 || hh >= H || ww < 0 || ww >= W) continue;
      add(CH::to_float(grow[uv]), tgt + (long long)(hh * W + ww) * C);
    }
  }
  // as a target: every (source frame t', offset l) that points at this frame, every source position that reaches here
  for (int ts = 0; ts < Tn; ++ts) {
    for (int l = 0; l < L; ++l) {
      if (stss_target_frame(ts, l, L, Tn) != t) continue;
      for (int uv = 0; uv < kk; ++uv) {
        const int hs = ph - (uv / k - d), ws = pw - (uv % k - d);
        if (hs < 0 || hs >= H || ws < 0 || ws >= W) continue;
        const long long sp = (long long)ts * HW + hs * W + ws;
        add(CH::to_float(gb[(sp * L + l) * kk + uv]), xb + sp * C);
      }
    }
  }
  T* drow = dx + warp * C;
#pragma unroll
  for (int i = 0; i < STSS_MAX_CHUNKS; ++i) {
    const int c = lane + 32 * i;
    if (c < nch) CH::store(drow + c * CH::N, acc[i]);
  }
}

}  // namespace otb

using namespace otb;

static int stss_check(int B, int T, int H, int W, int C, int L, int k, int elem_bytes, const void* a, const void* b2) {
  if (B <= 0 || T <= 0 || H <= 0 || W <= 0 || C <= 0 || L <= 0 || k <= 0 || (L & 1) == 0 || (k & 1) == 0) return -2;
  const int per = 16 / elem_bytes;
  if (C % per || C / per > 32 * STSS_MAX_CHUNKS) return -3;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b2)) & 15) return -4;
  return 0;
}

// x: (B, T, H*W, C) contiguous, bf16 (elem_bytes 2) or fp32 (4); out: (B, T, H*W, L, k*k) of the same type.
extern "C" int otb_stss_corr_fwd(const void* x, void* out, int B, int T, int H, int W, int C, int L, int k,
                                 int elem_bytes, cudaStream_t stream) {
  int r = stss_check(B, T, H, W, C, L, k, elem_bytes, x, x);
  if (r) return r;
  const long long warps = (long long)B * T * H * W * L;
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  if (elem_bytes == 2)
    stss_corr_fwd_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                                    static_cast<__nv_bfloat16*>(out), B, T, H, W, C, L, k);
  else if (elem_bytes == 4)
    stss_corr_fwd_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<float*>(out), B,
                                                            T, H, W, C, L, k);
  else
    return -5;
  return (int)cudaGetLastError();
}

// g: gradient of out, same shape and type; dx: (B, T, H*W, C).
extern "C" int otb_stss_corr_bwd(const void* x, const void* g, void* dx, int B, int T, int H, int W, int C, int L,
                                 int k, int elem_bytes, cudaStream_t stream) {
  int r = stss_check(B, T, H, W, C, L, k, elem_bytes, x, dx);
  if (r) return r;
  const long long warps = (long long)B * T * H * W;
  const unsigned blocks = (unsigned)((warps + 7) / 8);
  if (elem_bytes == 2)
    stss_corr_bwd_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(g), static_cast<__nv_bfloat16*>(dx), B, T,
        H, W, C, L, k);
  else if (elem_bytes == 4)
    stss_corr_bwd_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<const float*>(g),
                                                            static_cast<float*>(dx), B, T, H, W, C, L, k);
  else
    return -5;
  return (int)cudaGetLastError();
}
