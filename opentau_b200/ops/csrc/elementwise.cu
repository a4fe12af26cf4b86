// Memory-bound kernels: norms, gated activations, rotary embedding, losses, optimizer, image resize.
// All take bf16 activations with fp32 math; every kernel is a single pass over its inputs with
// 16-byte vector accesses so that the achieved DRAM bandwidth is the figure of merit.
#include "common.cuh"

namespace otb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum for up to 1024 threads; `red` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < nw) ? red[l] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < nw) ? red[l] : -INFINITY;
  t = warp_max(t);
  return t;
}

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 f;
  f = unpack_bf16(u.x); v[0] = f.x; v[1] = f.y;
  f = unpack_bf16(u.y); v[2] = f.x; v[3] = f.y;
  f = unpack_bf16(u.z); v[4] = f.x; v[5] = f.y;
  f = unpack_bf16(u.w); v[6] = f.x; v[7] = f.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* v) {
  uint4 o;
  o.x = pack_bf16(v[0], v[1]);
  o.y = pack_bf16(v[2], v[3]);
  o.z = pack_bf16(v[4], v[5]);
  o.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

// ------------------------------------------------------------------------------------------ RMSNorm
// One block per row.  mode: 0 = no weight, 1 = (1 + w), 2 = w.
// Adaptive form: y = xhat * (1 + scale) + shift with scale/shift rows taken from `mod`
// (row stride mod_stride, one mod row per `rows_per_mod` consecutive rows).
template <int MAXV>
__global__ void rms_fwd_kernel(const __nv_bfloat16* __restrict__ x, long long x_stride,
                               const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ mod,
                               long long mod_stride, int rows_per_mod, __nv_bfloat16* __restrict__ y,
                               float* __restrict__ rstd_out, int H, float eps, int mode) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * x_stride;
  float v[MAXV][8];
  float ss = 0.f;
  const int nvec = H >> 3;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
      load8(xr + idx * 8, v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
  const __nv_bfloat16* mrow = mod ? mod + (row / rows_per_mod) * mod_stride : nullptr;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
      float o[8];
      if (mrow) {
        float sc[8], sh[8];
        load8(mrow + idx * 8, sc);
        load8(mrow + H + idx * 8, sh);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[i][e] * rstd * (1.f + sc[e]) + sh[e];
      } else if (mode != 0) {
        float wf[8];
        load8(w + idx * 8, wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[i][e] * rstd * (mode == 1 ? 1.f + wf[e] : wf[e]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[i][e] * rstd;
      }
      store8(y + row * (long long)H + idx * 8, o);
    }
  }
}

// Backward.  dx = (g - xhat * mean(g * xhat)) * rstd with g = dy * wf (wf = 1+w | w | 1+scale | 1).
// Weight-gradient partials: each block owns `rows_per_block` rows and writes one fp32 row of
// dw_partial[gridDim.x][H] (no atomics; a second kernel sums the partials in a fixed order).
// Adaptive form additionally writes dscale = dy * xhat and dshift = dy per token.
template <int MAXV>
__global__ void rms_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                               long long x_stride, const __nv_bfloat16* __restrict__ w,
                               const __nv_bfloat16* __restrict__ mod, long long mod_stride, int rows_per_mod,
                               const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                               float* __restrict__ dw_partial, __nv_bfloat16* __restrict__ dscale,
                               __nv_bfloat16* __restrict__ dshift, const __nv_bfloat16* __restrict__ dres,
                               long long rows, int H, int mode, int rows_per_block) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  float dwacc[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[i][e] = 0.f;
  const long long r0 = (long long)blockIdx.x * rows_per_block;
  for (long long row = r0; row < min(r0 + (long long)rows_per_block, rows); ++row) {
    const float rstd = rstd_in[row];
    const __nv_bfloat16* xr = x + row * x_stride;
    const __nv_bfloat16* dyr = dy + row * (long long)H;
    const __nv_bfloat16* mrow = mod ? mod + (row / rows_per_mod) * mod_stride : nullptr;
    float g[MAXV][8], xh[MAXV][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      int idx = threadIdx.x + i * blockDim.x;
      if (idx < nvec) {
        float xv[8], dv[8], wf[8];
        load8(xr + idx * 8, xv);
        load8(dyr + idx * 8, dv);
        if (mrow) {
          load8(mrow + idx * 8, wf);
#pragma unroll
          for (int e = 0; e < 8; ++e) wf[e] += 1.f;
        } else if (mode != 0) {
          load8(w + idx * 8, wf);
          if (mode == 1) {
#pragma unroll
            for (int e = 0; e < 8; ++e) wf[e] += 1.f;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) wf[e] = 1.f;
        }
        float ds[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[i][e] = xv[e] * rstd;
          g[i][e] = dv[e] * wf[e];
          dot += g[i][e] * xh[i][e];
          ds[e] = dv[e] * xh[i][e];
          dwacc[i][e] += ds[e];
        }
        if (dscale) {
          store8(dscale + row * (long long)H + idx * 8, ds);
          store8(dshift + row * (long long)H + idx * 8, dv);
        }
      }
    }
    dot = block_sum(dot, red) / H;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      int idx = threadIdx.x + i * blockDim.x;
      if (idx < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (g[i][e] - xh[i][e] * dot) * rstd;
        if (dres) {   // the gradient that reached x through the residual branch: summed here, not by a separate add
          float rr[8];
          load8(dres + row * (long long)H + idx * 8, rr);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += rr[e];
        }
        store8(dx + row * (long long)H + idx * 8, o);
      }
    }
  }
  if (dw_partial) {
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      int idx = threadIdx.x + i * blockDim.x;
      if (idx < nvec) {
        float* o = dw_partial + (long long)blockIdx.x * H + idx * 8;
        *reinterpret_cast<float4*>(o) = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
        *reinterpret_cast<float4*>(o + 4) = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
      }
    }
  }
}

// LayerNorm backward.  xhat = (x - mean) * rstd, g = dy * w:
//   dx = (g - mean(g) - xhat * mean(g * xhat)) * rstd,   dw = sum_rows dy * xhat,   db = sum_rows dy.
// Same work split as rms_bwd_kernel: a block owns `rows_per_block` consecutive rows and writes one fp32 row of
// dw_partial[gridDim.x][H] and of db_partial[gridDim.x][H]; colsum_partials_kernel adds them up in a fixed order.
template <int MAXV>
__global__ void ln_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                              const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                              const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                              float* __restrict__ dw_partial, float* __restrict__ db_partial, long long rows, int H,
                              int rows_per_block) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  float dwacc[MAXV][8], dbacc[MAXV][8], wf[MAXV][8];
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[i][e] = dbacc[i][e] = wf[i][e] = 0.f;
    if (idx < nvec) load8(w + idx * 8, wf[i]);
  }
  const long long r0 = (long long)blockIdx.x * rows_per_block;
  for (long long row = r0; row < min(r0 + (long long)rows_per_block, rows); ++row) {
    const float mu = mean_in[row], rstd = rstd_in[row];
    const __nv_bfloat16* xr = x + row * (long long)H;
    const __nv_bfloat16* dyr = dy + row * (long long)H;
    float g[MAXV][8], xh[MAXV][8];
    float sum_g = 0.f, sum_gx = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (idx < nvec) {
        float xv[8], dv[8];
        load8(xr + idx * 8, xv);
        load8(dyr + idx * 8, dv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[i][e] = (xv[e] - mu) * rstd;
          g[i][e] = dv[e] * wf[i][e];
          sum_g += g[i][e];
          sum_gx += g[i][e] * xh[i][e];
          dwacc[i][e] += dv[e] * xh[i][e];
          dbacc[i][e] += dv[e];
        }
      }
    }
    const float m1 = block_sum(sum_g, red) / H;
    const float m2 = block_sum(sum_gx, red) / H;
#pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      if (idx < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (g[i][e] - m1 - xh[i][e] * m2) * rstd;
        store8(dx + row * (long long)H + idx * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
      float* ow = dw_partial + (long long)blockIdx.x * H + idx * 8;
      float* ob = db_partial + (long long)blockIdx.x * H + idx * 8;
      *reinterpret_cast<float4*>(ow) = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
      *reinterpret_cast<float4*>(ow + 4) = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
      *reinterpret_cast<float4*>(ob) = make_float4(dbacc[i][0], dbacc[i][1], dbacc[i][2], dbacc[i][3]);
      *reinterpret_cast<float4*>(ob + 4) = make_float4(dbacc[i][4], dbacc[i][5], dbacc[i][6], dbacc[i][7]);
    }
  }
}

// out[c] = sum_r partial[r][c]  (fixed order -> deterministic), cast to bf16; optionally += into out.
__global__ void colsum_partials_kernel(const float* __restrict__ partial, int nrows, int H,
                                       __nv_bfloat16* __restrict__ out, int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int r = 0; r < nrows; ++r) s += partial[(long long)r * H + c];
  if (accumulate) s += __bfloat162float(out[c]);
  out[c] = __float2bfloat16(s);
}

// Column sums of a bf16 [rows, H] matrix into fp32 partials [gridDim.y][H] (bias gradients).
__global__ void colsum_bf16_kernel(const __nv_bfloat16* __restrict__ a, long long rows, int H, long long lda,
                                   float* __restrict__ partial, int rows_per_block) {
  int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= H) return;
  long long r0 = (long long)blockIdx.y * rows_per_block;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (long long r = r0; r < min(r0 + (long long)rows_per_block, rows); ++r) {
    float v[8];
    load8(a + r * lda + c, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += v[e];
  }
  float* o = partial + (long long)blockIdx.y * H + c;
#pragma unroll
  for (int e = 0; e < 8; ++e) o[e] = acc[e];
}

// ------------------------------------------------------------------------------------------ LayerNorm
template <int MAXV>
__global__ void ln_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                              const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y,
                              float* __restrict__ mean_out, float* __restrict__ rstd_out, int H, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * (long long)H;
  float v[MAXV][8];
  float s = 0.f;
  const int nvec = H >> 3;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
      load8(xr + idx * 8, v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) s += v[i][e];
    }
  }
  const float mean = block_sum(s, red) / H;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float d = v[i][e] - mean;
        ss += d * d;
      }
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / H + eps);
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    int idx = threadIdx.x + i * blockDim.x;
    if (idx < nvec) {
      float wf[8], bf[8], o[8];
      load8(w + idx * 8, wf);
      load8(b + idx * 8, bf);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[i][e] - mean) * rstd * wf[e] + bf[e];
      store8(y + row * (long long)H + idx * 8, o);
    }
  }
}

// ------------------------------------------------------------------------------------------ GLU
// gu[M][2I] with 32-wide alternating gate/up blocks -> h[M][I].  act: 0 gelu_tanh, 1 silu.
__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h, long long M,
                               int I, int act) {
  const long long nvec = M * (long long)(I >> 3);
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec;
       t += (long long)gridDim.x * blockDim.x) {
    const long long row = t / (I >> 3);
    const int c = int(t - row * (I >> 3)) * 8;       // output column
    const int blk = c >> 5, off = c & 31;
    const __nv_bfloat16* g = gu + row * (2LL * I) + blk * 64 + off;
    float gv[8], uv[8], o[8];
    load8(g, gv);
    load8(g + 32, uv);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = (act == 0 ? gelu_tanh_f(gv[e]) : silu_f(gv[e])) * uv[e];
    store8(h + row * (long long)I + c, o);
  }
}

__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                               __nv_bfloat16* __restrict__ dgu, long long M, int I, int act) {
  const long long nvec = M * (long long)(I >> 3);
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec;
       t += (long long)gridDim.x * blockDim.x) {
    const long long row = t / (I >> 3);
    const int c = int(t - row * (I >> 3)) * 8;
    const int blk = c >> 5, off = c & 31;
    const long long base = row * (2LL * I) + blk * 64 + off;
    float gv[8], uv[8], dv[8], dg[8], du[8];
    load8(gu + base, gv);
    load8(gu + base + 32, uv);
    load8(dh + row * (long long)I + c, dv);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float x = gv[e], a, da;
      if (act == 0) {
        // s = sigmoid(2u) = 0.5 (1 + tanh u); 1 - tanh^2 u = 4 s (1 - s)
        const float k = 0.7978845608028654f;
        const float inner = k * (x + 0.044715f * x * x * x);
        const float s = __fdividef(1.f, 1.f + __expf(-2.f * inner));
        a = x * s;
        da = s + 2.f * x * s * (1.f - s) * k * (1.f + 3.f * 0.044715f * x * x);
      } else {
        float s = 1.f / (1.f + __expf(-x));
        a = x * s;
        da = s * (1.f + x * (1.f - s));
      }
      dg[e] = dv[e] * uv[e] * da;
      du[e] = dv[e] * a;
    }
    store8(dgu + base, dg);
    store8(dgu + base + 32, du);
  }
}

// ------------------------------------------------------------------------------------------ RoPE
// x: (B,S,H,D) with element strides (sb, ss, sh, 1); cos/sin: (B,S,D/2) fp32; y contiguous (B,S,H,D).
// Split-half rotation; inverse rotates by the negative angle.
// V = pairs per thread: 8 (16-byte accesses, head_dim % 16 == 0) or 4 (8-byte accesses, head_dim % 8 == 0, e.g. the
// 72-wide heads of the Qwen3-VL vision tower)
template <int V>
__device__ __forceinline__ void load_v(const __nv_bfloat16* p, float* v) {
  if constexpr (V == 8) {
    load8(p, v);
  } else {
    uint2 u = *reinterpret_cast<const uint2*>(p);
    float2 f;
    f = unpack_bf16(u.x); v[0] = f.x; v[1] = f.y;
    f = unpack_bf16(u.y); v[2] = f.x; v[3] = f.y;
  }
}
template <int V>
__device__ __forceinline__ void store_v(__nv_bfloat16* p, const float* v) {
  if constexpr (V == 8) {
    store8(p, v);
  } else {
    uint2 o;
    o.x = pack_bf16(v[0], v[1]);
    o.y = pack_bf16(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = o;
  }
}

template <int V>
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, long long sb, long long ss, long long sh,
                            const float* __restrict__ cosb, const float* __restrict__ sinb,
                            __nv_bfloat16* __restrict__ y, int B, int S, int H, int D, int inverse) {
  const int half = D >> 1;
  const int vec_per_head = half / V;             // V pairs per thread
  const long long total = (long long)B * S * H * vec_per_head;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    int v = int(t % vec_per_head);
    long long r = t / vec_per_head;
    int h = int(r % H);
    r /= H;
    int s = int(r % S);
    int b = int(r / S);
    const __nv_bfloat16* xp = x + b * sb + s * ss + h * sh + v * V;
    float x1[V], x2[V], o1[V], o2[V];
    load_v<V>(xp, x1);
    load_v<V>(xp + half, x2);
    const float* cp = cosb + ((long long)b * S + s) * half + v * V;
    const float* sp = sinb + ((long long)b * S + s) * half + v * V;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      float c = cp[e], sn = inverse ? -sp[e] : sp[e];
      o1[e] = x1[e] * c - x2[e] * sn;
      o2[e] = x2[e] * c + x1[e] * sn;
    }
    __nv_bfloat16* yp = y + (((long long)b * S + s) * H + h) * D + v * V;
    store_v<V>(yp, o1);
    store_v<V>(yp + half, o2);
  }
}

// ------------------------------------------------------------------------------------------ inference fusions
// After the fused q/k/v projection of ONE tower (no autograd): per (token, head) split the row, RMS-normalise q and
// k heads (Qwen3 / Gemma-3 qk-norm; optional), rotate q and k, and write q densely and k / v through strides, so
// that new keys and values can land directly behind the cached prefix.  One warp per (token, head slot).
__global__ void qkv_post_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld, const __nv_bfloat16* __restrict__ qw,
                                const __nv_bfloat16* __restrict__ kw, float eps, int unit_offset,
                                const float* __restrict__ cosb, const float* __restrict__ sinb,
                                __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out, long long k_sb,
                                long long k_ss, __nv_bfloat16* __restrict__ v_out, long long v_sb, long long v_ss, int B,
                                int T, int H, int Hkv, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const int slots = H + 2 * Hkv;
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (long long)B * T * slots) return;
  const int slot = int(wid % slots);
  const long long tok = wid / slots;
  const int t = int(tok % T), b = int(tok / T);
  const __nv_bfloat16* src = qkv + tok * ld + (long long)slot * D;
  const int half = D >> 1;
  const int kind = slot < H ? 0 : (slot < H + Hkv ? 1 : 2);   // q | k | v
  __nv_bfloat16* dst;
  if (kind == 0) dst = q_out + (tok * H + slot) * D;
  else if (kind == 1) dst = k_out + b * k_sb + t * k_ss + (long long)(slot - H) * D;
  else dst = v_out + b * v_sb + t * v_ss + (long long)(slot - H - Hkv) * D;
  if (kind == 2) {
    for (int i = lane; i < D; i += 32) dst[i] = src[i];
    return;
  }
  float x1[4], x2[4];                                          // D <= 256: at most 4 pairs per lane
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = lane + 32 * j;
    x1[j] = i < half ? __bfloat162float(src[i]) : 0.f;
    x2[j] = i < half ? __bfloat162float(src[i + half]) : 0.f;
    ss += x1[j] * x1[j] + x2[j] * x2[j];
  }
  const __nv_bfloat16* w = kind == 0 ? qw : kw;
  if (w != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / D + eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = lane + 32 * j;
      if (i < half) {
        const float w1 = __bfloat162float(w[i]) + (unit_offset ? 1.f : 0.f);
        const float w2 = __bfloat162float(w[i + half]) + (unit_offset ? 1.f : 0.f);
        // the unfused path stores the normalised head in bf16 before rotating it
        x1[j] = __bfloat162float(__float2bfloat16(x1[j] * rstd * w1));
        x2[j] = __bfloat162float(__float2bfloat16(x2[j] * rstd * w2));
      }
    }
  }
  const float* cp = cosb + tok * half;
  const float* sp = sinb + tok * half;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = lane + 32 * j;
    if (i < half) {
      const float c = cp[i], sn = sp[i];
      dst[i] = __float2bfloat16(x1[j] * c - x2[j] * sn);
      dst[i + half] = __float2bfloat16(x2[j] * c + x1[j] * sn);
    }
  }
}

// ------------------------------------------------------------------------------------------ patch embedding
// SigLIP patch embedding in ONE kernel and in fp32 (the model keeps this island in fp32 under every bf16 cast):
//   out[b, gy*gw + gx, n] = bias[n] + pos[gy*gw + gx, n] + sum_{c,py,px} W[n, (c,py,px)] * pix[b, c, gy*p+py, gx*p+px]
// The non-overlapping patches are gathered straight from the image (no unfolded copy), the product runs on the fp32
// pipes as a 64 x 64 x 16 shared-memory tiled GEMM with 4 x 4 outputs per thread, and bias, position table and the
// cast to the encoder dtype are the epilogue.  PixT = float or bf16, OutT = float or bf16.
template <typename PixT, typename OutT>
__global__ void __launch_bounds__(256)
patch_embed_kernel(const PixT* __restrict__ pix, const float* __restrict__ w, const float* __restrict__ bias,
                   const float* __restrict__ pos, OutT* __restrict__ out, int B, int C, int H, int W, int p, int N) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int gh = H / p, gw = W / p, P = gh * gw, K = C * p * p;
  const long long M = (long long)B * P;
  const long long m0 = (long long)blockIdx.x * BM;
  const int n0 = blockIdx.y * BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    // A tile: 64 patches x 16 taps, gathered from the image
    for (int e = threadIdx.x; e < BM * BK; e += 256) {
      const int mm = e / BK, kk = e % BK;
      const long long m = m0 + mm;
      const int k = k0 + kk;
      float v = 0.f;
      if (m < M && k < K) {
        const int b = int(m / P), pi = int(m % P), gy = pi / gw, gx = pi % gw;
        const int c = k / (p * p), r = k % (p * p), py = r / p, px = r % p;
        const PixT x = pix[(((long long)b * C + c) * H + gy * p + py) * W + gx * p + px];
        if constexpr (sizeof(PixT) == 4) v = x; else v = __bfloat162float(x);
      }
      As[kk][mm] = v;
    }
    // B tile: 64 output features x 16 taps of the flattened convolution weight
    for (int e = threadIdx.x; e < BN * BK; e += 256) {
      const int nn = e / BK, kk = e % BK;
      const int n = n0 + nn, k = k0 + kk;
      Bs[kk][nn] = (n < N && k < K) ? w[(long long)n * K + k] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], bb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bb[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long m = m0 + ty * 4 + i;
    if (m >= M) continue;
    const int pi = int(m % P);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      const float v = acc[i][j] + bias[n] + pos[(long long)pi * N + n];
      if constexpr (sizeof(OutT) == 4) out[m * N + n] = v; else out[m * N + n] = __float2bfloat16(v);
    }
  }
}

// ------------------------------------------------------------------------------------------ flow matching
// [sin | cos] embedding of scalar times with log-spaced periods: out[r, j] = sin(2 pi t_r / P_j),
// out[r, half + j] = cos(...), P_j = min * (max / min)^(j / (half - 1)).  One launch instead of a linspace / pow / mul /
// sin / cos / cat / cast chain per denoise step.  OutT = float or bf16.
template <typename OutT>
__global__ void time_embed_kernel(const float* __restrict__ t, OutT* __restrict__ out, long long rows, int dim,
                                  float min_period, float max_period) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = dim >> 1;
  const long long total = rows * half;
  const float log_ratio = logf(max_period / min_period);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / half;
    const int j = int(i - r * half);
    const float frac = half > 1 ? (float)j / (float)(half - 1) : 0.f;
    const float period = min_period * expf(frac * log_ratio);
    const float ang = 6.283185307179586f / period * t[r];
    float sn, cs;
    sincosf(ang, &sn, &cs);
    if constexpr (sizeof(OutT) == 4) {
      out[r * dim + j] = sn;
      out[r * dim + half + j] = cs;
    } else {
      out[r * dim + j] = __float2bfloat16(sn);
      out[r * dim + half + j] = __float2bfloat16(cs);
    }
  }
}

// Euler update of the denoise loop, in place on the fp32 sample: x += dt * v; rows marked frozen (a committed action
// prefix) are overwritten with the prefix instead.  v is bf16 or fp32; x, prefix are (rows, D); frozen is per row.
template <typename VT>
__global__ void euler_step_kernel(float* __restrict__ x, const VT* __restrict__ v, float dt,
                                  const unsigned char* __restrict__ frozen, const float* __restrict__ prefix,
                                  long long rows, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = rows * D;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / D;
    float vi;
    if constexpr (sizeof(VT) == 4) vi = v[i]; else vi = __bfloat162float(v[i]);
    float xi = x[i] + dt * vi;
    if (frozen != nullptr && frozen[r]) xi = prefix[i];
    x[i] = xi;
  }
}

// Training-side interpolation: x_t = t * noise + (1 - t) * a and the target u_t = noise - a, time per (batch, step) row.
__global__ void flow_interpolate_kernel(const float* __restrict__ a, const float* __restrict__ noise,
                                        const float* __restrict__ t, float* __restrict__ x_t, float* __restrict__ u_t,
                                        long long rows, int D) {
  const long long total = rows * D;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const float tt = t[i / D], ai = a[i], ni = noise[i];
    x_t[i] = tt * ni + (1.f - tt) * ai;
    u_t[i] = ni - ai;
  }
}

// ------------------------------------------------------------------------------------------ cross entropy
// logits fp32 [R][V] -> loss[r] = lse - logit[label], lse[r].  One block per row.
__global__ void ce_fwd_kernel(const float* __restrict__ logits, const long long* __restrict__ labels,
                              float* __restrict__ loss, float* __restrict__ lse_out, int V) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const float* lr = logits + row * (long long)V;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < V; c += blockDim.x) m = fmaxf(m, lr[c]);
  m = block_max(m, red);
  float s = 0.f;
  for (int c = threadIdx.x; c < V; c += blockDim.x) s += __expf(lr[c] - m);
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    float lse = m + logf(s);
    lse_out[row] = lse;
    loss[row] = lse - lr[labels[row]];
  }
}
// dlogits[r][c] = (softmax - onehot) * dloss[r], bf16.
__global__ void ce_bwd_kernel(const float* __restrict__ logits, const long long* __restrict__ labels,
                              const float* __restrict__ lse, const float* __restrict__ dloss,
                              __nv_bfloat16* __restrict__ dlogits, int V) {
  const long long row = blockIdx.x;
  const float* lr = logits + row * (long long)V;
  const float l = lse[row], d = dloss[row];
  const int lab = (int)labels[row];
  for (int c = threadIdx.x; c < V; c += blockDim.x) {
    float p = __expf(lr[c] - l) - (c == lab ? 1.f : 0.f);
    dlogits[row * (long long)V + c] = __float2bfloat16(p * d);
  }
}

// ------------------------------------------------------------------------------------------ optimizer
// Sum of squares of a bf16/fp32 gradient buffer into per-block fp32 partials (deterministic two-stage).
__device__ __forceinline__ void sumsq_load8(const __nv_bfloat16* p, float* v) { load8(p, v); }
__device__ __forceinline__ void sumsq_load8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
// `nvec` groups of 8 elements are read with 128-bit loads (0 when the buffer does not start on a 16-byte boundary);
// the elements after them one by one.  Fixed grid and fixed per-thread order: the result is deterministic.
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ g, long long n, long long nvec, float* __restrict__ partial) {
  __shared__ float red[32];
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec; t += stride) {
    float v[8];
    sumsq_load8(g + t * 8, v);
    s0 += v[0] * v[0] + v[4] * v[4];
    s1 += v[1] * v[1] + v[5] * v[5];
    s2 += v[2] * v[2] + v[6] * v[6];
    s3 += v[3] * v[3] + v[7] * v[7];
  }
  for (long long i = nvec * 8 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) {
    float v = static_cast<float>(g[i]);
    s0 += v * v;
  }
  float s = block_sum((s0 + s1) + (s2 + s3), red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// total = sum(partials) (+ extra terms added by the caller); writes the clip coefficient:
// scale[0] = grad_scale * min(1, max_norm / (sqrt(total) * grad_scale + 1e-6)), scale[1] = norm.
__global__ void clip_coef_kernel(const float* __restrict__ partial, int n, float grad_scale, float max_norm,
                                 float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    float norm = sqrtf(s) * grad_scale;
    float coef = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
    out[0] = grad_scale * coef;
    out[1] = norm;
  }
}
// Fused AdamW on flat buffers: fp32 master/m/v, bf16 gradient in, bf16 parameter copy out.
// `scale_ptr[0]` multiplies the gradient (1/world * clip coefficient), read on the device so that the
// step needs no host round trip.
template <typename G>
__global__ void adamw_kernel(float* __restrict__ p32, const G* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, __nv_bfloat16* __restrict__ p16, long long n, float lr,
                             float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                             const float* __restrict__ scale_ptr) {
  const float gs = scale_ptr ? scale_ptr[0] : 1.f;
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float gr = static_cast<float>(g[i]) * gs;
    float p = p32[i] * (1.f - lr * wd);
    float mm = beta1 * m[i] + (1.f - beta1) * gr;
    float vv = beta2 * v[i] + (1.f - beta2) * gr * gr;
    float denom = sqrtf(vv) * inv_sqrt_bc2 + eps;
    p -= lr * inv_bc1 * mm / denom;
    p32[i] = p;
    m[i] = mm;
    v[i] = vv;
    if (p16) p16[i] = __float2bfloat16(p);
  }
}

// Same update, 8 elements per thread: 128-bit accesses on every stream (two per fp32 array, one per bf16 array)
// and 8 independent loads in flight before the first use.  The launcher picks it when every pointer is 16-byte
// aligned; the last n % 8 elements go through the scalar kernel.
__device__ __forceinline__ void load8f(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void store8f(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void load8g(const __nv_bfloat16* p, float* v) { load8(p, v); }
__device__ __forceinline__ void load8g(const float* p, float* v) { load8f(p, v); }

template <typename G>
__global__ void __launch_bounds__(256) adamw_vec8_kernel(float* __restrict__ p32, const G* __restrict__ g,
                                                         float* __restrict__ m, float* __restrict__ v,
                                                         __nv_bfloat16* __restrict__ p16, long long nvec, float lr,
                                                         float beta1, float beta2, float eps, float wd, float bc1,
                                                         float bc2, const float* __restrict__ scale_ptr) {
  const float gs = scale_ptr ? scale_ptr[0] : 1.f;
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  const float decay = 1.f - lr * wd, step = lr * inv_bc1;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec;
       t += (long long)gridDim.x * blockDim.x) {
    const long long i = t * 8;
    float gr[8], pp[8], mm[8], vv[8];
    load8g(g + i, gr);
    load8f(p32 + i, pp);
    load8f(m + i, mm);
    load8f(v + i, vv);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = gr[k] * gs;
      float pk = pp[k] * decay;
      mm[k] = beta1 * mm[k] + (1.f - beta1) * gk;
      vv[k] = beta2 * vv[k] + (1.f - beta2) * gk * gk;
      const float denom = sqrtf(vv[k]) * inv_sqrt_bc2 + eps;
      pk -= step * mm[k] / denom;
      pp[k] = pk;
    }
    store8f(p32 + i, pp);
    store8f(m + i, mm);
    store8f(v + i, vv);
    if (p16) store8(p16 + i, pp);
  }
}

// ------------------------------------------------------------------------------------------ images
// Aspect-preserving bilinear resize (half-pixel centres, align_corners=False) into the bottom-right
// of a (Hout, Wout) canvas; the top/left margin is filled with pad_value.  in: (N, C, Hin, Win) float.
__global__ void resize_pad_kernel(const float* __restrict__ in, float* __restrict__ out, int NC, int Hin, int Win,
                                  int Hout, int Wout, int rh, int rw, float pad_value) {
  const long long total = (long long)NC * Hout * Wout;
  const int ph = Hout - rh, pw = Wout - rw;
  const float sy = (float)Hin / rh, sx = (float)Win / rw;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    int ox = int(t % Wout);
    long long r = t / Wout;
    int oy = int(r % Hout);
    int nc = int(r / Hout);
    float val = pad_value;
    if (oy >= ph && ox >= pw) {
      float fy = fmaxf((oy - ph + 0.5f) * sy - 0.5f, 0.f);
      float fx = fmaxf((ox - pw + 0.5f) * sx - 0.5f, 0.f);
      int y0 = min((int)fy, Hin - 1), x0 = min((int)fx, Win - 1);
      int y1 = min(y0 + 1, Hin - 1), x1 = min(x0 + 1, Win - 1);
      float wy = fy - y0, wx = fx - x0;
      const float* ip = in + (long long)nc * Hin * Win;
      float a = ip[y0 * Win + x0], b = ip[y0 * Win + x1], c = ip[y1 * Win + x0], d = ip[y1 * Win + x1];
      val = (a * (1 - wx) + b * wx) * (1 - wy) + (c * (1 - wx) + d * wx) * wy;
    }
    out[t] = val;
  }
}

// ------------------------------------------------------------------------------------------ gated residual
// out = x + y * gate, gate row = gate + (row / rows_per_gate) * gate_stride.
__global__ void gated_residual_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                                      const __nv_bfloat16* __restrict__ gate, long long gate_stride,
                                      int rows_per_gate, __nv_bfloat16* __restrict__ out, long long rows, int H) {
  const long long nvec = rows * (long long)(H >> 3);
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec;
       t += (long long)gridDim.x * blockDim.x) {
    const long long row = t / (H >> 3);
    const int c = int(t - row * (H >> 3)) * 8;
    float xv[8], yv[8], gv[8], o[8];
    load8(x + row * (long long)H + c, xv);
    load8(y + row * (long long)H + c, yv);
    load8(gate + (row / rows_per_gate) * gate_stride + c, gv);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = xv[e] + yv[e] * gv[e];
    store8(out + row * (long long)H + c, o);
  }
}

static inline int grid_for(long long work_items, int block, int max_blocks = 148 * 16) {
  long long g = (work_items + block - 1) / block;
  if (g > max_blocks) g = max_blocks;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace otb

using namespace otb;
typedef __nv_bfloat16 bf16;

// same dispatch through launch_pdl (the kernel must call pdl_wait() before it touches global memory)
#define LAUNCH_BY_H_PDL(KERNEL, H, ...)                                                                     \
  do {                                                                                                      \
    int nvec = (H) >> 3;                                                                                    \
    cudaError_t e_;                                                                                         \
    if (nvec <= 128) e_ = launch_pdl(KERNEL<1>, grid, dim3(128), 0, stream, 0u, __VA_ARGS__);               \
    else if (nvec <= 256) e_ = launch_pdl(KERNEL<1>, grid, dim3(256), 0, stream, 0u, __VA_ARGS__);          \
    else if (nvec <= 512) e_ = launch_pdl(KERNEL<2>, grid, dim3(256), 0, stream, 0u, __VA_ARGS__);          \
    else if (nvec <= 1024) e_ = launch_pdl(KERNEL<4>, grid, dim3(256), 0, stream, 0u, __VA_ARGS__);         \
    else return -10;                                                                                        \
    if (e_ != cudaSuccess) return (int)e_;                                                                  \
  } while (0)

#define LAUNCH_BY_H(KERNEL, H, ...)                                                    \
  do {                                                                                 \
    int nvec = (H) >> 3;                                                               \
    if (nvec <= 128) { KERNEL<1><<<grid, 128, 0, stream>>>(__VA_ARGS__); }             \
    else if (nvec <= 256) { KERNEL<1><<<grid, 256, 0, stream>>>(__VA_ARGS__); }        \
    else if (nvec <= 512) { KERNEL<2><<<grid, 256, 0, stream>>>(__VA_ARGS__); }        \
    else if (nvec <= 1024) { KERNEL<4><<<grid, 256, 0, stream>>>(__VA_ARGS__); }       \
    else return -10;                                                                   \
  } while (0)

extern "C" int otb_rms_fwd(const void* x, long long x_stride, const void* w, const void* mod, long long mod_stride,
                           int rows_per_mod, void* y, float* rstd, long long rows, int H, float eps, int mode,
                           cudaStream_t stream) {
  if (H % 8 || rows <= 0) return -1;
  dim3 grid((unsigned)rows);
  LAUNCH_BY_H_PDL(rms_fwd_kernel, H, (const bf16*)x, x_stride, (const bf16*)w, (const bf16*)mod, mod_stride,
                  rows_per_mod < 1 ? 1 : rows_per_mod, (bf16*)y, rstd, H, eps, mode);
  return (int)cudaGetLastError();
}

// dw_partial must hold nblocks*H floats where nblocks = ceil(rows / rows_per_block).
extern "C" int otb_rms_bwd(const void* dy, const void* x, long long x_stride, const void* w, const void* mod,
                           long long mod_stride, int rows_per_mod, const float* rstd, void* dx, float* dw_partial,
                           void* dscale, void* dshift, const void* dres, long long rows, int H, int mode,
                           int rows_per_block, cudaStream_t stream) {
  if (H % 8 || rows <= 0 || rows_per_block <= 0) return -1;
  dim3 grid((unsigned)((rows + rows_per_block - 1) / rows_per_block));
  LAUNCH_BY_H(rms_bwd_kernel, H, (const bf16*)dy, (const bf16*)x, x_stride, (const bf16*)w, (const bf16*)mod,
              mod_stride, rows_per_mod < 1 ? 1 : rows_per_mod, rstd, (bf16*)dx, dw_partial, (bf16*)dscale,
              (bf16*)dshift, (const bf16*)dres, rows, H, mode, rows_per_block);
  return (int)cudaGetLastError();
}

extern "C" int otb_colsum_partials(const float* partial, int nrows, int H, void* out, int accumulate,
                                   cudaStream_t stream) {
  colsum_partials_kernel<<<(H + 255) / 256, 256, 0, stream>>>(partial, nrows, H, (bf16*)out, accumulate);
  return (int)cudaGetLastError();
}

extern "C" int otb_colsum_bf16(const void* a, long long rows, int H, long long lda, float* partial,
                               int rows_per_block, cudaStream_t stream) {
  if (H % 8) return -1;
  dim3 grid((H / 8 + 127) / 128, (unsigned)((rows + rows_per_block - 1) / rows_per_block));
  colsum_bf16_kernel<<<grid, 128, 0, stream>>>((const bf16*)a, rows, H, lda, partial, rows_per_block);
  return (int)cudaGetLastError();
}

// dw_partial and db_partial each hold nblocks*H floats, nblocks = ceil(rows / rows_per_block); x, dy contiguous rows.
extern "C" int otb_ln_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                          float* dw_partial, float* db_partial, long long rows, int H, int rows_per_block,
                          cudaStream_t stream) {
  if (H % 8 || rows <= 0 || rows_per_block <= 0 || !dw_partial || !db_partial) return -1;
  dim3 grid((unsigned)((rows + rows_per_block - 1) / rows_per_block));
  LAUNCH_BY_H(ln_bwd_kernel, H, (const bf16*)dy, (const bf16*)x, (const bf16*)w, mean, rstd, (bf16*)dx, dw_partial,
              db_partial, rows, H, rows_per_block);
  return (int)cudaGetLastError();
}

extern "C" int otb_ln_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
                          long long rows, int H, float eps, cudaStream_t stream) {
  if (H % 8 || rows <= 0) return -1;
  dim3 grid((unsigned)rows);
  LAUNCH_BY_H(ln_fwd_kernel, H, (const bf16*)x, (const bf16*)w, (const bf16*)b, (bf16*)y, mean, rstd, H, eps);
  return (int)cudaGetLastError();
}

extern "C" int otb_glu_fwd(const void* gu, void* h, long long M, int I, int act, cudaStream_t stream) {
  if (I % 32) return -1;
  glu_fwd_kernel<<<grid_for(M * (I / 8), 256), 256, 0, stream>>>((const bf16*)gu, (bf16*)h, M, I, act);
  return (int)cudaGetLastError();
}

extern "C" int otb_glu_bwd(const void* gu, const void* dh, void* dgu, long long M, int I, int act,
                           cudaStream_t stream) {
  if (I % 32) return -1;
  glu_bwd_kernel<<<grid_for(M * (I / 8), 256), 256, 0, stream>>>((const bf16*)gu, (const bf16*)dh, (bf16*)dgu, M, I,
                                                                 act);
  return (int)cudaGetLastError();
}

extern "C" int otb_rope(const void* x, long long sb, long long ss, long long sh, const float* cosb,
                        const float* sinb, void* y, int B, int S, int H, int D, int inverse, cudaStream_t stream) {
  if (D % 8 || (sb % 8) || (ss % 8) || (sh % 8)) return -1;
  if (D % 16 == 0) {
    long long work = (long long)B * S * H * (D / 16);
    rope_kernel<8><<<grid_for(work, 256), 256, 0, stream>>>((const bf16*)x, sb, ss, sh, cosb, sinb, (bf16*)y, B, S, H,
                                                            D, inverse);
  } else {
    long long work = (long long)B * S * H * (D / 8);
    rope_kernel<4><<<grid_for(work, 256), 256, 0, stream>>>((const bf16*)x, sb, ss, sh, cosb, sinb, (bf16*)y, B, S, H,
                                                            D, inverse);
  }
  return (int)cudaGetLastError();
}

extern "C" int otb_qkv_post(const void* qkv, long long ld, const void* qw, const void* kw, float eps, int unit_offset,
                            const float* cosb, const float* sinb, void* q_out, void* k_out, long long k_sb,
                            long long k_ss, void* v_out, long long v_sb, long long v_ss, int B, int T, int H, int Hkv,
                            int D, cudaStream_t stream) {
  if (D % 2 || D > 256 || B <= 0 || T <= 0) return -1;
  const long long warps = (long long)B * T * (H + 2 * Hkv);
  const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
  cudaError_t e = launch_pdl(qkv_post_kernel, dim3(blocks), dim3(256), 0, stream, 0u, (const bf16*)qkv, ld,
                             (const bf16*)qw, (const bf16*)kw, eps, unit_offset, cosb, sinb, (bf16*)q_out, (bf16*)k_out,
                             k_sb, k_ss, (bf16*)v_out, v_sb, v_ss, B, T, H, Hkv, D);
  return (int)e;
}

extern "C" int otb_patch_embed(const void* pix, int pix_bf16, const float* w, const float* bias, const float* pos,
                               void* out, int out_bf16, int B, int C, int H, int W, int p, int N, cudaStream_t stream) {
  if (B <= 0 || C <= 0 || p <= 0 || H % p || W % p || N <= 0) return -1;
  const long long M = (long long)B * (H / p) * (W / p);
  dim3 grid((unsigned)((M + 63) / 64), (unsigned)((N + 63) / 64));
#define OTB_PE(PT, OT) patch_embed_kernel<PT, OT><<<grid, 256, 0, stream>>>((const PT*)pix, w, bias, pos, (OT*)out, B, C, H, W, p, N)
  if (pix_bf16 && out_bf16) OTB_PE(bf16, bf16);
  else if (pix_bf16) OTB_PE(bf16, float);
  else if (out_bf16) OTB_PE(float, bf16);
  else OTB_PE(float, float);
#undef OTB_PE
  return (int)cudaGetLastError();
}

extern "C" int otb_time_embed(const float* t, void* out, long long rows, int dim, float min_period, float max_period,
                              int out_bf16, cudaStream_t stream) {
  if (rows <= 0 || dim < 2 || dim % 2) return -1;
  const dim3 grid(grid_for(rows * (dim / 2), 256));
  cudaError_t e = out_bf16 ? launch_pdl(time_embed_kernel<bf16>, grid, dim3(256), 0, stream, 0u, t, (bf16*)out, rows,
                                        dim, min_period, max_period)
                           : launch_pdl(time_embed_kernel<float>, grid, dim3(256), 0, stream, 0u, t, (float*)out, rows,
                                        dim, min_period, max_period);
  return (int)e;
}

extern "C" int otb_euler_step(float* x, const void* v, int v_bf16, float dt, const unsigned char* frozen,
                              const float* prefix, long long rows, int D, cudaStream_t stream) {
  if (rows <= 0 || D <= 0 || (frozen != nullptr && prefix == nullptr)) return -1;
  const dim3 grid(grid_for(rows * D, 256));
  cudaError_t e = v_bf16 ? launch_pdl(euler_step_kernel<bf16>, grid, dim3(256), 0, stream, 0u, x, (const bf16*)v, dt,
                                      frozen, prefix, rows, D)
                         : launch_pdl(euler_step_kernel<float>, grid, dim3(256), 0, stream, 0u, x, (const float*)v, dt,
                                      frozen, prefix, rows, D);
  return (int)e;
}

extern "C" int otb_flow_interpolate(const float* a, const float* noise, const float* t, float* x_t, float* u_t,
                                    long long rows, int D, cudaStream_t stream) {
  if (rows <= 0 || D <= 0) return -1;
  flow_interpolate_kernel<<<grid_for(rows * D, 256), 256, 0, stream>>>(a, noise, t, x_t, u_t, rows, D);
  return (int)cudaGetLastError();
}

extern "C" int otb_ce_fwd(const float* logits, const long long* labels, float* loss, float* lse, long long rows,
                          int V, cudaStream_t stream) {
  ce_fwd_kernel<<<(unsigned)rows, 256, 0, stream>>>(logits, labels, loss, lse, V);
  return (int)cudaGetLastError();
}

extern "C" int otb_ce_bwd(const float* logits, const long long* labels, const float* lse, const float* dloss,
                          void* dlogits, long long rows, int V, cudaStream_t stream) {
  ce_bwd_kernel<<<(unsigned)rows, 256, 0, stream>>>(logits, labels, lse, dloss, (bf16*)dlogits, V);
  return (int)cudaGetLastError();
}

// nblocks partial sums are written to `partial` (caller provides >= nblocks floats); returns nblocks in *out_n.
extern "C" int otb_sumsq(const void* g, long long n, int is_bf16, float* partial, int nblocks,
                         cudaStream_t stream) {
  const long long nvec = (reinterpret_cast<uintptr_t>(g) & 15) == 0 ? n / 8 : 0;
  if (is_bf16) sumsq_kernel<bf16><<<nblocks, 512, 0, stream>>>((const bf16*)g, n, nvec, partial);
  else sumsq_kernel<float><<<nblocks, 512, 0, stream>>>((const float*)g, n, nvec, partial);
  return (int)cudaGetLastError();
}

extern "C" int otb_clip_coef(const float* partial, int n, float grad_scale, float max_norm, float* out,
                             cudaStream_t stream) {
  clip_coef_kernel<<<1, 256, 0, stream>>>(partial, n, grad_scale, max_norm, out);
  return (int)cudaGetLastError();
}

extern "C" int otb_adamw(float* p32, const void* g, int g_is_bf16, float* m, float* v, void* p16, long long n,
                         float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2,
                         const float* scale_ptr, cudaStream_t stream) {
  auto aligned16 = [](const void* q) { return q == nullptr || (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  long long done = 0;
  if (n >= 8 && aligned16(p32) && aligned16(g) && aligned16(m) && aligned16(v) && aligned16(p16)) {
    const long long nvec = n / 8;
    const int grid = grid_for(nvec, 256, 148 * 8);
    if (g_is_bf16)
      adamw_vec8_kernel<bf16><<<grid, 256, 0, stream>>>(p32, (const bf16*)g, m, v, (bf16*)p16, nvec, lr, beta1, beta2,
                                                        eps, wd, bc1, bc2, scale_ptr);
    else
      adamw_vec8_kernel<float><<<grid, 256, 0, stream>>>(p32, (const float*)g, m, v, (bf16*)p16, nvec, lr, beta1,
                                                         beta2, eps, wd, bc1, bc2, scale_ptr);
    done = nvec * 8;
  }
  const long long rest = n - done;       // everything when unaligned, else the last n % 8 elements
  if (rest > 0) {
    const int grid = grid_for(rest, 512, 148 * 8);
    bf16* p16r = p16 ? (bf16*)p16 + done : nullptr;
    if (g_is_bf16)
      adamw_kernel<bf16><<<grid, 512, 0, stream>>>(p32 + done, (const bf16*)g + done, m + done, v + done, p16r, rest,
                                                   lr, beta1, beta2, eps, wd, bc1, bc2, scale_ptr);
    else
      adamw_kernel<float><<<grid, 512, 0, stream>>>(p32 + done, (const float*)g + done, m + done, v + done, p16r,
                                                    rest, lr, beta1, beta2, eps, wd, bc1, bc2, scale_ptr);
  }
  return (int)cudaGetLastError();
}

extern "C" int otb_resize_pad(const float* in, float* out, int NC, int Hin, int Win, int Hout, int Wout, int rh,
                              int rw, float pad_value, cudaStream_t stream) {
  long long total = (long long)NC * Hout * Wout;
  resize_pad_kernel<<<grid_for(total, 256), 256, 0, stream>>>(in, out, NC, Hin, Win, Hout, Wout, rh, rw, pad_value);
  return (int)cudaGetLastError();
}

extern "C" int otb_gated_residual(const void* x, const void* y, const void* gate, long long gate_stride,
                                  int rows_per_gate, void* out, long long rows, int H, cudaStream_t stream) {
  if (H % 8) return -1;
  gated_residual_kernel<<<grid_for(rows * (H / 8), 256), 256, 0, stream>>>(
      (const bf16*)x, (const bf16*)y, (const bf16*)gate, gate_stride, rows_per_gate < 1 ? 1 : rows_per_gate,
      (bf16*)out, rows, H);
  return (int)cudaGetLastError();
}

// Status word helpers: the library owns one KernelStatus in device memory per device in use.
extern "C" int otb_status_alloc(void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, sizeof(KernelStatus));
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, sizeof(KernelStatus));
  *out = p;
  return (int)e;
}
extern "C" int otb_status_read(void* dev, unsigned int* host4, int reset) {
  cudaError_t e = cudaMemcpy(host4, dev, sizeof(KernelStatus), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess && reset) e = cudaMemset(dev, 0, sizeof(KernelStatus));
  return (int)e;
}
