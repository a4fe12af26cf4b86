// Training-side elementwise kernels that replace short chains of library launches in the step:
//
//   drop_res_fwd / drop_res_bwd   out = x + gate * dropout(y): the dropout after the attention output projection and
//                                 after the MLP, its (optional, per-sample) gate and the residual add in ONE pass.
//                                 The keep mask is never stored: both directions regenerate it from a counter-based
//                                 generator (Philox4x32-10 keyed by the call's seed, one call per 8 elements).
//   masked_mse_fwd / _bwd         flow-matching loss: sum and count of (u - v)^2 over the unmasked elements, per
//                                 sample, in one pass; the backward writes dv directly.
//   ce_tile_fwd                   one vocabulary tile of logits folded into the rows' running softmax statistics
//   pos_resample                  bicubic resample of the SigLIP position table to a native-resolution patch grid
//   embed_fwd / embed_bwd         token embedding gather (with the sqrt(d) scale) and its scatter-add backward into
//                                 an fp32 or bf16 gradient table without a dense one-hot product: rows are processed
//                                 by token ORDER (sorted ids), so each table row is written by one warp, in a fixed
//                                 order, without atomics.
//
// All kernels are bandwidth bound: 16-byte accesses, grid-stride loops, fp32 math.
#include "common.cuh"

namespace otb {

// ------------------------------------------------------------------------------------------ Philox4x32-10
struct U4 {
  unsigned x, y, z, w;
};
__device__ __forceinline__ U4 philox4x32_10(U4 c, unsigned k0, unsigned k1) {
  constexpr unsigned M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned hi0 = __umulhi(M0, c.x), lo0 = M0 * c.x;
    const unsigned hi1 = __umulhi(M1, c.z), lo1 = M1 * c.z;
    c = U4{hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0};
    k0 += W0;
    k1 += W1;
  }
  return c;
}
// keep flags of the 8 elements of vector `vec` (16 random bits each); keep when r16 >= thresh16 (thresh = p * 65536)
__device__ __forceinline__ void keep8(unsigned long long vec, unsigned seed_lo, unsigned seed_hi, unsigned thresh16,
                                      bool* keep) {
  const U4 r = philox4x32_10(U4{(unsigned)vec, (unsigned)(vec >> 32), 0u, 0u}, seed_lo, seed_hi);
  const unsigned w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    keep[2 * i] = (w[i] & 0xFFFFu) >= thresh16;
    keep[2 * i + 1] = (w[i] >> 16) >= thresh16;
  }
}

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float* f) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 t;
  t = unpack_bf16(u.x); f[0] = t.x; f[1] = t.y;
  t = unpack_bf16(u.y); f[2] = t.x; f[3] = t.y;
  t = unpack_bf16(u.z); f[4] = t.x; f[5] = t.y;
  t = unpack_bf16(u.w); f[6] = t.x; f[7] = t.y;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float* f) {
  uint4 o;
  o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]); o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

// out[r, :] = x[r, :] + gate[r / rows_per_gate, :] * keep * y[r, :] / (1 - p)       (gate == nullptr: 1)
__global__ void drop_res_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                                    const __nv_bfloat16* __restrict__ gate, long long gate_stride, int rows_per_gate,
                                    __nv_bfloat16* __restrict__ out, long long rows, int H, unsigned thresh16,
                                    float inv_keep, unsigned seed_lo, unsigned seed_hi) {
  const int hv = H >> 3;
  const long long nvec = rows * hv;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec;
       t += (long long)gridDim.x * blockDim.x) {
    const long long r = t / hv;
    const int c = (int)(t - r * hv) * 8;
    float xv[8], yv[8], gv[8];
    ld8(x + r * H + c, xv);
    ld8(y + r * H + c, yv);
    if (gate != nullptr) ld8(gate + (r / rows_per_gate) * gate_stride + c, gv);
    bool keep[8];
    keep8((unsigned long long)t, seed_lo, seed_hi, thresh16, keep);
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float d = keep[e] ? yv[e] * inv_keep : 0.f;
      o[e] = xv[e] + (gate != nullptr ? gv[e] * d : d);
    }
    st8(out + r * H + c, o);
  }
}

// dy[r, :] = dout[r, :] * gate * keep / (1 - p).  With a gate, one thread owns a (gate row, 8 columns) pair and walks
// its rows_per_gate rows, so dgate[g, :] = sum_r dout * keep * y / (1 - p) needs no atomics and no second pass.
__global__ void drop_res_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                                    const __nv_bfloat16* __restrict__ gate, long long gate_stride, int rows_per_gate,
                                    __nv_bfloat16* __restrict__ dy, float* __restrict__ dgate, long long rows, int H,
                                    unsigned thresh16, float inv_keep, unsigned seed_lo, unsigned seed_hi) {
  const int hv = H >> 3;
  if (gate == nullptr) {
    const long long nvec = rows * hv;
    for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec;
         t += (long long)gridDim.x * blockDim.x) {
      float g[8];
      ld8(dout + t * 8, g);
      bool keep[8];
      keep8((unsigned long long)t, seed_lo, seed_hi, thresh16, keep);
#pragma unroll
      for (int e = 0; e < 8; ++e) g[e] = keep[e] ? g[e] * inv_keep : 0.f;
      st8(dy + t * 8, g);
    }
    return;
  }
  const long long n_gates = rows / rows_per_gate;
  const long long work = n_gates * hv;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < work;
       t += (long long)gridDim.x * blockDim.x) {
    const long long gr = t / hv;
    const int c = (int)(t - gr * hv) * 8;
    float gv[8], acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    ld8(gate + gr * gate_stride + c, gv);
    for (int i = 0; i < rows_per_gate; ++i) {
      const long long r = gr * rows_per_gate + i;
      float g[8], yv[8], o[8];
      ld8(dout + r * H + c, g);
      ld8(y + r * H + c, yv);
      bool keep[8];
      keep8((unsigned long long)(r * hv + (c >> 3)), seed_lo, seed_hi, thresh16, keep);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float m = keep[e] ? inv_keep : 0.f;
        o[e] = g[e] * gv[e] * m;
        acc[e] += g[e] * yv[e] * m;
      }
      st8(dy + r * H + c, o);
    }
    float4* d = reinterpret_cast<float4*>(dgate + gr * H + c);
    d[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    d[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
}

// ------------------------------------------------------------------------------------------ masked MSE
// u, v: (B, T, D) fp32.  Element (b, t, d) counts when !frozen[b, t] && !pad[b, t] && d < real_dim[b] (null pointers
// mean "no such mask").  One block per sample: sums[b] = sum of squared differences, counts[b] = counted elements.
__global__ void masked_mse_fwd_kernel(const float* __restrict__ u, const float* __restrict__ v,
                                      const unsigned char* __restrict__ frozen, const unsigned char* __restrict__ pad,
                                      const long long* __restrict__ real_dim, int T, int D, float* __restrict__ sums,
                                      float* __restrict__ counts) {
  __shared__ float red_s[32], red_c[32];
  const int b = blockIdx.x;
  const int rd = real_dim != nullptr ? (int)real_dim[b] : D;
  float s = 0.f, c = 0.f;
  for (int i = threadIdx.x; i < T * D; i += blockDim.x) {
    const int t = i / D, d = i - t * D;
    const bool on = d < rd && !(frozen != nullptr && frozen[b * T + t]) && !(pad != nullptr && pad[b * T + t]);
    if (on) {
      const float e = u[((long long)b * T + t) * D + d] - v[((long long)b * T + t) * D + d];
      s += e * e;
      c += 1.f;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    c += __shfl_xor_sync(0xffffffffu, c, o);
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) red_s[w] = s, red_c[w] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    float ts = 0.f, tc = 0.f;
    for (int i = 0; i < nw; ++i) ts += red_s[i], tc += red_c[i];
    sums[b] = ts;
    counts[b] = tc;
  }
}
// dv = -2 (u - v) * mask * coef[0]      (coef = upstream gradient / (total count + 1e-8), a device scalar)
__global__ void masked_mse_bwd_kernel(const float* __restrict__ u, const float* __restrict__ v,
                                      const unsigned char* __restrict__ frozen, const unsigned char* __restrict__ pad,
                                      const long long* __restrict__ real_dim, int B, int T, int D,
                                      const float* __restrict__ coef, float* __restrict__ dv) {
  const float k = -2.f * coef[0];
  const long long n = (long long)B * T * D;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int d = (int)(i % D);
    const long long bt = i / D;
    const int b = (int)(bt / T);
    const int rd = real_dim != nullptr ? (int)real_dim[b] : D;
    const bool on = d < rd && !(frozen != nullptr && frozen[bt]) && !(pad != nullptr && pad[bt]);
    dv[i] = on ? k * (u[i] - v[i]) : 0.f;
  }
}

// ------------------------------------------------------------------------------------------ vocabulary-tiled CE
// One tile of logits (rows x Vc, fp32, columns [c0, c0 + Vc) of the vocabulary) is folded into the running softmax
// statistics of every row: m = running max, s = running sum of exp(logit - m); the target logit is picked up by the
// tile that holds the row's label.  After the last tile lse = m + log(s) and loss = lse - target: the full
// rows x vocabulary logits never exist.
__global__ void ce_tile_fwd_kernel(const float* __restrict__ logits, const long long* __restrict__ labels,
                                   long long c0, int Vc, float* __restrict__ m_run, float* __restrict__ s_run,
                                   float* __restrict__ tgt) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const float* lr = logits + row * (long long)Vc;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < Vc; c += blockDim.x) m = fmaxf(m, lr[c]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) red[w] = m;
  __syncthreads();
  m = red[0];
  for (int i = 1; i < nw; ++i) m = fmaxf(m, red[i]);
  __syncthreads();
  float s = 0.f;
  for (int c = threadIdx.x; c < Vc; c += blockDim.x) s += __expf(lr[c] - m);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (l == 0) red[w] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float ts = 0.f;
    for (int i = 0; i < nw; ++i) ts += red[i];
    const float m_old = m_run[row], s_old = s_run[row];
    const float m_new = fmaxf(m_old, m);
    s_run[row] = s_old * __expf(m_old - m_new) + ts * __expf(m - m_new);     // exp(-inf) = 0 on the first tile
    m_run[row] = m_new;
    const long long lab = labels[row] - c0;
    if (lab >= 0 && lab < Vc) tgt[row] = lr[lab];
  }
}

// ------------------------------------------------------------------------------------------ position table resample
// Bicubic (A = -0.75, half-pixel centres, border indices clamped: the convention of F.interpolate(mode="bicubic",
// align_corners=False)) resample of a (g x g, d) fp32 table to (gh x gw, d).
__device__ __forceinline__ void cubic_weights(float t, float* w) {
  constexpr float A = -0.75f;
  const float x0 = t + 1.f, x1 = t, x2 = 1.f - t, x3 = 2.f - t;
  w[0] = ((A * x0 - 5.f * A) * x0 + 8.f * A) * x0 - 4.f * A;
  w[1] = ((A + 2.f) * x1 - (A + 3.f)) * x1 * x1 + 1.f;
  w[2] = ((A + 2.f) * x2 - (A + 3.f)) * x2 * x2 + 1.f;
  w[3] = ((A * x3 - 5.f * A) * x3 + 8.f * A) * x3 - 4.f * A;
}
__global__ void pos_resample_kernel(const float* __restrict__ tab, int g, int d, float* __restrict__ out, int gh,
                                    int gw) {
  const long long n = (long long)gh * gw * d;
  const float sy = (float)g / gh, sx = (float)g / gw;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % d);
    const int pos = (int)(i / d);
    const int oy = pos / gw, ox = pos - oy * gw;
    const float fy = (oy + 0.5f) * sy - 0.5f, fx = (ox + 0.5f) * sx - 0.5f;
    const int iy = (int)floorf(fy), ix = (int)floorf(fx);
    float wy[4], wx[4];
    cubic_weights(fy - iy, wy);
    cubic_weights(fx - ix, wx);
    float acc = 0.f;
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int yy = min(max(iy - 1 + a, 0), g - 1);
      float row = 0.f;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int xx = min(max(ix - 1 + b, 0), g - 1);
        row += wx[b] * tab[((long long)yy * g + xx) * d + c];
      }
      acc += wy[a] * row;
    }
    out[i] = acc;
  }
}

// ------------------------------------------------------------------------------------------ embedding
// out[i, :] = table[ids[i], :] * scale
__global__ void embed_fwd_kernel(const __nv_bfloat16* __restrict__ table, const long long* __restrict__ ids,
                                 __nv_bfloat16* __restrict__ out, long long n_tok, int H, long long vocab,
                                 float scale) {
  const int hv = H >> 3;
  const long long nvec = n_tok * hv;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < nvec;
       t += (long long)gridDim.x * blockDim.x) {
    const long long r = t / hv;
    const int c = (int)(t - r * hv) * 8;
    long long id = ids[r];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);          // ids are validated on the host; never read outside
    float f[8];
    ld8(table + id * H + c, f);
    if (scale != 1.f) {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] *= scale;
    }
    st8(out + r * H + c, f);
  }
}
// sorted_ids ascending with order[j] = position of the j-th smallest id.  One warp per (j, 256-column chunk): it
// works only when j starts a run of equal ids; then it sums the dout rows of the run in order and ADDS the sum (times
// scale) to grad[id, :], which no other warp touches.  No atomics, fixed summation order, no host-side run count.
template <typename G>
__global__ void embed_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const long long* __restrict__ sorted_ids,
                                 const long long* __restrict__ order, long long n_tok, G* __restrict__ grad, int H,
                                 long long vocab, long long pad_id, float scale) {
  const int lane = threadIdx.x & 31;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int chunks = (H + 255) / 256;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long wk = warp; wk < n_tok * chunks; wk += n_warps) {
    const long long j0 = wk / chunks;
    const int c = (int)(wk - j0 * chunks) * 256 + lane * 8;
    const long long id = sorted_ids[j0];
    if (j0 > 0 && sorted_ids[j0 - 1] == id) continue;        // not the first of its run
    if (c >= H || id < 0 || id >= vocab || id == pad_id) continue;   // the padding row takes no gradient
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (long long j = j0; j < n_tok && sorted_ids[j] == id; ++j) {
      float f[8];
      ld8(dout + order[j] * H + c, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    G* g = grad + id * H + c;
    if constexpr (sizeof(G) == 4) {
      float4* g4 = reinterpret_cast<float4*>(g);
      float4 a = g4[0], b = g4[1];
      a.x += acc[0] * scale; a.y += acc[1] * scale; a.z += acc[2] * scale; a.w += acc[3] * scale;
      b.x += acc[4] * scale; b.y += acc[5] * scale; b.z += acc[6] * scale; b.w += acc[7] * scale;
      g4[0] = a;
      g4[1] = b;
    } else {
      float cur[8];
      ld8(reinterpret_cast<const __nv_bfloat16*>(g), cur);
#pragma unroll
      for (int e = 0; e < 8; ++e) cur[e] += acc[e] * scale;
      st8(reinterpret_cast<__nv_bfloat16*>(g), cur);
    }
  }
}

// out[b, s, :] = s < S1 ? a[b, s, :] : c[b, s - S1, :] for rows of E two-byte elements (E a multiple of 8, 16-byte
// aligned rows): the sequence concatenation of cached and new keys / values.  One 16-byte piece per thread.
__global__ void seq_concat_kernel(const uint4* __restrict__ a, long long a_sb, long long a_ss, const uint4* __restrict__ c,
                                  long long c_sb, long long c_ss, uint4* __restrict__ out, long long B, int S1, int S2,
                                  int vec) {
  const long long total = B * (long long)(S1 + S2) * vec;
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < total;
       t += (long long)gridDim.x * blockDim.x) {
    const int v = int(t % vec);
    const long long row = t / vec;
    const int s = int(row % (S1 + S2));
    const long long b = row / (S1 + S2);
    out[t] = s < S1 ? a[b * a_sb + (long long)s * a_ss + v] : c[b * c_sb + (long long)(s - S1) * c_ss + v];
  }
}


}  // namespace otb

using namespace otb;

static int grid_for(long long work, int block) {
  long long g = (work + block - 1) / block;
  if (g < 1) g = 1;
  if (g > 148LL * 16) g = 148LL * 16;
  return (int)g;
}

extern "C" int otb_drop_res_fwd(const void* x, const void* y, const void* gate, long long gate_stride,
                                int rows_per_gate, void* out, long long rows, int H, float p,
                                unsigned long long seed, cudaStream_t stream) {
  if (H % 8 || rows < 0 || p < 0.f || p >= 1.f || (gate != nullptr && (rows_per_gate < 1 || rows % rows_per_gate ||
                                                                          gate_stride % 8)))
    return -1;
  if (rows == 0) return 0;
  const unsigned thresh = (unsigned)(p * 65536.f);
  drop_res_fwd_kernel<<<grid_for(rows * (H / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(y),
      static_cast<const __nv_bfloat16*>(gate), gate_stride, rows_per_gate, static_cast<__nv_bfloat16*>(out), rows, H,
      thresh, 65536.f / (65536.f - (float)thresh), (unsigned)seed, (unsigned)(seed >> 32));
  return (int)cudaGetLastError();
}

extern "C" int otb_drop_res_bwd(const void* dout, const void* y, const void* gate, long long gate_stride,
                                int rows_per_gate, void* dy, float* dgate, long long rows, int H, float p,
                                unsigned long long seed, cudaStream_t stream) {
  if (H % 8 || rows < 0 || p < 0.f || p >= 1.f ||
      (gate != nullptr && (rows_per_gate < 1 || rows % rows_per_gate || gate_stride % 8 || y == nullptr ||
                           dgate == nullptr)))
    return -1;
  if (rows == 0) return 0;
  const unsigned thresh = (unsigned)(p * 65536.f);
  const long long work = gate != nullptr ? (rows / rows_per_gate) * (H / 8) : rows * (H / 8);
  drop_res_bwd_kernel<<<grid_for(work, gate != nullptr ? 128 : 256), gate != nullptr ? 128 : 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(y),
      static_cast<const __nv_bfloat16*>(gate), gate_stride, rows_per_gate, static_cast<__nv_bfloat16*>(dy), dgate,
      rows, H, thresh, 65536.f / (65536.f - (float)thresh), (unsigned)seed, (unsigned)(seed >> 32));
  return (int)cudaGetLastError();
}

extern "C" int otb_masked_mse_fwd(const float* u, const float* v, const unsigned char* frozen,
                                  const unsigned char* pad, const long long* real_dim, int B, int T, int D,
                                  float* sums, float* counts, cudaStream_t stream) {
  if (B < 1 || T < 1 || D < 1) return -1;
  masked_mse_fwd_kernel<<<B, 256, 0, stream>>>(u, v, frozen, pad, real_dim, T, D, sums, counts);
  return (int)cudaGetLastError();
}
extern "C" int otb_masked_mse_bwd(const float* u, const float* v, const unsigned char* frozen,
                                  const unsigned char* pad, const long long* real_dim, int B, int T, int D,
                                  const float* coef, float* dv, cudaStream_t stream) {
  if (B < 1 || T < 1 || D < 1) return -1;
  masked_mse_bwd_kernel<<<grid_for((long long)B * T * D, 256), 256, 0, stream>>>(u, v, frozen, pad, real_dim, B, T, D,
                                                                                 coef, dv);
  return (int)cudaGetLastError();
}

extern "C" int otb_ce_tile_fwd(const float* logits, const long long* labels, long long c0, long long rows, int Vc,
                               float* m_run, float* s_run, float* tgt, cudaStream_t stream) {
  if (rows < 1 || Vc < 1) return -1;
  ce_tile_fwd_kernel<<<(unsigned)rows, 256, 0, stream>>>(logits, labels, c0, Vc, m_run, s_run, tgt);
  return (int)cudaGetLastError();
}

extern "C" int otb_pos_resample(const float* tab, int g, int d, float* out, int gh, int gw, cudaStream_t stream) {
  if (g < 1 || d < 1 || gh < 1 || gw < 1) return -1;
  pos_resample_kernel<<<grid_for((long long)gh * gw * d, 256), 256, 0, stream>>>(tab, g, d, out, gh, gw);
  return (int)cudaGetLastError();
}

extern "C" int otb_embed_fwd(const void* table, const long long* ids, void* out, long long n_tok, int H,
                             long long vocab, float scale, cudaStream_t stream) {
  if (H % 8 || n_tok < 0 || vocab < 1) return -1;
  if (n_tok == 0) return 0;
  embed_fwd_kernel<<<grid_for(n_tok * (H / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(table), ids, static_cast<__nv_bfloat16*>(out), n_tok, H, vocab, scale);
  return (int)cudaGetLastError();
}
extern "C" int otb_embed_bwd(const void* dout, const long long* sorted_ids, const long long* order, long long n_tok,
                             void* grad, int grad_fp32, int H, long long vocab, long long pad_id, float scale,
                             cudaStream_t stream) {
  if (H % 8 || n_tok < 0 || vocab < 1) return -1;
  if (n_tok == 0) return 0;
  const long long warps = n_tok * ((H + 255) / 256);
  const int grid = grid_for(warps * 32, 256);
  if (grad_fp32)
    embed_bwd_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(dout), sorted_ids, order,
                                                      n_tok, static_cast<float*>(grad), H, vocab, pad_id, scale);
  else
    embed_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(dout), sorted_ids,
                                                              order, n_tok, static_cast<__nv_bfloat16*>(grad), H,
                                                              vocab, pad_id, scale);
  return (int)cudaGetLastError();
}

// a: (B, S1, E), c: (B, S2, E) with batch / row strides in ELEMENTS (multiples of 8), innermost contiguous; out: (B, S1 + S2, E)
// contiguous.  Two-byte elements.
extern "C" int otb_seq_concat(const void* a, long long a_sb, long long a_ss, const void* c, long long c_sb, long long c_ss,
                              void* out, long long B, int S1, int S2, int E, cudaStream_t stream) {
  if (B <= 0 || S1 < 0 || S2 < 0 || S1 + S2 <= 0 || E <= 0 || E % 8) return -2;
  if ((a_sb | a_ss | c_sb | c_ss) % 8) return -3;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(out)) & 15) return -4;
  const int vec = E / 8;
  const long long total = B * (long long)(S1 + S2) * vec;
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  seq_concat_kernel<<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(a), a_sb / 8, a_ss / 8,
                                                static_cast<const uint4*>(c), c_sb / 8, c_ss / 8,
                                                static_cast<uint4*>(out), B, S1, S2, vec);
  return (int)cudaGetLastError();
}

// Zero-fill of a dense buffer through the driver's memset path (the flat gradient buffer: several GB per step).
extern "C" int otb_zero_bytes(void* p, unsigned long long bytes, cudaStream_t stream) {
  if (!p || bytes == 0) return p ? 0 : -1;
  return (int)cudaMemsetAsync(p, 0, (size_t)bytes, stream);
}
