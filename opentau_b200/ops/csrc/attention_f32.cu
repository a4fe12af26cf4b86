// Exact fp32 block-causal attention, forward and backward, on the CUDA cores (no tensor-core rounding): the path that
// fp32 policies and fp32 validation runs take, where O(S^2) score tensors of a dense evaluation would not fit.
//
// Decomposition (all three kernels): a 256-thread block owns 32 "owner" rows -- query rows of one head in the forward
// and dQ kernels, keys of one kv head in the dK/dV kernel -- four per warp, and streams tiles of 32 rows of the other
// side through padded shared memory (row stride D + 4 floats: the 128-bit reads of 32 lanes at 32 different rows fall
// into disjoint bank groups).  Inside a tile a lane owns one streamed row for the inner products (score = <q, k>,
// dP = <dO, v>: owner row broadcast from shared memory, streamed row read once for the warp's four owner rows) and
// owns head-dim columns lane, lane + 32, ... for the accumulation (probabilities broadcast from a per-warp strip of
// shared memory).  Softmax statistics live in registers, replicated over the lanes of the warp.
//
//   forward : online softmax; writes O (B,Sq,H*D) and the natural-log LSE (B,H,Sq); a row that sees no key gets
//             O = 0 and LSE = 0
//   dQ      : P is recomputed from LSE; dS = P * (dP - delta) * scale; dQ += dS K
//   dK / dV : the block loops over every head of the GQA group, so the sum over the group happens in registers
//             (no atomics, fixed order)
//   delta   : rowsum(O * dO), one warp per row
//
// Visibility of (query i, key j): q_valid[i] && k_valid[j] && k_blk[j] <= q_blk[i].  Streamed tiles whose keys are
// all hidden from every owner row (or the reverse) are skipped after their block ids are loaded.
#include <cuda_runtime.h>
#include <limits.h>
#include <math.h>
#include <stdint.h>

namespace otb {

constexpr int F32_ROWS = 32;      // owner rows per block = streamed rows per tile
constexpr int F32_THREADS = 256;  // 8 warps x 4 owner rows
constexpr int F32_RPW = 4;        // owner rows per warp

struct F32Params {
  const float* q;
  const float* k;
  const float* v;
  long long q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh;
  const int* q_blk;
  const int* k_blk;
  const unsigned char* q_valid;
  const unsigned char* k_valid;
  int B, Sq, Sk, H, Hkv, D;
  float scale;
};

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// rows [r0, r0 + 32) of a (rows, D) matrix with row stride `rs` -> shared tile with row stride D + 4; rows past `nrows`
// are zero-filled.  All 256 threads; 128-bit accesses (D is a multiple of 4, bases 16-byte aligned).
__device__ __forceinline__ void load_tile(float* dst, const float* src, long long rs, int r0, int nrows, int D) {
  const int ld = D + 4, vec = D >> 2;
  for (int i = threadIdx.x; i < F32_ROWS * vec; i += F32_THREADS) {
    const int r = i / vec, c = (i - r * vec) << 2;
    float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r0 + r < nrows) x = *reinterpret_cast<const float4*>(src + (long long)(r0 + r) * rs + c);
    *reinterpret_cast<float4*>(dst + r * ld + c) = x;
  }
}

// inner products of the warp's four owner rows (shared, broadcast) with this lane's streamed row (shared)
__device__ __forceinline__ void dot4(const float* own, const float* mine, int ld, int D, float out[F32_RPW]) {
#pragma unroll
  for (int r = 0; r < F32_RPW; ++r) out[r] = 0.f;
  for (int c = 0; c < D; c += 4) {
    const float4 y = *reinterpret_cast<const float4*>(mine + c);
#pragma unroll
    for (int r = 0; r < F32_RPW; ++r) {
      const float4 x = *reinterpret_cast<const float4*>(own + r * ld + c);
      out[r] = fmaf(x.x, y.x, fmaf(x.y, y.y, fmaf(x.z, y.z, fmaf(x.w, y.w, out[r]))));
    }
  }
}

// ---------------------------------------------------------------------------------------------------------- forward
template <int DC>  // DC = ceil(D / 32): head-dim columns per lane
__global__ void __launch_bounds__(F32_THREADS) attn_f32_fwd_kernel(F32Params p, float* __restrict__ o,
                                                                   float* __restrict__ lse) {
  extern __shared__ __align__(16) float smem[];
  const int D = p.D, ld = D + 4;
  float* sQ = smem;                       // [32][ld]
  float* sK = sQ + F32_ROWS * ld;         // [32][ld]
  float* sV = sK + F32_ROWS * ld;         // [32][ld]
  float* sP = sV + F32_ROWS * ld;         // [8 warps][4][32]
  int* sKb = reinterpret_cast<int*>(sP + 8 * F32_RPW * 32);   // [32] block id of the tile's keys (INT_MAX = hidden)
  __shared__ int s_tile_min;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * F32_ROWS, h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.H / p.Hkv);
  const float* qb = p.q + (long long)b * p.q_sb + (long long)h * p.q_sh;
  const float* kb = p.k + (long long)b * p.k_sb + (long long)kvh * p.k_sh;
  const float* vb = p.v + (long long)b * p.v_sb + (long long)kvh * p.v_sh;
  load_tile(sQ, qb, p.q_ss, q0, p.Sq, D);

  int row_blk[F32_RPW];
  bool row_ok[F32_RPW];
  int blk_max = INT_MIN;
#pragma unroll
  for (int r = 0; r < F32_RPW; ++r) {
    const int i = q0 + warp * F32_RPW + r;
    row_ok[r] = i < p.Sq && p.q_valid[(long long)b * p.Sq + i] != 0;
    row_blk[r] = row_ok[r] ? p.q_blk[(long long)b * p.Sq + i] : INT_MIN;
  }
  // the largest block id among the block's valid query rows: a key tile above it is hidden from all of them
  {
    const int i = q0 + lane;
    int mine = INT_MIN;
    if (i < p.Sq && p.q_valid[(long long)b * p.Sq + i]) mine = p.q_blk[(long long)b * p.Sq + i];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mine = max(mine, __shfl_xor_sync(0xffffffffu, mine, off));
    blk_max = mine;
  }

  float m[F32_RPW], l[F32_RPW], acc[F32_RPW][DC];
#pragma unroll
  for (int r = 0; r < F32_RPW; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < DC; ++c) acc[r][c] = 0.f;
  }
  const float* own = sQ + warp * F32_RPW * ld;
  float* myP = sP + warp * F32_RPW * 32;

  for (int k0 = 0; k0 < p.Sk; k0 += F32_ROWS) {
    __syncthreads();   // the previous tile is no longer read
    if (threadIdx.x < 32) {
      const int j = k0 + threadIdx.x;
      int kbv = INT_MAX;
      if (j < p.Sk && p.k_valid[(long long)b * p.Sk + j]) kbv = p.k_blk[(long long)b * p.Sk + j];
      sKb[threadIdx.x] = kbv;
      int mn = kbv;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, off));
      if (threadIdx.x == 0) s_tile_min = mn;
    }
    __syncthreads();
    if (s_tile_min > blk_max) continue;   // uniform over the block
    load_tile(sK, kb, p.k_ss, k0, p.Sk, D);
    load_tile(sV, vb, p.v_ss, k0, p.Sk, D);
    __syncthreads();

    float s[F32_RPW];
    dot4(own, sK + lane * ld, ld, D, s);
    const int kblk = sKb[lane];
#pragma unroll
    for (int r = 0; r < F32_RPW; ++r) {
      const bool vis = row_ok[r] && kblk <= row_blk[r];
      const float sv = vis ? s[r] * p.scale : -INFINITY;
      const float mt = warp_max(sv);
      const float mn = fmaxf(m[r], mt);
      float pr = 0.f, corr = 1.f;
      if (mn != -INFINITY) {
        pr = vis ? expf(sv - mn) : 0.f;
        corr = m[r] == -INFINITY ? 0.f : expf(m[r] - mn);
      }
      l[r] = l[r] * corr + warp_sum(pr);
      m[r] = mn;
#pragma unroll
      for (int c = 0; c < DC; ++c) acc[r][c] *= corr;
      myP[r * 32 + lane] = pr;
    }
    __syncwarp();
    for (int j = 0; j < F32_ROWS; ++j) {
      float pj[F32_RPW];
#pragma unroll
      for (int r = 0; r < F32_RPW; ++r) pj[r] = myP[r * 32 + j];
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        const int d = lane + 32 * c;
        if (d < D) {
          const float vv = sV[j * ld + d];
#pragma unroll
          for (int r = 0; r < F32_RPW; ++r) acc[r][c] = fmaf(pj[r], vv, acc[r][c]);
        }
      }
    }
    __syncwarp();
  }

#pragma unroll
  for (int r = 0; r < F32_RPW; ++r) {
    const int i = q0 + warp * F32_RPW + r;
    if (i >= p.Sq) continue;
    const bool any = l[r] > 0.f;
    const float inv = any ? 1.f / l[r] : 0.f;
    float* orow = o + ((long long)b * p.Sq + i) * p.H * D + (long long)h * D;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int d = lane + 32 * c;
      if (d < D) orow[d] = acc[r][c] * inv;
    }
    if (lane == 0) lse[((long long)b * p.H + h) * p.Sq + i] = any ? m[r] + logf(l[r]) : 0.f;
  }
}

// delta[b,h,i] = sum_d O[b,i,h,d] * dO[b,i,h,d]; one warp per row
__global__ void attn_f32_delta_kernel(const float* __restrict__ o, const float* __restrict__ d_o,
                                      float* __restrict__ delta, int B, int S, int H, int D) {
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= (long long)B * S * H) return;
  float a = 0.f;
  for (int d = lane; d < D; d += 32) a = fmaf(o[row * D + d], d_o[row * D + d], a);
  a = warp_sum(a);
  if (lane == 0) {
    const int h = int(row % H);
    const long long bs = row / H;
    delta[((bs / S) * H + h) * S + bs % S] = a;
  }
}

// --------------------------------------------------------------------------------------------------------------- dQ
template <int DC>
__global__ void __launch_bounds__(F32_THREADS) attn_f32_dq_kernel(F32Params p, const float* __restrict__ d_o,
                                                                  const float* __restrict__ lse,
                                                                  const float* __restrict__ delta,
                                                                  float* __restrict__ dq) {
  extern __shared__ __align__(16) float smem[];
  const int D = p.D, ld = D + 4;
  float* sQ = smem;
  float* sDO = sQ + F32_ROWS * ld;
  float* sK = sDO + F32_ROWS * ld;
  float* sV = sK + F32_ROWS * ld;
  float* sP = sV + F32_ROWS * ld;
  int* sKb = reinterpret_cast<int*>(sP + 8 * F32_RPW * 32);
  __shared__ int s_tile_min;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * F32_ROWS, h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.H / p.Hkv);
  const float* qb = p.q + (long long)b * p.q_sb + (long long)h * p.q_sh;
  const float* kb = p.k + (long long)b * p.k_sb + (long long)kvh * p.k_sh;
  const float* vb = p.v + (long long)b * p.v_sb + (long long)kvh * p.v_sh;
  const float* dob = d_o + (long long)b * p.Sq * p.H * D + (long long)h * D;   // contiguous (B,Sq,H,D)
  load_tile(sQ, qb, p.q_ss, q0, p.Sq, D);
  load_tile(sDO, dob, (long long)p.H * D, q0, p.Sq, D);

  int row_blk[F32_RPW];
  bool row_ok[F32_RPW];
  float row_lse[F32_RPW], row_delta[F32_RPW];
#pragma unroll
  for (int r = 0; r < F32_RPW; ++r) {
    const int i = q0 + warp * F32_RPW + r;
    row_ok[r] = i < p.Sq && p.q_valid[(long long)b * p.Sq + i] != 0;
    row_blk[r] = row_ok[r] ? p.q_blk[(long long)b * p.Sq + i] : INT_MIN;
    row_lse[r] = row_ok[r] ? lse[((long long)b * p.H + h) * p.Sq + i] : 0.f;
    row_delta[r] = row_ok[r] ? delta[((long long)b * p.H + h) * p.Sq + i] : 0.f;
  }
  int blk_max;
  {
    const int i = q0 + lane;
    int mine = INT_MIN;
    if (i < p.Sq && p.q_valid[(long long)b * p.Sq + i]) mine = p.q_blk[(long long)b * p.Sq + i];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mine = max(mine, __shfl_xor_sync(0xffffffffu, mine, off));
    blk_max = mine;
  }
  float acc[F32_RPW][DC];
#pragma unroll
  for (int r = 0; r < F32_RPW; ++r)
#pragma unroll
    for (int c = 0; c < DC; ++c) acc[r][c] = 0.f;
  const float* ownQ = sQ + warp * F32_RPW * ld;
  const float* ownDO = sDO + warp * F32_RPW * ld;
  float* myP = sP + warp * F32_RPW * 32;

  for (int k0 = 0; k0 < p.Sk; k0 += F32_ROWS) {
    __syncthreads();
    if (threadIdx.x < 32) {
      const int j = k0 + threadIdx.x;
      int kbv = INT_MAX;
      if (j < p.Sk && p.k_valid[(long long)b * p.Sk + j]) kbv = p.k_blk[(long long)b * p.Sk + j];
      sKb[threadIdx.x] = kbv;
      int mn = kbv;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, off));
      if (threadIdx.x == 0) s_tile_min = mn;
    }
    __syncthreads();
    if (s_tile_min > blk_max) continue;
    load_tile(sK, kb, p.k_ss, k0, p.Sk, D);
    load_tile(sV, vb, p.v_ss, k0, p.Sk, D);
    __syncthreads();
    float s[F32_RPW], dp[F32_RPW];
    dot4(ownQ, sK + lane * ld, ld, D, s);
    dot4(ownDO, sV + lane * ld, ld, D, dp);
    const int kblk = sKb[lane];
#pragma unroll
    for (int r = 0; r < F32_RPW; ++r) {
      const bool vis = row_ok[r] && kblk <= row_blk[r];
      const float pr = vis ? expf(s[r] * p.scale - row_lse[r]) : 0.f;
      myP[r * 32 + lane] = pr * (dp[r] - row_delta[r]) * p.scale;
    }
    __syncwarp();
    for (int j = 0; j < F32_ROWS; ++j) {
      float dj[F32_RPW];
#pragma unroll
      for (int r = 0; r < F32_RPW; ++r) dj[r] = myP[r * 32 + j];
#pragma unroll
      for (int c = 0; c < DC; ++c) {
        const int d = lane + 32 * c;
        if (d < D) {
          const float kk = sK[j * ld + d];
#pragma unroll
          for (int r = 0; r < F32_RPW; ++r) acc[r][c] = fmaf(dj[r], kk, acc[r][c]);
        }
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int r = 0; r < F32_RPW; ++r) {
    const int i = q0 + warp * F32_RPW + r;
    if (i >= p.Sq) continue;
    float* row = dq + (((long long)b * p.Sq + i) * p.H + h) * D;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int d = lane + 32 * c;
      if (d < D) row[d] = acc[r][c];
    }
  }
}

// ------------------------------------------------------------------------------------------------------------ dK, dV
template <int DC>
__global__ void __launch_bounds__(F32_THREADS) attn_f32_dkv_kernel(F32Params p, const float* __restrict__ d_o,
                                                                   const float* __restrict__ lse,
                                                                   const float* __restrict__ delta,
                                                                   float* __restrict__ dk, float* __restrict__ dv) {
  extern __shared__ __align__(16) float smem[];
  const int D = p.D, ld = D + 4;
  float* sK = smem;                        // owner tiles
  float* sV = sK + F32_ROWS * ld;
  float* sQ = sV + F32_ROWS * ld;          // streamed tiles
  float* sDO = sQ + F32_ROWS * ld;
  float* sP = sDO + F32_ROWS * ld;         // [8][4][32] probabilities
  float* sS = sP + 8 * F32_RPW * 32;       // [8][4][32] dS
  int* sQb = reinterpret_cast<int*>(sS + 8 * F32_RPW * 32);   // [32] block id of the tile's queries (INT_MIN = hidden)
  float* sL = reinterpret_cast<float*>(sQb + 32);             // [32] lse
  float* sDl = sL + 32;                                       // [32] delta
  __shared__ int s_tile_max;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * F32_ROWS, kvh = blockIdx.y, b = blockIdx.z;
  const int g = p.H / p.Hkv;
  const float* kb = p.k + (long long)b * p.k_sb + (long long)kvh * p.k_sh;
  const float* vb = p.v + (long long)b * p.v_sb + (long long)kvh * p.v_sh;
  load_tile(sK, kb, p.k_ss, k0, p.Sk, D);
  load_tile(sV, vb, p.v_ss, k0, p.Sk, D);

  int key_blk[F32_RPW];
  bool key_ok[F32_RPW];
#pragma unroll
  for (int r = 0; r < F32_RPW; ++r) {
    const int j = k0 + warp * F32_RPW + r;
    key_ok[r] = j < p.Sk && p.k_valid[(long long)b * p.Sk + j] != 0;
    key_blk[r] = key_ok[r] ? p.k_blk[(long long)b * p.Sk + j] : INT_MAX;
  }
  int blk_min;   // the smallest block id among the block's valid keys: a query tile below it sees none of them
  {
    const int j = k0 + lane;
    int mine = INT_MAX;
    if (j < p.Sk && p.k_valid[(long long)b * p.Sk + j]) mine = p.k_blk[(long long)b * p.Sk + j];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mine = min(mine, __shfl_xor_sync(0xffffffffu, mine, off));
    blk_min = mine;
  }
  float ak[F32_RPW][DC], av[F32_RPW][DC];
#pragma unroll
  for (int r = 0; r < F32_RPW; ++r)
#pragma unroll
    for (int c = 0; c < DC; ++c) ak[r][c] = av[r][c] = 0.f;
  const float* ownK = sK + warp * F32_RPW * ld;
  const float* ownV = sV + warp * F32_RPW * ld;
  float* myP = sP + warp * F32_RPW * 32;
  float* myS = sS + warp * F32_RPW * 32;

  for (int hh = 0; hh < g; ++hh) {
    const int h = kvh * g + hh;
    const float* qb = p.q + (long long)b * p.q_sb + (long long)h * p.q_sh;
    const float* dob = d_o + (long long)b * p.Sq * p.H * D + (long long)h * D;
    for (int q0 = 0; q0 < p.Sq; q0 += F32_ROWS) {
      __syncthreads();
      if (threadIdx.x < 32) {
        const int i = q0 + threadIdx.x;
        int qbv = INT_MIN;
        float lv = 0.f, dl = 0.f;
        if (i < p.Sq && p.q_valid[(long long)b * p.Sq + i]) {
          qbv = p.q_blk[(long long)b * p.Sq + i];
          lv = lse[((long long)b * p.H + h) * p.Sq + i];
          dl = delta[((long long)b * p.H + h) * p.Sq + i];
        }
        sQb[threadIdx.x] = qbv;
        sL[threadIdx.x] = lv;
        sDl[threadIdx.x] = dl;
        int mx = qbv;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        if (threadIdx.x == 0) s_tile_max = mx;
      }
      __syncthreads();
      if (s_tile_max < blk_min) continue;
      load_tile(sQ, qb, p.q_ss, q0, p.Sq, D);
      load_tile(sDO, dob, (long long)p.H * D, q0, p.Sq, D);
      __syncthreads();
      float s[F32_RPW], dp[F32_RPW];
      dot4(ownK, sQ + lane * ld, ld, D, s);      // lane = query row of the tile
      dot4(ownV, sDO + lane * ld, ld, D, dp);
      const int qblk = sQb[lane];
      const float lv = sL[lane], dl = sDl[lane];
#pragma unroll
      for (int r = 0; r < F32_RPW; ++r) {
        const bool vis = key_ok[r] && qblk != INT_MIN && key_blk[r] <= qblk;
        const float pr = vis ? expf(s[r] * p.scale - lv) : 0.f;
        myP[r * 32 + lane] = pr;
        myS[r * 32 + lane] = pr * (dp[r] - dl) * p.scale;
      }
      __syncwarp();
      for (int i = 0; i < F32_ROWS; ++i) {
        float pi[F32_RPW], si[F32_RPW];
#pragma unroll
        for (int r = 0; r < F32_RPW; ++r) {
          pi[r] = myP[r * 32 + i];
          si[r] = myS[r * 32 + i];
        }
#pragma unroll
        for (int c = 0; c < DC; ++c) {
          const int d = lane + 32 * c;
          if (d < D) {
            const float dd = sDO[i * ld + d], qq = sQ[i * ld + d];
#pragma unroll
            for (int r = 0; r < F32_RPW; ++r) {
              av[r][c] = fmaf(pi[r], dd, av[r][c]);
              ak[r][c] = fmaf(si[r], qq, ak[r][c]);
            }
          }
        }
      }
      __syncwarp();
    }
  }
#pragma unroll
  for (int r = 0; r < F32_RPW; ++r) {
    const int j = k0 + warp * F32_RPW + r;
    if (j >= p.Sk) continue;
    float* rk = dk + (((long long)b * p.Sk + j) * p.Hkv + kvh) * D;
    float* rv = dv + (((long long)b * p.Sk + j) * p.Hkv + kvh) * D;
#pragma unroll
    for (int c = 0; c < DC; ++c) {
      const int d = lane + 32 * c;
      if (d < D) {
        rk[d] = ak[r][c];
        rv[d] = av[r][c];
      }
    }
  }
}

static int check(const F32Params& p) {
  if (p.B <= 0 || p.Sq <= 0 || p.Sk <= 0 || p.H <= 0 || p.Hkv <= 0 || p.H % p.Hkv) return -2;
  if (p.D % 4 || p.D < 4 || p.D > 256) return -4;
  const long long st[9] = {p.q_sb, p.q_ss, p.q_sh, p.k_sb, p.k_ss, p.k_sh, p.v_sb, p.v_ss, p.v_sh};
  for (int i = 0; i < 9; ++i)
    if (st[i] % 4) return -5;
  if ((reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v)) & 15)
    return -6;
  return 0;
}

template <typename K>
static int set_smem(K kern, size_t bytes) {
  return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace otb

using namespace otb;

#define F32_DISPATCH(D, CALL)                      \
  do {                                             \
    const int dc_ = ((D) + 31) / 32;               \
    if (dc_ <= 1) { CALL(1); }                     \
    else if (dc_ <= 2) { CALL(2); }                \
    else if (dc_ <= 3) { CALL(3); }                \
    else if (dc_ <= 4) { CALL(4); }                \
    else if (dc_ <= 6) { CALL(6); }                \
    else { CALL(8); }                              \
  } while (0)

static F32Params make_params(const float* q, const float* k, const float* v, const int* q_blk, const int* k_blk,
                             const unsigned char* q_valid, const unsigned char* k_valid, int B, int Sq, int Sk, int H,
                             int Hkv, int D, long long q_sb, long long q_ss, long long q_sh, long long k_sb,
                             long long k_ss, long long k_sh, long long v_sb, long long v_ss, long long v_sh,
                             float scale) {
  F32Params p;
  p.q = q; p.k = k; p.v = v;
  p.q_sb = q_sb; p.q_ss = q_ss; p.q_sh = q_sh; p.k_sb = k_sb; p.k_ss = k_ss; p.k_sh = k_sh;
  p.v_sb = v_sb; p.v_ss = v_ss; p.v_sh = v_sh;
  p.q_blk = q_blk; p.k_blk = k_blk; p.q_valid = q_valid; p.k_valid = k_valid;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.H = H; p.Hkv = Hkv; p.D = D; p.scale = scale;
  return p;
}

// q (B,Sq,H,D), k / v (B,Sk,Hkv,D) fp32 with element strides (innermost 1); o (B,Sq,H*D) and lse (B,H,Sq) contiguous.
extern "C" int otb_attn_f32_fwd(const float* q, const float* k, const float* v, float* o, float* lse, const int* q_blk,
                                const int* k_blk, const unsigned char* q_valid, const unsigned char* k_valid, int B,
                                int Sq, int Sk, int H, int Hkv, int D, long long q_sb, long long q_ss, long long q_sh,
                                long long k_sb, long long k_ss, long long k_sh, long long v_sb, long long v_ss,
                                long long v_sh, float scale, cudaStream_t stream) {
  const F32Params p = make_params(q, k, v, q_blk, k_blk, q_valid, k_valid, B, Sq, Sk, H, Hkv, D, q_sb, q_ss, q_sh, k_sb,
                                  k_ss, k_sh, v_sb, v_ss, v_sh, scale);
  int r = check(p);
  if (r) return r;
  const size_t smem = (size_t)(3 * F32_ROWS * (D + 4) + 8 * F32_RPW * 32 + 32) * 4;
  const dim3 grid((Sq + F32_ROWS - 1) / F32_ROWS, H, B);
#define CALL(DC)                                                            \
  r = set_smem(attn_f32_fwd_kernel<DC>, smem);                              \
  if (r) return r;                                                          \
  attn_f32_fwd_kernel<DC><<<grid, F32_THREADS, smem, stream>>>(p, o, lse)
  F32_DISPATCH(D, CALL);
#undef CALL
  return (int)cudaGetLastError();
}

// o, d_o (B,Sq,H,D) contiguous; delta: scratch (B,H,Sq); dq (B,Sq,H,D), dk / dv (B,Sk,Hkv,D) contiguous outputs.
extern "C" int otb_attn_f32_bwd(const float* q, const float* k, const float* v, const float* o, const float* d_o,
                                const float* lse, float* delta, float* dq, float* dk, float* dv, const int* q_blk,
                                const int* k_blk, const unsigned char* q_valid, const unsigned char* k_valid, int B,
                                int Sq, int Sk, int H, int Hkv, int D, long long q_sb, long long q_ss, long long q_sh,
                                long long k_sb, long long k_ss, long long k_sh, long long v_sb, long long v_ss,
                                long long v_sh, float scale, cudaStream_t stream) {
  const F32Params p = make_params(q, k, v, q_blk, k_blk, q_valid, k_valid, B, Sq, Sk, H, Hkv, D, q_sb, q_ss, q_sh, k_sb,
                                  k_ss, k_sh, v_sb, v_ss, v_sh, scale);
  int r = check(p);
  if (r) return r;
  {
    const long long rows = (long long)B * Sq * H;
    const long long blocks = (rows * 32 + 255) / 256;
    attn_f32_delta_kernel<<<(unsigned)blocks, 256, 0, stream>>>(o, d_o, delta, B, Sq, H, D);
  }
  const size_t smem_q = (size_t)(4 * F32_ROWS * (D + 4) + 8 * F32_RPW * 32 + 32) * 4;
  const size_t smem_kv = (size_t)(4 * F32_ROWS * (D + 4) + 2 * 8 * F32_RPW * 32 + 96) * 4;
  const dim3 grid_q((Sq + F32_ROWS - 1) / F32_ROWS, H, B);
  const dim3 grid_kv((Sk + F32_ROWS - 1) / F32_ROWS, Hkv, B);
#define CALL(DC)                                                                            \
  r = set_smem(attn_f32_dq_kernel<DC>, smem_q);                                             \
  if (r) return r;                                                                          \
  attn_f32_dq_kernel<DC><<<grid_q, F32_THREADS, smem_q, stream>>>(p, d_o, lse, delta, dq);   \
  r = set_smem(attn_f32_dkv_kernel<DC>, smem_kv);                                           \
  if (r) return 100000 + r;                                                                 \
  attn_f32_dkv_kernel<DC><<<grid_kv, F32_THREADS, smem_kv, stream>>>(p, d_o, lse, delta, dk, dv)
  F32_DISPATCH(D, CALL);
#undef CALL
  return (int)cudaGetLastError();
}
