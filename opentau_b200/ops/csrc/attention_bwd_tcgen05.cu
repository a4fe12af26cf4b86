// Block-causal flash attention backward for sm_100a (tcgen05 + TMEM + TMA).
//
// Three launches of one templated kernel, each an "inner products -> elementwise -> accumulate" pipeline
// with the same warp roles as the forward kernel (warp 0 TMA, warp 1 MMA, warps 2..9 elementwise: two warps per
// TMEM lane quadrant split the columns of a block; groups of 32 columns that are fully visible or fully hidden for a
// row skip the per-element mask test):
//
//   MODE_DQ  tile = 128 query rows (position x head-of-group); stream key blocks j:
//              S = Q K_j^T, dP = dO V_j^T  ->  dS = P o (dP - delta) * scale  ->  dQ += dS K_j
//   MODE_DK  tile = 128 keys of one kv head; stream query-row blocks i (all heads of the group, so
//            the GQA sum happens inside the accumulator, without atomics):
//              S^T = K Q_i^T, dP^T = V dO_i^T  ->  dS^T  ->  dK += dS^T Q_i
//   MODE_DV  tile = 128 keys; stream query-row blocks:
//              S^T = K Q_i^T  ->  P^T  ->  dV += P^T dO_i
//
// P is recomputed from the saved log-sum-exp (no running maximum needed); delta = rowsum(O o dO) comes
// from a small pre-kernel.  Splitting dK and dV keeps each accumulator (128 x D fp32 = up to 256 TMEM
// columns) next to double-buffered score tiles inside the 512-column tensor memory at D = 256.
// Results are deterministic: no atomics, fixed accumulation order.
#include "common.cuh"
#include <limits.h>

namespace otb {

constexpr unsigned KID_ATTN_BWD = 3;
constexpr int BW_M = 128;
enum { MODE_DQ = 0, MODE_DK = 1, MODE_DV = 2 };

struct BwdParams {
  int B, Sq, Sk, H, Hkv, D, Dmma, g;
  float scale, scale_log2;
  const int* q_blk;
  const int* k_blk;
  const unsigned char* q_valid;
  const unsigned char* k_valid;
  const float* lse;     // (B, H, Sq), natural log
  const float* delta;   // (B, H, Sq)
  __nv_bfloat16* out;   // dq (B,Sq,H,D) | dk, dv (B,Sk,Hkv,D), contiguous
  KernelStatus* status;
};

template <int MODE, int DPAD, int BN>
struct BwdSmem {
  static constexpr int NF = MODE == MODE_DV ? 1 : 2;          // fixed tiles
  static constexpr int NCHUNK = DPAD / 64;
  static constexpr int F_BYTES = BW_M * DPAD * 2;
  static constexpr int Y_BYTES = BN * DPAD * 2;
  static constexpr int STAGE_BYTES = 2 * Y_BYTES;
  static constexpr int T_CHUNKS = (BN + 63) / 64;
  static constexpr int T_BYTES = T_CHUNKS * BW_M * 128;
  static constexpr int OFF_F = 0;
  static constexpr int OFF_Y = NF * F_BYTES;
  static constexpr int OFF_T = OFF_Y + 2 * STAGE_BYTES;
  static constexpr int OFF_META = OFF_T + 2 * T_BYTES;        // per slot: int blk[BN], float lse2[BN], float delta[BN]
  static constexpr int OFF_KMM = OFF_META + 2 * BN * 12;       // int kmm[2][BN/32][2]: min / max block id per 32 columns
  static constexpr int OFF_BAR = OFF_KMM + 2 * (BN / 32) * 2 * 4;
  static constexpr int NBAR = 16;
  static constexpr int TOTAL = OFF_BAR + NBAR * 8 + 32 + 1024;
  static constexpr int NS = MODE == MODE_DV ? 1 : 2;          // score tiles per block
  static constexpr int TMEM_ACC = 2 * NS * BN;                // accumulator column offset
};

__device__ __forceinline__ float bw_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int MODE, int DPAD, int BN>
__global__ void __launch_bounds__(320, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_f1, const __grid_constant__ CUtensorMap tm_f2,
                const __grid_constant__ CUtensorMap tm_y1, const __grid_constant__ CUtensorMap tm_y2, BwdParams p) {
  using L = BwdSmem<MODE, DPAD, BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sF = smem + L::OFF_F;
  uint8_t* sY = smem + L::OFF_Y;
  uint8_t* sT = smem + L::OFF_T;
  int* meta_blk = reinterpret_cast<int*>(smem + L::OFF_META);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* f_full = bars + 0;
  uint64_t* y_full = bars + 1;    // [2]
  uint64_t* y_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;    // [2]
  uint64_t* s_free = bars + 7;    // [2]
  uint64_t* t_full = bars + 9;    // [2]
  uint64_t* t_free = bars + 11;   // [2]
  uint64_t* acc_full = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* range_smem = reinterpret_cast<int*>(tmem_slot + 2);   // [0] = first block, [1] = end (exclusive, in elements)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int g = p.g;
  const int pos_per_tile = BW_M / g;   // MODE_DQ: positions per row tile
  const int pos_per_blk = BN / g;      // MODE_DK/DV: positions per streamed query block

  if (threadIdx.x == 0) {
    mbar_init(f_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&y_full[i], 1);
      mbar_init(&y_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 256);
      mbar_init(&t_full[i], 256);
      mbar_init(&t_free[i], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    range_smem[0] = INT_MAX;
    range_smem[1] = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tm_f1);
    tma_prefetch_desc(&tm_y1);
    tma_prefetch_desc(&tm_y2);
    if (MODE != MODE_DV) tma_prefetch_desc(&tm_f2);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_acc = tmem_base + L::TMEM_ACC;

  // ---- range of streamed blocks that can contain a visible (query, key) pair
  __shared__ int s_ext, s_any;
  if (threadIdx.x == 0) {
    s_ext = (MODE == MODE_DQ) ? INT_MIN : INT_MAX;
    s_any = 0;
  }
  __syncthreads();
  if (MODE == MODE_DQ) {
    const int p0 = tile * pos_per_tile;
    int qmax = INT_MIN;
    bool any = false;
    for (int i = threadIdx.x; i < pos_per_tile; i += blockDim.x) {
      const int pos = p0 + i;
      if (pos < p.Sq && p.q_valid[(long long)b * p.Sq + pos]) {
        qmax = max(qmax, p.q_blk[(long long)b * p.Sq + pos]);
        any = true;
      }
    }
    if (any) {
      atomicMax(&s_ext, qmax);
      atomicOr(&s_any, 1);
    }
    __syncthreads();
    int last = -1;
    if (s_any) {
      const int qm = s_ext;
#pragma unroll 8
      for (int j = threadIdx.x; j < p.Sk; j += blockDim.x) {
        const int kbj = p.k_blk[(long long)b * p.Sk + j];
        const int kvj = p.k_valid[(long long)b * p.Sk + j];
        if (kvj && kbj <= qm) last = max(last, j);
      }
    }
    if (last >= 0) atomicMax(&range_smem[1], last + 1);
    if (threadIdx.x == 0) range_smem[0] = 0;
  } else {
    const int k0 = tile * BW_M;
    int kmin = INT_MAX;
    bool any = false;
    for (int i = threadIdx.x; i < BW_M; i += blockDim.x) {
      const int key = k0 + i;
      if (key < p.Sk && p.k_valid[(long long)b * p.Sk + key]) {
        kmin = min(kmin, p.k_blk[(long long)b * p.Sk + key]);
        any = true;
      }
    }
    if (any) {
      atomicMin(&s_ext, kmin);
      atomicOr(&s_any, 1);
    }
    __syncthreads();
    int first = INT_MAX, last = -1;
    if (s_any) {
      const int km = s_ext;
#pragma unroll 8
      for (int i = threadIdx.x; i < p.Sq; i += blockDim.x) {
        const int qbi = p.q_blk[(long long)b * p.Sq + i];
        const int qvi = p.q_valid[(long long)b * p.Sq + i];
        if (qvi && qbi >= km) {
          first = min(first, i);
          last = max(last, i);
        }
      }
    }
    if (last >= 0) {
      atomicMin(&range_smem[0], first);
      atomicMax(&range_smem[1], last + 1);
    }
  }
  __syncthreads();
  int blk0, nblk;
  if (MODE == MODE_DQ) {
    blk0 = 0;
    nblk = max(1, (range_smem[1] + BN - 1) / BN);
  } else {
    const int first = range_smem[0] == INT_MAX ? 0 : range_smem[0];
    blk0 = first / pos_per_blk;
    const int endb = (range_smem[1] + pos_per_blk - 1) / pos_per_blk;
    nblk = max(1, endb - blk0);
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      mbar_expect_tx(f_full, L::NF * L::F_BYTES);
#pragma unroll
      for (int c = 0; c < L::NCHUNK; ++c) {
        if (MODE == MODE_DQ) {
          tma_load_4d(sF + c * (BW_M * 128), &tm_f1, f_full, c * 64, kvh * g, tile * pos_per_tile, b);
          tma_load_4d(sF + L::F_BYTES + c * (BW_M * 128), &tm_f2, f_full, c * 64, kvh * g, tile * pos_per_tile, b);
        } else {
          tma_load_4d(sF + c * (BW_M * 128), &tm_f1, f_full, c * 64, kvh, tile * BW_M, b);
          if (MODE == MODE_DK)
            tma_load_4d(sF + L::F_BYTES + c * (BW_M * 128), &tm_f2, f_full, c * 64, kvh, tile * BW_M, b);
        }
      }
      for (int j = 0; j < nblk; ++j) {
        const int slot = j & 1, u = j >> 1;
        mbar_wait(&y_empty[slot], (u & 1) ^ 1, abort_flag, p.status, KID_ATTN_BWD, 1, j);
        uint8_t* y1 = sY + slot * L::STAGE_BYTES;
        uint8_t* y2 = y1 + L::Y_BYTES;
        mbar_expect_tx(&y_full[slot], L::STAGE_BYTES);
        const int blk = blk0 + j;
#pragma unroll
        for (int c = 0; c < L::NCHUNK; ++c) {
          if (MODE == MODE_DQ) {
            tma_load_4d(y1 + c * (BN * 128), &tm_y1, &y_full[slot], c * 64, kvh, blk * BN, b);
            tma_load_4d(y2 + c * (BN * 128), &tm_y2, &y_full[slot], c * 64, kvh, blk * BN, b);
          } else {
            tma_load_4d(y1 + c * (BN * 128), &tm_y1, &y_full[slot], c * 64, kvh * g, blk * pos_per_blk, b);
            tma_load_4d(y2 + c * (BN * 128), &tm_y2, &y_full[slot], c * 64, kvh * g, blk * pos_per_blk, b);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc_bf16(BW_M, BN, 0, 0);
      const uint32_t idesc_acc = make_idesc_bf16(BW_M, p.Dmma, 0, 1);
      const int ksteps = p.Dmma / 16;
      const uint32_t f_addr = smem_u32(sF);
      auto issue_scores = [&](int j) {
        const int slot = j & 1, u = j >> 1;
        mbar_wait(&y_full[slot], u & 1, abort_flag, p.status, KID_ATTN_BWD, 2, j);
        mbar_wait(&s_free[slot], (u & 1) ^ 1, abort_flag, p.status, KID_ATTN_BWD, 3, j);
        tc_fence_after();
        const uint32_t y_addr = smem_u32(sY + slot * L::STAGE_BYTES);
#pragma unroll
        for (int s = 0; s < L::NS; ++s) {
          const uint32_t fa = f_addr + s * L::F_BYTES;
          const uint32_t ya = y_addr + s * L::Y_BYTES;
          const uint32_t d = tmem_base + slot * (L::NS * BN) + s * BN;
          for (int kk = 0; kk < ksteps; ++kk) {
            const int c = kk >> 2, w = kk & 3;
            uint64_t ad = make_smem_desc(fa + c * (BW_M * 128) + w * 32, 16, 1024);
            uint64_t bd = make_smem_desc(ya + c * (BN * 128) + w * 32, 16, 1024);
            umma_ss(d, ad, bd, idesc_s, kk != 0 ? 1u : 0u);
          }
        }
        umma_commit(&s_full[slot]);
      };
      mbar_wait(f_full, 0, abort_flag, p.status, KID_ATTN_BWD, 4, 0);
      issue_scores(0);
      for (int j = 0; j < nblk; ++j) {
        const int slot = j & 1, u = j >> 1;
        if (j + 1 < nblk) issue_scores(j + 1);
        mbar_wait(&t_full[slot], u & 1, abort_flag, p.status, KID_ATTN_BWD, 5, j);
        tc_fence_after();
        const uint32_t t_addr = smem_u32(sT + slot * L::T_BYTES);
        const uint32_t yb = smem_u32(sY + slot * L::STAGE_BYTES + (MODE == MODE_DV ? L::Y_BYTES : 0));
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          uint64_t ad = make_smem_desc(t_addr + (kk >> 2) * (BW_M * 128) + (kk & 3) * 32, 16, 1024);
          uint64_t bd = make_smem_desc(yb + kk * 2048, BN * 128, 1024);
          umma_ss(tmem_acc, ad, bd, idesc_acc, (j | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&y_empty[slot]);
        umma_commit(&t_free[slot]);
      }
      umma_commit(acc_full);
    }
  } else {
    // ------------------------------------------------------------------ elementwise + epilogue
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;            // which half of a block's columns this thread handles
    const int row = quad * 32 + lane;
    const int st = threadIdx.x - 64;             // 0..255
    int* kmm = reinterpret_cast<int*>(smem + L::OFF_KMM);
    constexpr int HB = BN / 2;                   // columns per thread per block
    constexpr int PIECE = HB >= 32 ? 32 : 16;    // columns per TMEM read
    constexpr int NP = HB / PIECE;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    float* meta_lse = reinterpret_cast<float*>(meta_blk + 2 * BN);
    float* meta_delta = meta_lse + 2 * BN;
    const float LOG2E = 1.4426950408889634f;

    // per-row constants
    bool row_ok;
    int row_blk = 0;
    float row_lse2 = 0.f, row_delta = 0.f;
    long long out_off;
    bool row_in;
    if (MODE == MODE_DQ) {
      const int pos = tile * pos_per_tile + row / g;
      const int head = kvh * g + row % g;
      row_in = pos < p.Sq;
      row_ok = row_in && p.q_valid[(long long)b * p.Sq + pos] != 0;
      if (row_ok) {
        row_blk = p.q_blk[(long long)b * p.Sq + pos];
        row_lse2 = p.lse[((long long)b * p.H + head) * p.Sq + pos] * LOG2E;
        row_delta = p.delta[((long long)b * p.H + head) * p.Sq + pos];
      }
      out_off = (((long long)b * p.Sq + pos) * p.H + head) * p.D;
    } else {
      const int key = tile * BW_M + row;
      row_in = key < p.Sk;
      row_ok = row_in && p.k_valid[(long long)b * p.Sk + key] != 0;
      if (row_ok) row_blk = p.k_blk[(long long)b * p.Sk + key];
      out_off = (((long long)b * p.Sk + key) * p.Hkv + kvh) * p.D;
    }

    for (int j = 0; j < nblk; ++j) {
      const int slot = j & 1, u = j >> 1;
      const int blk = blk0 + j;
      if (st < BN) {
        if (MODE == MODE_DQ) {
          const int key = blk * BN + st;
          int kb = INT_MAX;
          if (key < p.Sk) {
            const int kbv = p.k_blk[(long long)b * p.Sk + key];
            const int kvv = p.k_valid[(long long)b * p.Sk + key];
            kb = kvv ? kbv : INT_MAX;
          }
          meta_blk[slot * BN + st] = kb;
          const int mn = __reduce_min_sync(0xffffffffu, kb), mxk = __reduce_max_sync(0xffffffffu, kb);
          if (lane == 0) {
            kmm[(slot * (BN / 32) + st / 32) * 2 + 0] = mn;
            kmm[(slot * (BN / 32) + st / 32) * 2 + 1] = mxk;
          }
        } else {
          const int pos = blk * pos_per_blk + st / g;
          const int head = kvh * g + st % g;
          int qb = INT_MIN;
          float l2 = INFINITY, dl = 0.f;
          if (pos < p.Sq) {
            // four independent loads; the validity only selects afterwards
            const int qvv = p.q_valid[(long long)b * p.Sq + pos];
            const int qbv = p.q_blk[(long long)b * p.Sq + pos];
            const float lv = p.lse[((long long)b * p.H + head) * p.Sq + pos];
            const float dv2 = p.delta[((long long)b * p.H + head) * p.Sq + pos];
            if (qvv) {
              qb = qbv;
              l2 = lv * LOG2E;
              dl = dv2;
            }
          }
          meta_blk[slot * BN + st] = qb;
          meta_lse[slot * BN + st] = l2;
          meta_delta[slot * BN + st] = dl;
          const int mn = __reduce_min_sync(0xffffffffu, qb), mxk = __reduce_max_sync(0xffffffffu, qb);
          if (lane == 0) {
            kmm[(slot * (BN / 32) + st / 32) * 2 + 0] = mn;
            kmm[(slot * (BN / 32) + st / 32) * 2 + 1] = mxk;
          }
        }
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      const int* mb = meta_blk + slot * BN;
      const float* ml = meta_lse + slot * BN;
      const float* md = meta_delta + slot * BN;
      mbar_wait(&s_full[slot], u & 1, abort_flag, p.status, KID_ATTN_BWD, 6, j);
      tc_fence_after();
      if (j >= 2) mbar_wait(&t_free[slot], (u - 1) & 1, abort_flag, p.status, KID_ATTN_BWD, 7, j);
      const uint32_t s_addr = tmem_base + slot * (L::NS * BN) + lane_off;
      uint8_t* trow = sT + slot * L::T_BYTES + row * 128;
#pragma unroll
      for (int c = 0; c < NP; ++c) {
        const int col0 = half * HB + c * PIECE;
        uint32_t rs[PIECE];
        uint32_t rd[PIECE];
        __syncwarp();
        if (PIECE == 32) {
          tmem_ld_x32(s_addr + col0, rs);
          if (MODE != MODE_DV) tmem_ld_x32(s_addr + BN + col0, rd);
        } else {
          tmem_ld_x16(s_addr + col0, rs);
          if (MODE != MODE_DV) tmem_ld_x16(s_addr + BN + col0, rd);
        }
        // visibility of this group of columns for this row: 2 = all, 0 = none, 1 = test each
        const int gi = (slot * (BN / 32) + col0 / 32) * 2;
        const int gmin = kmm[gi], gmax = kmm[gi + 1];
        int cls;
        if (MODE == MODE_DQ) cls = (!row_ok || gmin > row_blk) ? 0 : (gmax <= row_blk ? 2 : 1);
        else cls = (!row_ok || gmax < row_blk) ? 0 : (gmin >= row_blk ? 2 : 1);
        tmem_wait_ld();
        uint32_t packed[PIECE / 2];
        if (cls == 0) {
#pragma unroll
          for (int e = 0; e < PIECE / 2; ++e) packed[e] = 0u;
        } else {
#pragma unroll
          for (int e = 0; e < PIECE; e += 2) {
            float v[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int col = col0 + e + h;
              bool vis = true;
              float l2, dl;
              if (MODE == MODE_DQ) {
                if (cls == 1) vis = mb[col] <= row_blk;
                l2 = row_lse2;
                dl = row_delta;
              } else {
                if (cls == 1) vis = row_blk <= mb[col];
                l2 = ml[col];
                dl = md[col];
              }
              float pr = vis ? bw_exp2(fmaf(__uint_as_float(rs[e + h]), p.scale_log2, -l2)) : 0.f;
              if (MODE == MODE_DV) v[h] = pr;
              else v[h] = pr * (__uint_as_float(rd[e + h]) - dl) * p.scale;
            }
            packed[e >> 1] = pack_bf16(v[0], v[1]);
          }
        }
        const int chunk = col0 / 64;
        const int unit0 = (col0 % 64) / 8;
#pragma unroll
        for (int q4 = 0; q4 < PIECE / 8; ++q4) {
          const int unit = (unit0 + q4) ^ (row & 7);
          uint4 val = make_uint4(packed[q4 * 4 + 0], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
          *reinterpret_cast<uint4*>(trow + chunk * (BW_M * 128) + unit * 16) = val;
        }
      }
      tc_fence_before();
      mbar_arrive(&s_free[slot]);
      fence_async_smem();
      mbar_arrive(&t_full[slot]);
    }

    mbar_wait(acc_full, 0, abort_flag, p.status, KID_ATTN_BWD, 9, 0);
    tc_fence_after();
    __nv_bfloat16* orow = p.out + out_off;
    const int n16 = p.Dmma / 16;
    const int a_lo = half ? (n16 + 1) / 2 : 0, a_hi = half ? n16 : (n16 + 1) / 2;
#pragma unroll 1
    for (int c = a_lo; c < a_hi; ++c) {
      uint32_t r[16];
      __syncwarp();
      tmem_ld_x16(tmem_acc + lane_off + c * 16, r);
      tmem_wait_ld();
      if (row_in) {
#pragma unroll
        for (int h8 = 0; h8 < 2; ++h8) {
          const int col = c * 16 + h8 * 8;
          if (col < p.D) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r[h8 * 8 + 0]), __uint_as_float(r[h8 * 8 + 1]));
            o.y = pack_bf16(__uint_as_float(r[h8 * 8 + 2]), __uint_as_float(r[h8 * 8 + 3]));
            o.z = pack_bf16(__uint_as_float(r[h8 * 8 + 4]), __uint_as_float(r[h8 * 8 + 5]));
            o.w = pack_bf16(__uint_as_float(r[h8 * 8 + 6]), __uint_as_float(r[h8 * 8 + 7]));
            *reinterpret_cast<uint4*>(orow + col) = o;
          }
        }
      }
    }
    tc_fence_before();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[b,h,s] = sum_d O[b,s,h,d] * dO[b,s,h,d]; one warp per (b,s,h) row.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int B, int S, int H, int D) {
  const long long rowi = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (rowi >= (long long)B * S * H) return;
  const __nv_bfloat16* a = o + rowi * D;
  const __nv_bfloat16* c = d_o + rowi * D;
  float acc = 0.f;
  for (int i = lane * 8; i < D; i += 256) {
    uint4 ua = *reinterpret_cast<const uint4*>(a + i);
    uint4 uc = *reinterpret_cast<const uint4*>(c + i);
    float2 x, y;
    x = unpack_bf16(ua.x); y = unpack_bf16(uc.x); acc += x.x * y.x + x.y * y.y;
    x = unpack_bf16(ua.y); y = unpack_bf16(uc.y); acc += x.x * y.x + x.y * y.y;
    x = unpack_bf16(ua.z); y = unpack_bf16(uc.z); acc += x.x * y.x + x.y * y.y;
    x = unpack_bf16(ua.w); y = unpack_bf16(uc.w); acc += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const int h = int(rowi % H);
    const long long bs = rowi / H;
    const int s = int(bs % S);
    const int b = int(bs / S);
    delta[((long long)b * H + h) * S + s] = acc;
  }
}

static int make_map4b(CUtensorMap* m, const void* base, int D, int Hx, int S, int B, long long sh, long long ss,
                      long long sb, int box_h, int box_s) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hx, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)sh * 2, (uint64_t)ss * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, (uint32_t)box_h, (uint32_t)box_s, 1};
  return make_tmap_bf16(m, base, 4, dims, strides, box);
}

struct Strides {
  long long sb, ss, sh;
};

template <int MODE, int DPAD, int BN>
static int launch_bwd(const void* q, Strides qs, const void* k, Strides ks, const void* v, Strides vs, const void* d_o,
                      const BwdParams& p, cudaStream_t stream) {
  using L = BwdSmem<MODE, DPAD, BN>;
  static bool configured = false;
  auto kern = attn_bwd_kernel<MODE, DPAD, BN>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int g = p.g;
  if (MODE != MODE_DQ && (BN % g)) return -20;
  CUtensorMap f1, f2, y1, y2;
  const Strides dos = {(long long)p.Sq * p.H * p.D, (long long)p.H * p.D, (long long)p.D};
  int r;
  if (MODE == MODE_DQ) {
    r = make_map4b(&f1, q, p.D, p.H, p.Sq, p.B, qs.sh, qs.ss, qs.sb, g, BW_M / g);
    if (r) return 1000 + r;
    r = make_map4b(&f2, d_o, p.D, p.H, p.Sq, p.B, dos.sh, dos.ss, dos.sb, g, BW_M / g);
    if (r) return 2000 + r;
    r = make_map4b(&y1, k, p.D, p.Hkv, p.Sk, p.B, ks.sh, ks.ss, ks.sb, 1, BN);
    if (r) return 3000 + r;
    r = make_map4b(&y2, v, p.D, p.Hkv, p.Sk, p.B, vs.sh, vs.ss, vs.sb, 1, BN);
    if (r) return 4000 + r;
  } else {
    r = make_map4b(&f1, k, p.D, p.Hkv, p.Sk, p.B, ks.sh, ks.ss, ks.sb, 1, BW_M);
    if (r) return 1000 + r;
    r = make_map4b(&f2, v, p.D, p.Hkv, p.Sk, p.B, vs.sh, vs.ss, vs.sb, 1, BW_M);
    if (r) return 2000 + r;
    r = make_map4b(&y1, q, p.D, p.H, p.Sq, p.B, qs.sh, qs.ss, qs.sb, g, BN / g);
    if (r) return 3000 + r;
    r = make_map4b(&y2, d_o, p.D, p.H, p.Sq, p.B, dos.sh, dos.ss, dos.sb, g, BN / g);
    if (r) return 4000 + r;
  }
  dim3 grid;
  if (MODE == MODE_DQ) grid = dim3((p.Sq + BW_M / g - 1) / (BW_M / g), p.Hkv, p.B);
  else grid = dim3((p.Sk + BW_M - 1) / BW_M, p.Hkv, p.B);
  kern<<<grid, 320, L::TOTAL, stream>>>(f1, f2, y1, y2, p);
  return (int)cudaGetLastError();
}

}  // namespace otb

using namespace otb;

// q (B,Sq,H,D), k/v (B,Sk,Hkv,D) with element strides; o, do: (B,Sq,H,D) contiguous; lse (B,H,Sq);
// delta: scratch (B,H,Sq) fp32; dq (B,Sq,H,D), dk/dv (B,Sk,Hkv,D) contiguous outputs.
extern "C" int otb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, float* delta, void* dq, void* dk, void* dv, const int* q_blk,
                            const int* k_blk, const unsigned char* q_valid, const unsigned char* k_valid, int B,
                            int Sq, int Sk, int H, int Hkv, int D, long long q_sb, long long q_ss, long long q_sh,
                            long long k_sb, long long k_ss, long long k_sh, long long v_sb, long long v_ss,
                            long long v_sh, float scale, void* status, cudaStream_t stream) {
  if (B <= 0 || Sq <= 0 || Sk <= 0 || H <= 0 || Hkv <= 0 || H % Hkv) return -2;
  const int g = H / Hkv;
  if (g > 32 || (32 % g)) return -3;
  if (D % 8 || D > 256 || D < 16) return -4;
  const long long strides[9] = {q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh};
  for (int i = 0; i < 9; ++i)
    if (strides[i] % 8) return -5;
  {
    const long long rows = (long long)B * Sq * H;
    const int threads = 256;
    const long long blocks = (rows * 32 + threads - 1) / threads;
    attn_delta_kernel<<<(unsigned)blocks, threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(o),
                                                               static_cast<const __nv_bfloat16*>(d_o), delta, B, Sq,
                                                               H, D);
  }
  BwdParams p;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.H = H; p.Hkv = Hkv; p.D = D; p.g = g;
  p.Dmma = (D + 15) / 16 * 16;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.q_blk = q_blk; p.k_blk = k_blk; p.q_valid = q_valid; p.k_valid = k_valid;
  p.lse = lse; p.delta = delta;
  p.status = static_cast<KernelStatus*>(status);
  const Strides qs = {q_sb, q_ss, q_sh}, ks = {k_sb, k_ss, k_sh}, vs = {v_sb, v_ss, v_sh};
  const int dpad = D <= 64 ? 64 : (D <= 128 ? 128 : 256);
  int r = 0;
#define RUN3(DP, BN_QK, BN_V)                                                          \
  p.out = static_cast<__nv_bfloat16*>(dq);                                             \
  r = launch_bwd<MODE_DQ, DP, BN_QK>(q, qs, k, ks, v, vs, d_o, p, stream);              \
  if (r) return r;                                                                     \
  p.out = static_cast<__nv_bfloat16*>(dk);                                             \
  r = launch_bwd<MODE_DK, DP, BN_QK>(q, qs, k, ks, v, vs, d_o, p, stream);              \
  if (r) return 100000 + r;                                                            \
  p.out = static_cast<__nv_bfloat16*>(dv);                                             \
  r = launch_bwd<MODE_DV, DP, BN_V>(q, qs, k, ks, v, vs, d_o, p, stream);               \
  if (r) return 200000 + r;
  if (dpad == 64) { RUN3(64, 64, 128) }
  else if (dpad == 128) { RUN3(128, 64, 64) }
  else { RUN3(256, 32, 64) }
#undef RUN3
  return 0;
}
