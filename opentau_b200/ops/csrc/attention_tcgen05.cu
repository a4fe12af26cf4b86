// Block-causal flash attention forward for sm_100a: TMA-fed, S = Q K^T and O += P V on tcgen05 with
// both accumulators in tensor memory, online softmax by 128 threads that each own one TMEM lane.
//
// Mask rule (same as the dense reference): query i sees key j iff q_valid[i] && k_valid[j] &&
// k_blk[j] <= q_blk[i].  Cached cross-attention keys carry k_blk = INT_MIN.  Rows that see no key
// produce O = 0 and LSE = 0.
//
// Work decomposition: one CTA per (batch, kv head, tile of 128 "rows"), where a row is a
// (query position, query head of the GQA group) pair: 128 rows = (128/g) positions x g heads, so one
// K/V tile load serves every head of the group (MQA: g = 8 -> K/V traffic / 8).
//
// Warps: 0 = TMA producer, 1 = MMA issuer (owns TMEM), 2..5 = softmax / correction / epilogue.
// Per KV block j:  MMA issues S[j+1] = Q K_{j+1}^T early, softmax turns S[j] into bf16 P in shared
// memory (128B-swizzled, K-major), MMA issues O += P V_j.  O is rescaled lazily: only when the running
// row maximum grew by more than 2^8 since the maximum in use, so the common case touches O never.
#include "common.cuh"
#include <limits.h>

namespace otb {

constexpr unsigned KID_ATTN = 2;
constexpr int ATT_M = 128;

struct AttnParams {
  int B, Sq, Sk, H, Hkv, D, Dmma, g;
  float scale_log2;                 // scale * log2(e)
  const int* q_blk;                 // (B, Sq)
  const int* k_blk;                 // (B, Sk)
  const unsigned char* q_valid;     // (B, Sq)
  const unsigned char* k_valid;     // (B, Sk)
  __nv_bfloat16* o;                 // (B, Sq, H, D) contiguous
  float* lse;                       // (B, H, Sq)
  // split-KV (few query tiles, many keys: a denoising step against a cached prefix): CTA (tile, split) covers its
  // share of the key blocks and leaves an unnormalised partial; attn_combine_kernel merges the partials
  int skip_reach;                   // visit every key block: skip the prologue scan for the last reachable key
  int nsplit;                       // 1: write o / lse directly
  float* part_o;                    // (nsplit, B, Sq, H, D) fp32, accumulators expressed against part m
  float2* part_ml;                  // (nsplit, B, H, Sq): (running maximum in log2 units, row sum)
  KernelStatus* status;
};

template <int DPAD, int BN>
struct AttnSmem {
  static constexpr int NCHUNK = DPAD / 64;
  static constexpr int Q_BYTES = ATT_M * DPAD * 2;
  static constexpr int KV_TILE = BN * DPAD * 2;        // one K or V tile
  static constexpr int STAGE_BYTES = 2 * KV_TILE;      // K and V of one block
  static constexpr int P_BYTES = ATT_M * BN * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = Q_BYTES;
  static constexpr int OFF_P = OFF_KV + 2 * STAGE_BYTES;
  static constexpr int OFF_META = OFF_P + 2 * P_BYTES;  // int kmeta[2][BN]
  static constexpr int OFF_RED = OFF_META + 2 * BN * 4;  // float red[2][128]: row max / row sum exchange
  static constexpr int OFF_KMM = OFF_RED + 2 * ATT_M * 4;  // int kmm[2][BN/32][2]: min / max block id per 32 keys
  static constexpr int OFF_BAR = OFF_KMM + 2 * (BN / 32) * 2 * 4;
  static constexpr int NBAR = 16;
  static constexpr int USED = OFF_BAR + NBAR * 8 + 32;
  // room for rounding the base up to 1024 bytes (the kernel has no static shared memory, so the base normally is
  // aligned already); capped at the 227 KB a CTA may own, and checked at run time
  static constexpr int TOTAL = USED + 1024 <= 232448 ? USED + 1024 : 232448;
  static_assert(USED <= 232448, "shared memory budget");
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int DPAD, int BN>
__global__ void __launch_bounds__(320, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                const __grid_constant__ CUtensorMap tma_v, AttnParams p) {
  using L = AttnSmem<DPAD, BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem + L::OFF_Q;
  uint8_t* sKV = smem + L::OFF_KV;
  uint8_t* sP = smem + L::OFF_P;
  int* kmeta = reinterpret_cast<int*>(smem + L::OFF_META);
  float* red = reinterpret_cast<float*>(smem + L::OFF_RED);
  int* kmm = reinterpret_cast<int*>(smem + L::OFF_KMM);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;     // [2]
  uint64_t* s_free = bars + 7;     // [2]
  uint64_t* p_full = bars + 9;     // [2]
  uint64_t* p_free = bars + 11;    // [2]
  uint64_t* o_full = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* kv_end_smem = reinterpret_cast<int*>(tmem_slot + 2);
  int& s_qmax = *reinterpret_cast<int*>(tmem_slot + 3);
  int& s_any = *reinterpret_cast<int*>(tmem_slot + 4);
  if ((int)(smem - smem_raw) + L::USED > L::TOTAL) {   // base less aligned than assumed: refuse instead of overrunning
    if (threadIdx.x == 0) report_timeout(p.status, KID_ATTN, 99, (unsigned)(smem - smem_raw));
    return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x / p.nsplit, split = blockIdx.x % p.nsplit, kvh = blockIdx.y, b = blockIdx.z;
  const int g = p.g;
  const int pos_per_tile = ATT_M / g;
  const int p0 = tile * pos_per_tile;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 256);
      mbar_init(&p_full[i], 256);
      mbar_init(&p_free[i], 1);
    }
    mbar_init(o_full, 1);
    *abort_flag = 0;
    *kv_end_smem = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;            // two buffers of BN columns
  const uint32_t tmem_O = tmem_base + 2 * BN;   // Dmma columns
  pdl_launch_dependents();                      // after the TMEM allocation (see common.cuh)
  pdl_wait();                                   // q / k / v and the masks come from the preceding kernels

  // ---- how many keys can this tile reach?  1 + the last key index j that is valid and has
  //      k_blk[j] <= the largest valid q_blk in the tile (no monotonicity assumed).  With split keys the scan is
  //      skipped: the few tiles of such a launch reach (almost) every key, blocks without a visible key cost one
  //      masked pass, and the scan itself is a serial prologue of two dependent global reads per key.  The same holds
  //      for a launch with ONE query tile per (batch, kv head): a short suffix attending to a cached prefix.
  if (p.skip_reach) {
    if (threadIdx.x == 0) *kv_end_smem = p.Sk;
    __syncthreads();
  } else {
    int qmax = INT_MIN;
    bool any_q = false;
    for (int i = threadIdx.x; i < pos_per_tile; i += blockDim.x) {
      int pos = p0 + i;
      if (pos < p.Sq && p.q_valid[(long long)b * p.Sq + pos]) {
        qmax = max(qmax, p.q_blk[(long long)b * p.Sq + pos]);
        any_q = true;
      }
    }
    // block-wide max of qmax (values) through shared atomics on a small scratch word
    if (threadIdx.x == 0) {
      s_qmax = INT_MIN;
      s_any = 0;
    }
    __syncthreads();
    if (any_q) {
      atomicMax(&s_qmax, qmax);
      atomicOr(&s_any, 1);
    }
    __syncthreads();
    int last = -1;
    if (s_any) {
      const int qm = s_qmax;
      // both loads are unconditional and the loop is unrolled, so several keys are in flight per thread
#pragma unroll 8
      for (int j = threadIdx.x; j < p.Sk; j += blockDim.x) {
        const int kbj = p.k_blk[(long long)b * p.Sk + j];
        const int kvj = p.k_valid[(long long)b * p.Sk + j];
        if (kvj && kbj <= qm) last = max(last, j);
      }
    }
    if (last >= 0) atomicMax(kv_end_smem, last + 1);
    __syncthreads();
  }
  const int kv_end = *kv_end_smem;
  const int nblk_all = max(1, (kv_end + BN - 1) / BN);
  // this CTA's key blocks [jb0, jb0 + nblk).  A split beyond the reachable keys still runs one block: every key in
  // it is invisible to the tile, so it contributes a zero row sum that the combine step ignores.
  const int per_split = (nblk_all + p.nsplit - 1) / p.nsplit;
  const int jb0 = split * per_split;
  const int nblk = max(1, min(nblk_all, jb0 + per_split) - jb0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int c = 0; c < L::NCHUNK; ++c)
        tma_load_4d(sQ + c * (ATT_M * 128), &tma_q, q_full, c * 64, kvh * g, p0, b);
      for (int j = 0; j < nblk; ++j) {
        const int slot = j & 1, u = j >> 1;
        mbar_wait(&kv_empty[slot], (u & 1) ^ 1, abort_flag, p.status, KID_ATTN, 1, j);
        uint8_t* sk = sKV + slot * L::STAGE_BYTES;
        uint8_t* sv = sk + L::KV_TILE;
        mbar_expect_tx(&kv_full[slot], L::STAGE_BYTES);
#pragma unroll
        for (int c = 0; c < L::NCHUNK; ++c) {
          tma_load_4d(sk + c * (BN * 128), &tma_k, &kv_full[slot], c * 64, kvh, (jb0 + j) * BN, b);
          tma_load_4d(sv + c * (BN * 128), &tma_v, &kv_full[slot], c * 64, kvh, (jb0 + j) * BN, b);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_qk = make_idesc_bf16(ATT_M, BN, 0, 0);
      const uint32_t idesc_pv = make_idesc_bf16(ATT_M, p.Dmma, 0, 1);
      const int ksteps_qk = p.Dmma / 16;
      const uint32_t q_addr = smem_u32(sQ);
      auto issue_qk = [&](int j) {
        const int slot = j & 1, u = j >> 1;
        mbar_wait(&kv_full[slot], u & 1, abort_flag, p.status, KID_ATTN, 2, j);
        mbar_wait(&s_free[slot], (u & 1) ^ 1, abort_flag, p.status, KID_ATTN, 3, j);
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sKV + slot * L::STAGE_BYTES);
        for (int kk = 0; kk < ksteps_qk; ++kk) {
          const int c = kk >> 2, w = kk & 3;
          uint64_t ad = make_smem_desc(q_addr + c * (ATT_M * 128) + w * 32, 16, 1024);
          uint64_t bd = make_smem_desc(k_addr + c * (BN * 128) + w * 32, 16, 1024);
          umma_ss(tmem_S + slot * BN, ad, bd, idesc_qk, kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[slot]);
      };
      mbar_wait(q_full, 0, abort_flag, p.status, KID_ATTN, 4, 0);
      issue_qk(0);
      for (int j = 0; j < nblk; ++j) {
        const int slot = j & 1, u = j >> 1;
        if (j + 1 < nblk) issue_qk(j + 1);
        mbar_wait(&p_full[slot], u & 1, abort_flag, p.status, KID_ATTN, 5, j);
        tc_fence_after();
        const uint32_t p_addr = smem_u32(sP + slot * L::P_BYTES);
        const uint32_t v_addr = smem_u32(sKV + slot * L::STAGE_BYTES + L::KV_TILE);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          uint64_t ad = make_smem_desc(p_addr + (kk >> 2) * (ATT_M * 128) + (kk & 3) * 32, 16, 1024);
          uint64_t bd = make_smem_desc(v_addr + kk * 2048, BN * 128, 1024);
          umma_ss(tmem_O, ad, bd, idesc_pv, (j | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&kv_empty[slot]);
        umma_commit(&p_free[slot]);
      }
      umma_commit(o_full);
    }
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    // Eight warps: two per TMEM lane quadrant.  Both threads of a pair own the same row (TMEM lane) and split the
    // columns of S, of P and of O between them; the row maximum (per block) and the row sum (once, at the end) are
    // exchanged through shared memory.  The scores of a block are read from TMEM once and stay in registers.
    // Masking is decided per 32 keys from the min / max block id of those keys: fully visible and fully hidden
    // groups take paths without per-element tests.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;            // 0: first half of the columns, 1: second half
    const int row = quad * 32 + lane;            // TMEM lane owned by this thread
    const int st = threadIdx.x - 64;             // 0..255 index among softmax threads
    const int pos = p0 + row / g;
    const int head = kvh * g + row % g;
    const bool row_in = pos < p.Sq;
    const bool q_ok = row_in && p.q_valid[(long long)b * p.Sq + pos] != 0;
    const int qb = q_ok ? p.q_blk[(long long)b * p.Sq + pos] : INT_MIN;
    const uint32_t lane_off = uint32_t(quad * 32) << 16;
    constexpr int HB = BN / 2;                   // columns per thread
    constexpr int NCH = HB / 32;                 // 32-column groups per thread
    const int c0 = half * HB;
    float m_used = -INFINITY;   // maximum the accumulators are currently expressed against
    float l = 0.f;              // this thread's part of the row sum
    const float scale = p.scale_log2;
    const int n16 = p.Dmma / 16;
    const int o_lo = half ? (n16 + 1) / 2 : 0, o_hi = half ? n16 : (n16 + 1) / 2;   // this thread's O column groups

    auto load_meta = [&](int jj) -> int {
      const int key = (jb0 + jj) * BN + st;
      if (st >= BN || key >= p.Sk) return INT_MAX;
      const int kbv = p.k_blk[(long long)b * p.Sk + key];
      const int kvv = p.k_valid[(long long)b * p.Sk + key];
      return kvv ? kbv : INT_MAX;
    };
    int kb_next = load_meta(0);
    for (int j = 0; j < nblk; ++j) {
      const int slot = j & 1, u = j >> 1;
      if (st < BN) {                              // whole warps: st < BN covers warps 0 .. BN/32-1 of the group
        kmeta[slot * BN + st] = kb_next;
        const int mn = __reduce_min_sync(0xffffffffu, kb_next);
        const int mxk = __reduce_max_sync(0xffffffffu, kb_next);
        if (lane == 0) {
          kmm[(slot * (BN / 32) + st / 32) * 2 + 0] = mn;
          kmm[(slot * (BN / 32) + st / 32) * 2 + 1] = mxk;
        }
      }
      kb_next = (j + 1 < nblk) ? load_meta(j + 1) : INT_MAX;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      const int* km = kmeta + slot * BN + c0;
      mbar_wait(&s_full[slot], u & 1, abort_flag, p.status, KID_ATTN, 6, j);
      tc_fence_after();
      const uint32_t s_addr = tmem_S + slot * BN + c0 + lane_off;
      // ---- read this thread's scores once; visibility class per 32 keys: 2 = all, 0 = none, 1 = test each
      uint32_t r[NCH][32];
      int cls[NCH];
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        __syncwarp();
        tmem_ld_x32(s_addr + c * 32, r[c]);
        const int gi = (slot * (BN / 32) + (c0 / 32) + c) * 2;
        const int gmin = kmm[gi], gmax = kmm[gi + 1];
        cls[c] = (!q_ok || gmin > qb) ? 0 : (gmax <= qb ? 2 : 1);
      }
      tmem_wait_ld();
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        if (cls[c] == 2) {
#pragma unroll
          for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(r[c][e]));
        } else if (cls[c] == 1) {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (km[c * 32 + e] <= qb) mx = fmaxf(mx, __uint_as_float(r[c][e]));
        }
      }
      mx *= scale;                                // scale > 0: max commutes with it
      red[half * ATT_M + row] = mx;
      asm volatile("bar.sync 2, 256;" ::: "memory");
      mx = fmaxf(mx, red[(half ^ 1) * ATT_M + row]);
      const float m_new = fmaxf(m_used, mx);
      // lazy rescale decision (warp-uniform because tcgen05.ld/st are warp-collective; both warps of a pair hold
      // the same rows and the same maxima, so they decide alike)
      const bool want = (m_new > m_used + 8.0f) || (m_used == -INFINITY && m_new != -INFINITY);
      const bool any_want = __any_sync(0xffffffffu, want);
      float alpha = 1.f;
      if (want) {
        alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
        m_used = m_new;
      }
      // P buffer `slot` was last read by PV(j-2)
      if (j >= 2) mbar_wait(&p_free[slot], ((u - 1) & 1), abort_flag, p.status, KID_ATTN, 7, j);
      if (any_want && j > 0) {
        // O may only be touched once PV(j-1) has retired
        const int ps = (j - 1) & 1, pu = (j - 1) >> 1;
        mbar_wait(&p_free[ps], pu & 1, abort_flag, p.status, KID_ATTN, 8, j);
        tc_fence_after();
        const uint32_t o_addr = tmem_O + lane_off;
#pragma unroll 1
        for (int c = o_lo; c < o_hi; ++c) {
          uint32_t ro[16];
          __syncwarp();
          tmem_ld_x16(o_addr + c * 16, ro);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 16; ++e) ro[e] = __float_as_uint(__uint_as_float(ro[e]) * alpha);
          tmem_st_x16(o_addr + c * 16, ro);
        }
        tmem_wait_st();
      }
      l *= alpha;
      // ---- probabilities -> bf16 -> swizzled shared memory (A operand of the PV product)
      uint8_t* prow = sP + slot * L::P_BYTES + row * 128;
      float lsum = 0.f;
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        uint32_t packed[16];
        if (cls[c] == 2) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0f = fast_exp2(fmaf(__uint_as_float(r[c][e]), scale, -m_safe));
            const float p1f = fast_exp2(fmaf(__uint_as_float(r[c][e + 1]), scale, -m_safe));
            lsum += p0f + p1f;
            packed[e >> 1] = pack_bf16(p0f, p1f);
          }
        } else if (cls[c] == 1) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0f = km[c * 32 + e] <= qb ? fast_exp2(fmaf(__uint_as_float(r[c][e]), scale, -m_safe)) : 0.f;
            const float p1f =
                km[c * 32 + e + 1] <= qb ? fast_exp2(fmaf(__uint_as_float(r[c][e + 1]), scale, -m_safe)) : 0.f;
            lsum += p0f + p1f;
            packed[e >> 1] = pack_bf16(p0f, p1f);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) packed[e] = 0u;
        }
        // 32 keys = 64 bytes = four 16-byte units; unit index within the 128-byte row is XOR-swizzled
        const int col = c0 + c * 32;
        const int chunk = col / 64;                // 64-key chunk (16 KB apart)
        const int unit0 = (col % 64) / 8;          // first 16-byte unit inside the row
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int unit = (unit0 + q4) ^ (row & 7);
          uint4 val = make_uint4(packed[q4 * 4 + 0], packed[q4 * 4 + 1], packed[q4 * 4 + 2], packed[q4 * 4 + 3]);
          *reinterpret_cast<uint4*>(prow + chunk * (ATT_M * 128) + unit * 16) = val;
        }
      }
      l += lsum;
      // S buffer is free for QK(j+2); P is visible to the tensor core (async proxy)
      tc_fence_before();
      mbar_arrive(&s_free[slot]);
      fence_async_smem();
      mbar_arrive(&p_full[slot]);
    }

    // ---- epilogue: O / l -> bf16 -> global, LSE.  The two threads of a row add their partial sums first.
    asm volatile("bar.sync 1, 256;" ::: "memory");   // every read of `red` from the last block is done
    red[half * ATT_M + row] = l;
    asm volatile("bar.sync 2, 256;" ::: "memory");
    l += red[(half ^ 1) * ATT_M + row];
    mbar_wait(o_full, 0, abort_flag, p.status, KID_ATTN, 9, 0);
    tc_fence_after();
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
    const uint32_t o_addr = tmem_O + lane_off;
    __nv_bfloat16* orow = p.o + (((long long)b * p.Sq + pos) * p.H + head) * p.D;
    float* prow_o = p.nsplit > 1
                        ? p.part_o + ((((long long)split * p.B + b) * p.Sq + pos) * p.H + head) * (long long)p.D
                        : nullptr;
#pragma unroll 1
    for (int c = o_lo; c < o_hi; ++c) {
      uint32_t ro[16];
      __syncwarp();
      tmem_ld_x16(o_addr + c * 16, ro);
      tmem_wait_ld();
      if (row_in && prow_o != nullptr) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int col = c * 16 + q4 * 4;
          if (col < p.D)
            *reinterpret_cast<float4*>(prow_o + col) =
                make_float4(__uint_as_float(ro[q4 * 4 + 0]), __uint_as_float(ro[q4 * 4 + 1]),
                            __uint_as_float(ro[q4 * 4 + 2]), __uint_as_float(ro[q4 * 4 + 3]));
        }
      } else if (row_in) {
#pragma unroll
        for (int h8 = 0; h8 < 2; ++h8) {
          const int col = c * 16 + h8 * 8;
          if (col < p.D) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(ro[h8 * 8 + 0]) * inv_l, __uint_as_float(ro[h8 * 8 + 1]) * inv_l);
            o.y = pack_bf16(__uint_as_float(ro[h8 * 8 + 2]) * inv_l, __uint_as_float(ro[h8 * 8 + 3]) * inv_l);
            o.z = pack_bf16(__uint_as_float(ro[h8 * 8 + 4]) * inv_l, __uint_as_float(ro[h8 * 8 + 5]) * inv_l);
            o.w = pack_bf16(__uint_as_float(ro[h8 * 8 + 6]) * inv_l, __uint_as_float(ro[h8 * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + col) = o;
          }
        }
      }
    }
    if (row_in && half == 0) {
      if (p.nsplit > 1) {
        p.part_ml[(((long long)split * p.B + b) * p.H + head) * p.Sq + pos] = make_float2(m_used, l);
      } else {
        const float lse = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : 0.f;
        p.lse[((long long)b * p.H + head) * p.Sq + pos] = lse;
      }
    }
    tc_fence_before();
  }

  // ---------------------------------------------------------------------- teardown
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

// Merge of the split-KV partials: one warp per (batch, position, head) row.
//   M = max_s m_s over splits with l_s > 0,  L = sum_s l_s 2^(m_s - M),  O = sum_s O_s 2^(m_s - M) / L
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float2* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ o, float* __restrict__ lse, int nsplit, int B, int Sq,
                                    int H, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long rows = (long long)B * Sq * H;
  if (row >= rows) return;
  const int head = int(row % H);
  const long long bp = row / H;                    // b * Sq + pos
  const int pos = int(bp % Sq), b = int(bp / Sq);
  // lane s < nsplit owns split s: (maximum, row sum); the weights travel by shuffle
  float m_s = -INFINITY, l_s = 0.f;
  if (lane < nsplit) {
    const float2 ml = part_ml[(((long long)lane * B + b) * H + head) * Sq + pos];
    l_s = ml.y;
    m_s = ml.y > 0.f ? ml.x : -INFINITY;
  }
  float M = m_s;
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));   // nsplit <= 8
  const float w_s = (m_s == -INFINITY) ? 0.f : fast_exp2(m_s - M);
  float L = l_s * w_s;
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
  M = __shfl_sync(0xffffffffu, M, 0);
  L = __shfl_sync(0xffffffffu, L, 0);
  const float inv = L > 0.f ? 1.f / L : 0.f;
  float w[8];
#pragma unroll
  for (int s = 0; s < 8; ++s) w[s] = __shfl_sync(0xffffffffu, w_s, s) * inv;   // zero for s >= nsplit
  const long long split_stride = (long long)B * Sq * H * D;
  const float* src = part_o + (bp * H + head) * (long long)D;
  for (int c = lane; c < D / 4; c += 32) {
    float4 v[8];
#pragma unroll
    for (int s = 0; s < 8; ++s)
      v[s] = s < nsplit ? *reinterpret_cast<const float4*>(src + s * split_stride + c * 4) : make_float4(0, 0, 0, 0);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      acc.x += v[s].x * w[s]; acc.y += v[s].y * w[s]; acc.z += v[s].z * w[s]; acc.w += v[s].w * w[s];
    }
    uint2 packed = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    *reinterpret_cast<uint2*>(o + row * D + c * 4) = packed;
  }
  if (lane == 0) lse[((long long)b * H + head) * Sq + pos] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : 0.f;
}

// rank-4 bf16 map over a (B, S, Hx, D) tensor with element strides (sb, ss, sh, 1); dims innermost first
static int make_map4(CUtensorMap* m, const void* base, int D, int Hx, int S, int B, long long sh, long long ss,
                     long long sb, int box_h, int box_s) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hx, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)sh * 2, (uint64_t)ss * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, (uint32_t)box_h, (uint32_t)box_s, 1};
  return make_tmap_bf16(m, base, 4, dims, strides, box);
}

template <int DPAD, int BN>
static int launch_attn(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p,
                       cudaStream_t stream) {
  using L = AttnSmem<DPAD, BN>;
  static bool configured = false;
  auto kern = attn_fwd_kernel<DPAD, BN>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int pos_per_tile = ATT_M / p.g;
  dim3 grid(((p.Sq + pos_per_tile - 1) / pos_per_tile) * p.nsplit, p.Hkv, p.B);
  cudaError_t e = launch_pdl(kern, grid, dim3(320), (size_t)L::TOTAL, stream, 0u, tq, tk, tv, p);
  if (e != cudaSuccess || p.nsplit == 1) return (int)e;
  const long long rows = (long long)p.B * p.Sq * p.H;
  e = launch_pdl(attn_combine_kernel, dim3((unsigned)((rows * 32 + 255) / 256)), dim3(256), 0, stream, 0u,
                 (const float*)p.part_o, (const float2*)p.part_ml, p.o, p.lse, p.nsplit, p.B, p.Sq, p.H, p.D);
  return (int)e;
}

}  // namespace otb

using namespace otb;

// q: (B,Sq,H,D) strides (q_sb,q_ss,q_sh,1); k,v: (B,Sk,Hkv,D); o: (B,Sq,H,D) contiguous; lse: (B,H,Sq).
static int attn_fwd_impl(const void* q, const void* k, const void* v, void* o, float* lse, const int* q_blk,
                         const int* k_blk, const unsigned char* q_valid, const unsigned char* k_valid, int B, int Sq,
                         int Sk, int H, int Hkv, int D, long long q_sb, long long q_ss, long long q_sh, long long k_sb,
                         long long k_ss, long long k_sh, long long v_sb, long long v_ss, long long v_sh, float scale,
                         int nsplit, float* part_o, float* part_ml, void* status, cudaStream_t stream) {
  if (nsplit < 1 || nsplit > 8 || (nsplit > 1 && (part_o == nullptr || part_ml == nullptr || D % 4))) return -7;
  if (B <= 0 || Sq <= 0 || Sk <= 0 || H <= 0 || Hkv <= 0 || H % Hkv) return -2;
  const int g = H / Hkv;
  if (g > 128 || (128 % g)) return -3;
  if (D % 8 || D > 256 || D < 16) return -4;
  const long long strides[9] = {q_sb, q_ss, q_sh, k_sb, k_ss, k_sh, v_sb, v_ss, v_sh};
  for (int i = 0; i < 9; ++i)
    if (strides[i] % 8) return -5;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return -6;
  AttnParams p;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.H = H; p.Hkv = Hkv; p.D = D; p.g = g;
  p.Dmma = (D + 15) / 16 * 16;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.q_blk = q_blk; p.k_blk = k_blk; p.q_valid = q_valid; p.k_valid = k_valid;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.nsplit = nsplit;
  p.skip_reach = (nsplit > 1 || Sq <= ATT_M / g) ? 1 : 0;
  p.part_o = part_o;
  p.part_ml = reinterpret_cast<float2*>(part_ml);
  p.status = static_cast<KernelStatus*>(status);
  const int dpad = D <= 64 ? 64 : (D <= 128 ? 128 : 256);
  const int bn = dpad == 256 ? 64 : 128;
  CUtensorMap tq, tk, tv;
  int r = make_map4(&tq, q, D, H, Sq, B, q_sh, q_ss, q_sb, g, ATT_M / g);
  if (r) return 1000 + r;
  r = make_map4(&tk, k, D, Hkv, Sk, B, k_sh, k_ss, k_sb, 1, bn);
  if (r) return 2000 + r;
  r = make_map4(&tv, v, D, Hkv, Sk, B, v_sh, v_ss, v_sb, 1, bn);
  if (r) return 3000 + r;
  switch (dpad) {
    case 64: return launch_attn<64, 128>(tq, tk, tv, p, stream);
    case 128: return launch_attn<128, 128>(tq, tk, tv, p, stream);
    default: return launch_attn<256, 64>(tq, tk, tv, p, stream);
  }
}

extern "C" int otb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* q_blk,
                            const int* k_blk, const unsigned char* q_valid, const unsigned char* k_valid, int B,
                            int Sq, int Sk, int H, int Hkv, int D, long long q_sb, long long q_ss, long long q_sh,
                            long long k_sb, long long k_ss, long long k_sh, long long v_sb, long long v_ss,
                            long long v_sh, float scale, void* status, cudaStream_t stream) {
  return attn_fwd_impl(q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid, B, Sq, Sk, H, Hkv, D, q_sb, q_ss, q_sh, k_sb,
                       k_ss, k_sh, v_sb, v_ss, v_sh, scale, 1, nullptr, nullptr, status, stream);
}

// Split-KV form: `nsplit` (2..8) CTAs per query tile share the key blocks; part_o holds nsplit*B*Sq*H*D floats and
// part_ml 2*nsplit*B*H*Sq floats of scratch.  Same result as otb_attn_fwd up to fp32 rounding of the merge.
extern "C" int otb_attn_fwd_splitkv(const void* q, const void* k, const void* v, void* o, float* lse, const int* q_blk,
                                    const int* k_blk, const unsigned char* q_valid, const unsigned char* k_valid,
                                    int B, int Sq, int Sk, int H, int Hkv, int D, long long q_sb, long long q_ss,
                                    long long q_sh, long long k_sb, long long k_ss, long long k_sh, long long v_sb,
                                    long long v_ss, long long v_sh, float scale, int nsplit, float* part_o,
                                    float* part_ml, void* status, cudaStream_t stream) {
  return attn_fwd_impl(q, k, v, o, lse, q_blk, k_blk, q_valid, k_valid, B, Sq, Sk, H, Hkv, D, q_sb, q_ss, q_sh, k_sb,
                       k_ss, k_sh, v_sb, v_ss, v_sh, scale, nsplit, part_o, part_ml, status, stream);
}

// key-block width the forward kernel uses for this head dimension (callers size split-KV from it)
extern "C" int otb_attn_block(int D) { return D > 128 ? 64 : 128; }
