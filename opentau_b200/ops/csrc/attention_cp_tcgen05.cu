// Context-parallel block-causal flash attention forward for sm_100a: the sequence is sharded over the ranks of one
// NVSwitch domain, every rank computes attention of ITS queries against the keys/values of ALL ranks, and the
// K/V exchange happens inside the attention kernel.
//
// Each rank keeps its K and V shard, laid out (B, Sl, Hkv, D), in peer-visible memory.  The grid has two kinds of
// CTAs.  The first NC blocks are copiers: one thread each drives bulk async copies (peer -> shared -> local), 16 KB
// at a time and a dozen in flight, that pull every OTHER rank's shard into a local gathered buffer
// (W, B, Sl, Hkv, D) exactly once, in ring order after the own rank, and count the landed pieces per (source,
// batch, key block).  The remaining blocks are attention CTAs (same tcgen05 / TMEM pipeline as the single-GPU
// kernel): their TMA producer reads the own shard in place first (no copy, no wait: the diagonal work starts at
// once), then walks the other sources in the same ring order and starts a key block as soon as its count is
// complete, so the NVLink transfer overlaps the softmax / tensor-core work on earlier keys.  (Reading remote K/V
// tiles directly would cross the link once per query tile: peer lines are not kept in the local L2.)
//
// Key metadata (block id, validity) is passed for the full sequence in gathered order (source-major); it derives
// from the batch layout, which every rank knows, so it needs no exchange.  Peers publish "my shard for step e is
// written" through a ready flag; the caller double-buffers the shards by step parity.  All waits are bounded.
// Mask rule, lazy rescale, GQA row packing and the output / LSE layout are those of the single-GPU kernel.
#include "common.cuh"
#include <limits.h>

namespace otb {

constexpr unsigned KID_ATTN = 30;
constexpr int CP_MAX_RANKS = 8;
constexpr int CP_PIECE = 16384;
constexpr int ATT_M = 128;

struct PtrArray {
  void* p[CP_MAX_RANKS];
};

struct AttnParams {
  int B, Sq, Sk, H, Hkv, D, Dmma, g;
  int W, rank, Sl, NC, nblk_src;    // ranks, this rank, keys per rank, copier CTAs, key blocks per source
  unsigned epoch;                   // step counter of this call site (1, 2, 3, ...)
  float scale_log2;                 // scale * log2(e)
  const int* q_blk;                 // (B, Sq) local queries
  const int* k_blk;                 // (B, Sk = W*Sl) all keys, source-major
  const unsigned char* q_valid;     // (B, Sq)
  const unsigned char* k_valid;     // (B, Sk)
  __nv_bfloat16* o;                 // (B, Sq, H, D) contiguous
  float* lse;                       // (B, H, Sq)
  const unsigned* ready;            // local flags[W]: ready[r] >= epoch once rank r published its K/V shard
  unsigned* gcount;                 // local [W*B*nblk_src] landed pieces per (source, batch, key block); monotonic
  unsigned* gtotal;                 // local [W*B] landed pieces per (source, batch); monotonic
  unsigned* ticket;                 // local piece dispenser; monotonic
  uint8_t* kg;                      // local gathered K (W, B, Sl, Hkv, D) bf16
  uint8_t* vg;                      // local gathered V
  long long budget;
  KernelStatus* status;
};

__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_load_5d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z,
                                            int w, int v) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z),
      "r"(w), "r"(v)
      : "memory");
}

// 16 KB pieces of key block j (rows j*BN .. of a shard with Sl rows of `rowbytes` bytes), for K or V alone
__device__ __forceinline__ int cp_pieces(int j, int BN, int Sl, int rowbytes) {
  const long long bytes = (long long)min(BN, Sl - j * BN) * rowbytes;
  return (int)((bytes + CP_PIECE - 1) / CP_PIECE);
}

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
  static constexpr int USED = OFF_BAR + NBAR * 8 + 64;
  // room for rounding the base up to 1024 bytes (the kernel has no static shared memory, so the base normally is
  // aligned already); capped at the 227 KB a CTA may own, and checked at run time
  static constexpr int TOTAL = USED + 1024 <= 232448 ? USED + 1024 : 232448;
  static_assert(USED <= 232448, "shared memory budget");
  static constexpr int NBUF = (OFF_BAR / CP_PIECE) >= 12 ? 12 : 8;  // copier buffers (copier CTAs use the tile area)
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int DPAD, int BN>
__global__ void __launch_bounds__(320, 1)
attn_fwd_cp_kernel(const __grid_constant__ CUtensorMap tma_q, const __grid_constant__ CUtensorMap tma_k,
                   const __grid_constant__ CUtensorMap tma_v, const __grid_constant__ CUtensorMap tma_k_own,
                   const __grid_constant__ CUtensorMap tma_v_own, const __grid_constant__ PtrArray k_peers,
                   const __grid_constant__ PtrArray v_peers, AttnParams p) {
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
  int* nb_smem = reinterpret_cast<int*>(tmem_slot + 2);  // [W] key blocks to visit per source
  int& s_qmax = *reinterpret_cast<int*>(tmem_slot + 2 + CP_MAX_RANKS);
  int& s_any = *reinterpret_cast<int*>(tmem_slot + 3 + CP_MAX_RANKS);
  if ((int)(smem - smem_raw) + L::USED > L::TOTAL) {   // base less aligned than assumed: refuse instead of overrunning
    if (threadIdx.x == 0) report_timeout(p.status, KID_ATTN, 99, (unsigned)(smem - smem_raw));
    return;
  }

  const int W = p.W;
  const int rowbytes = p.Hkv * p.D * 2;

  // ====================================================================== copier CTAs
  if ((int)blockIdx.x < p.NC) {
    if (threadIdx.x != 0) return;
    constexpr int NBUF = L::NBUF;
    // LD peer loads in flight (they carry the NVLink latency); a buffer is free again once its store has READ it
    // (ST stores reading), while pieces are counted CL stores late, when their writes have certainly completed, so
    // that no wait in the loop is on the latency of a store
    constexpr int ST = 2, LD = NBUF - ST, CL = 8, RING = 4 * NBUF;
    static_assert(LD + CL + 2 <= RING, "bookkeeping ring too small");
    uint64_t* cbar = bars;  // NBUF barriers (the attention barriers are unused in a copier CTA)
    for (int i = 0; i < NBUF; ++i) mbar_init(&cbar[i], 1);
    *abort_flag = 0;
    mbar_fence_init();
    // one ticket = K or V of one (ring step, batch, key block): up to ppb pieces.  A ticket per piece would put a
    // global atomic round trip and the index arithmetic on the serial path of every 16 KB.
    const long long per_src = (long long)p.B * p.nblk_src * 2;
    const long long total = per_src * (W - 1);  // the own shard is read in place, never copied
    const unsigned per_step = (unsigned)total + (unsigned)p.NC;
    const unsigned base = (p.epoch - 1u) * per_step;
    const long long shard_bytes = (long long)p.B * p.Sl * rowbytes;
    unsigned seen = 1u << p.rank;
    unsigned* cnt_of[RING] = {};
    uint8_t* dst_of[RING] = {};
    uint32_t bytes_of[RING] = {};
    long long issued = 0, stored = 0, counted = 0;
    auto store_one = [&]() {
      const int m = (int)(stored % NBUF), q = (int)(stored % RING);
      mbar_wait(&cbar[m], (uint32_t)((stored / NBUF) & 1), abort_flag, p.status, KID_ATTN, 20, m);
      bulk_store(dst_of[q], smem + m * CP_PIECE, bytes_of[q]);
      bulk_commit();
      ++stored;
    };
    auto count_upto = [&](long long upto) {
      if (counted < upto) fence_proxy_async_all();
      while (counted < upto) {
        unsigned* c = cnt_of[counted % RING];
        red_release_gpu_add(c, 1u);
        red_release_gpu_add(p.gtotal + (c - p.gcount) / p.nblk_src, 1u);   // (source, batch) total
        ++counted;
      }
    };
    while (true) {
      if (*abort_flag) break;
      const unsigned tk = atomicAdd(p.ticket, 1u) - base;
      if (tk >= (unsigned)total) break;
      // ticket -> (ring step s, batch b, key block j, K|V)
      const int s = (int)(tk / per_src);
      int r = (int)(tk - (long long)s * per_src);
      const int b = r / (p.nblk_src * 2);
      r -= b * p.nblk_src * 2;
      const int j = r >> 1;
      const int is_v = r & 1;
      const int src = (p.rank + 1 + s) % W;
      const long long blk_bytes = (long long)min(BN, p.Sl - j * BN) * rowbytes;
      if (!(seen & (1u << src))) {
        if ((int)(ld_acquire_sys_u32(p.ready + src) - p.epoch) < 0) {
          const long long t0 = clock64();
          while ((int)(ld_acquire_sys_u32(p.ready + src) - p.epoch) < 0) {
            if (clock64() - t0 > p.budget) {
              *abort_flag = 1;
              report_timeout(p.status, KID_ATTN, 21, (unsigned)src);
              break;
            }
            __nanosleep(200);
          }
        }
        seen |= 1u << src;
        if (*abort_flag) break;
      }
      const long long off0 = ((long long)b * p.Sl + (long long)j * BN) * rowbytes;
      const uint8_t* gsrc0 = static_cast<const uint8_t*>(is_v ? v_peers.p[src] : k_peers.p[src]) + off0;
      uint8_t* gdst0 = (is_v ? p.vg : p.kg) + (long long)src * shard_bytes + off0;
      unsigned* cnt = p.gcount + ((long long)src * p.B + b) * p.nblk_src + j;
      for (long long off_in_blk = 0; off_in_blk < blk_bytes; off_in_blk += CP_PIECE) {
        const uint32_t bytes = (uint32_t)min((long long)CP_PIECE, blk_bytes - off_in_blk);
        // the buffer about to be refilled was read by the store issued NBUF pieces ago
        if (issued >= NBUF) bulk_wait_read<ST - 1>();
        const int m = (int)(issued % NBUF), q = (int)(issued % RING);
        cnt_of[q] = cnt;
        dst_of[q] = gdst0 + off_in_blk;
        bytes_of[q] = bytes;
        mbar_expect_tx(&cbar[m], bytes);
        bulk_load(smem + m * CP_PIECE, gsrc0 + off_in_blk, bytes, &cbar[m]);
        ++issued;
        if (issued - stored >= LD) {
          store_one();
          bulk_wait<CL>();  // every store but the latest CL has completed: those pieces may be counted
          count_upto(stored - CL);
        }
        if (*abort_flag) break;
      }
    }
    if (*abort_flag) {
      // a wait gave up: let the copies already in flight land in this CTA's shared memory before it exits
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      bulk_wait<0>();
      return;
    }
    while (stored < issued) store_one();
    bulk_wait<0>();
    count_upto(stored);
    return;
  }

  // ====================================================================== attention CTAs
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = p.g;
  const int pos_per_tile = ATT_M / g;
  const int ntile = (p.Sq + pos_per_tile - 1) / pos_per_tile;
  const int a_id = (int)blockIdx.x - p.NC;
  const int tile = a_id % ntile, kvh = (a_id / ntile) % p.Hkv, b = a_id / (ntile * p.Hkv);
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
    for (int i = 0; i < CP_MAX_RANKS; ++i) nb_smem[i] = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_q);
    tma_prefetch_desc(&tma_k);
    tma_prefetch_desc(&tma_v);
    tma_prefetch_desc(&tma_k_own);
    tma_prefetch_desc(&tma_v_own);
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

  // ---- per source: how many key blocks can this tile reach?  1 + the last key of that source that is valid and
  //      has k_blk <= the largest valid q_blk in the tile, rounded up to blocks.
  {
    int qmax = INT_MIN;
    bool any_q = false;
    for (int i = threadIdx.x; i < pos_per_tile; i += blockDim.x) {
      int pos = p0 + i;
      if (pos < p.Sq && p.q_valid[(long long)b * p.Sq + pos]) {
        qmax = max(qmax, p.q_blk[(long long)b * p.Sq + pos]);
        any_q = true;
      }
    }
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
    if (s_any) {
      const int qm = s_qmax;
      // per source: each thread keeps its own maximum and issues ONE shared-memory atomic (an atomic per visible key
      // would serialise thousands of same-address operations per CTA)
      for (int src = 0; src < W; ++src) {
        int last = -1;
        const long long base_k = (long long)b * p.Sk + (long long)src * p.Sl;
#pragma unroll 8
        for (int j = threadIdx.x; j < p.Sl; j += blockDim.x) {
          const int kbj = p.k_blk[base_k + j];
          const int kvj = p.k_valid[base_k + j];
          if (kvj && kbj <= qm) last = max(last, j);
        }
        if (last >= 0) atomicMax(&nb_smem[src], last / BN + 1);
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int i = 0; i < W; ++i) tot += nb_smem[i];
      if (tot == 0) nb_smem[p.rank] = 1;  // the pipeline needs one block so that O is defined (all masked -> zeros)
    }
    __syncthreads();
  }

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int c = 0; c < L::NCHUNK; ++c)
        tma_load_4d(sQ + c * (ATT_M * 128), &tma_q, q_full, c * 64, kvh * g, p0, b);
      int it = 0;
      unsigned per_sb = 0;  // pieces of one (source, batch): K and V of every key block
      for (int jj = 0; jj < p.nblk_src; ++jj) per_sb += 2u * (unsigned)cp_pieces(jj, BN, p.Sl, rowbytes);
      for (int s = 0; s < W; ++s) {
        const int src = (p.rank + s) % W;
        const int nb = nb_smem[src];
        // every piece of (src, b) has landed: no more polling, no more proxy fences.  The own shard is read where
        // the host wrote it, so the diagonal work starts at once while the copiers fetch the other ranks' keys.
        const bool own = src == p.rank;
        bool src_done = own;
        for (int j = 0; j < nb; ++j, ++it) {
          const int slot = it & 1, u = it >> 1;
          if (!src_done) {
            if ((int)(ld_acquire_gpu_u32(p.gtotal + src * p.B + b) - p.epoch * per_sb) >= 0) {
              src_done = true;
            } else {
              // wait until the copiers have landed K and V of this (source, batch, key block)
              const unsigned target = p.epoch * 2u * (unsigned)cp_pieces(j, BN, p.Sl, rowbytes);
              const unsigned* cnt = p.gcount + ((long long)src * p.B + b) * p.nblk_src + j;
              if ((int)(ld_acquire_gpu_u32(cnt) - target) < 0) {
                const long long t0 = clock64();
                while ((int)(ld_acquire_gpu_u32(cnt) - target) < 0) {
                  if (*abort_flag) break;
                  if (clock64() - t0 > p.budget) {
                    *abort_flag = 1;
                    report_timeout(p.status, KID_ATTN, 22, (unsigned)(src * 1024 + j));
                    break;
                  }
                  __nanosleep(100);
                }
              }
            }
            fence_proxy_async_all();  // the pieces were written through the async proxy by other CTAs
          }
          mbar_wait(&kv_empty[slot], (u & 1) ^ 1, abort_flag, p.status, KID_ATTN, 1, it);
          uint8_t* sk = sKV + slot * L::STAGE_BYTES;
          uint8_t* sv = sk + L::KV_TILE;
          mbar_expect_tx(&kv_full[slot], L::STAGE_BYTES);
#pragma unroll
          for (int c = 0; c < L::NCHUNK; ++c) {
            if (own) {
              tma_load_4d(sk + c * (BN * 128), &tma_k_own, &kv_full[slot], c * 64, kvh, j * BN, b);
              tma_load_4d(sv + c * (BN * 128), &tma_v_own, &kv_full[slot], c * 64, kvh, j * BN, b);
            } else {
              tma_load_5d(sk + c * (BN * 128), &tma_k, &kv_full[slot], c * 64, kvh, j * BN, b, src);
              tma_load_5d(sv + c * (BN * 128), &tma_v, &kv_full[slot], c * 64, kvh, j * BN, b, src);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      int nblk = 0;
      for (int i = 0; i < W; ++i) nblk += nb_smem[i];
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

    // key metadata (INT_MAX = invisible to everyone) of block (source, jb), fetched one block ahead so that the
    // global-load latency overlaps the softmax work of the current block
    auto load_meta = [&](int src, int jb) -> int {
      const int kin = jb * BN + st;               // index inside the source's shard
      if (st >= BN || kin >= p.Sl) return INT_MAX;
      const long long key = (long long)b * p.Sk + (long long)src * p.Sl + kin;
      const int kbv = p.k_blk[key];
      const int kvv = p.k_valid[key];
      return kvv ? kbv : INT_MAX;
    };
    // the block after (rs, jb) in ring order, skipping sources this tile does not reach; rs == W: none
    auto next_block = [&](int& rs, int& jb) {
      ++jb;
      while (rs < W && jb >= nb_smem[(p.rank + rs) % W]) {
        ++rs;
        jb = 0;
      }
    };
    int nrs = 0, njb = -1;
    next_block(nrs, njb);                         // first block
    int kb_next = nrs < W ? load_meta((p.rank + nrs) % W, njb) : INT_MAX;
    int j = 0;  // running block counter over all sources (pipeline slot / phase)
    for (int rs = 0; rs < W; ++rs) {
      const int src = (p.rank + rs) % W;
      const int nb = nb_smem[src];
      for (int jb = 0; jb < nb; ++jb, ++j) {
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
      next_block(nrs, njb);
      kb_next = nrs < W ? load_meta((p.rank + nrs) % W, njb) : INT_MAX;
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
#pragma unroll 1
    for (int c = o_lo; c < o_hi; ++c) {
      uint32_t ro[16];
      __syncwarp();
      tmem_ld_x16(o_addr + c * 16, ro);
      tmem_wait_ld();
      if (row_in) {
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
      const float lse = l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : 0.f;
      p.lse[((long long)b * p.H + head) * p.Sq + pos] = lse;
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

// rank-4 bf16 map over a (B, S, Hx, D) tensor with element strides (sb, ss, sh, 1); dims innermost first
static int cp_make_map4(CUtensorMap* m, const void* base, int D, int Hx, int S, int B, long long sh, long long ss,
                        long long sb, int box_h, int box_s) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hx, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)sh * 2, (uint64_t)ss * 2, (uint64_t)sb * 2};
  uint32_t box[4] = {64, (uint32_t)box_h, (uint32_t)box_s, 1};
  return make_tmap_bf16(m, base, 4, dims, strides, box);
}

// rank-5 map over the gathered (W, B, Sl, Hkv, D) buffer
static int cp_make_map5(CUtensorMap* m, const void* base, int D, int Hkv, int Sl, int B, int W, int box_s) {
  uint64_t dims[5] = {(uint64_t)D, (uint64_t)Hkv, (uint64_t)Sl, (uint64_t)B, (uint64_t)W};
  uint64_t strides[4] = {(uint64_t)D * 2, (uint64_t)Hkv * D * 2, (uint64_t)Sl * Hkv * D * 2,
                         (uint64_t)B * Sl * Hkv * D * 2};
  uint32_t box[5] = {64, 1, (uint32_t)box_s, 1, 1};
  return make_tmap_bf16(m, base, 5, dims, strides, box);
}

template <int DPAD, int BN>
static int launch_attn_cp(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tko,
                          const CUtensorMap& tvo, const PtrArray& kp, const PtrArray& vp, const AttnParams& p, cudaStream_t stream) {
  using L = AttnSmem<DPAD, BN>;
  static bool configured = false;
  auto kern = attn_fwd_cp_kernel<DPAD, BN>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int pos_per_tile = ATT_M / p.g;
  const int ntile = (p.Sq + pos_per_tile - 1) / pos_per_tile;
  const int grid = p.NC + ntile * p.Hkv * p.B;
  kern<<<grid, 320, L::TOTAL, stream>>>(tq, tk, tv, tko, tvo, kp, vp, p);
  return (int)cudaGetLastError();
}

}  // namespace otb

using namespace otb;

// key-block width the kernel uses for head dim D (the caller sizes `gcount` with it)
extern "C" int otb_attn_cp_block(int D) { return D > 128 ? 64 : 128; }

// q: local queries (B,Sq,H,D) with strides (q_sb,q_ss,q_sh,1); o: (B,Sq,H,D) contiguous; lse: (B,H,Sq).
// k_peers[r] / v_peers[r]: rank r's contiguous (B,Sl,Hkv,D) shard as mapped into this process (this step's parity).
// kg / vg: local gathered buffers (W,B,Sl,Hkv,D).  gcount: local unsigned[W*B*(ceil(Sl/BN) + 1) + 1], zeroed once and owned
// by this call site; `epoch` must go 1, 2, 3, ... on it.  k_blk / k_valid: (B, W*Sl) for all keys, source-major.
extern "C" int otb_attn_fwd_cp(const void* q, void* o, float* lse, const int* q_blk, const int* k_blk,
                               const unsigned char* q_valid, const unsigned char* k_valid, int B, int Sq, int Sl, int H,
                               int Hkv, int D, long long q_sb, long long q_ss, long long q_sh, void* const* k_peers,
                               void* const* v_peers, void* kg, void* vg, void* gcount, const void* ready, int rank,
                               int W, unsigned epoch, int num_copiers, float scale, long long budget, void* status,
                               cudaStream_t stream) {
  if (B <= 0 || Sq <= 0 || Sl <= 0 || H <= 0 || Hkv <= 0 || H % Hkv) return -2;
  const int g = H / Hkv;
  if (g > 128 || (128 % g)) return -3;
  if (D % 8 || D > 256 || D < 16) return -4;
  if ((q_sb % 8) || (q_ss % 8) || (q_sh % 8)) return -5;
  if (W < 1 || W > CP_MAX_RANKS || rank < 0 || rank >= W || num_copiers < 1 || epoch == 0) return -9;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(kg) |
       reinterpret_cast<uintptr_t>(vg)) & 15)
    return -6;
  PtrArray kp, vp;
  memset(&kp, 0, sizeof(kp));
  memset(&vp, 0, sizeof(vp));
  for (int r = 0; r < W; ++r) {
    if ((reinterpret_cast<uintptr_t>(k_peers[r]) | reinterpret_cast<uintptr_t>(v_peers[r])) & 15) return -6;
    kp.p[r] = k_peers[r];
    vp.p[r] = v_peers[r];
  }
  const int dpad = D <= 64 ? 64 : (D <= 128 ? 128 : 256);
  const int bn = otb_attn_cp_block(D);
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.B = B; p.Sq = Sq; p.Sk = W * Sl; p.H = H; p.Hkv = Hkv; p.D = D; p.g = g;
  p.Dmma = (D + 15) / 16 * 16;
  p.W = W; p.rank = rank; p.Sl = Sl; p.NC = num_copiers; p.nblk_src = (Sl + bn - 1) / bn;
  p.epoch = epoch;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.q_blk = q_blk; p.k_blk = k_blk; p.q_valid = q_valid; p.k_valid = k_valid;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.ready = static_cast<const unsigned*>(ready);
  p.gcount = static_cast<unsigned*>(gcount);
  p.gtotal = p.gcount + (size_t)W * B * p.nblk_src;
  p.ticket = p.gtotal + (size_t)W * B;
  p.kg = static_cast<uint8_t*>(kg);
  p.vg = static_cast<uint8_t*>(vg);
  p.budget = budget;
  p.status = static_cast<KernelStatus*>(status);
  CUtensorMap tq, tk, tv, tko, tvo;
  int r = cp_make_map4(&tq, q, D, H, Sq, B, q_sh, q_ss, q_sb, g, ATT_M / g);
  if (r) return 1000 + r;
  r = cp_make_map5(&tk, kg, D, Hkv, Sl, B, W, bn);
  if (r) return 2000 + r;
  r = cp_make_map5(&tv, vg, D, Hkv, Sl, B, W, bn);
  if (r) return 3000 + r;
  const long long row = (long long)Hkv * D;
  r = cp_make_map4(&tko, k_peers[rank], D, Hkv, Sl, B, D, row, row * Sl, 1, bn);
  if (r) return 4000 + r;
  r = cp_make_map4(&tvo, v_peers[rank], D, Hkv, Sl, B, D, row, row * Sl, 1, bn);
  if (r) return 5000 + r;
  switch (dpad) {
    case 64: return launch_attn_cp<64, 128>(tq, tk, tv, tko, tvo, kp, vp, p, stream);
    case 128: return launch_attn_cp<128, 128>(tq, tk, tv, tko, tvo, kp, vp, p, stream);
    default: return launch_attn_cp<256, 64>(tq, tk, tv, tko, tvo, kp, vp, p, stream);
  }
}

// stores `epoch` into ready[rank] of every rank: "my K/V shard for this step is written"
__global__ void cp_publish_kernel(PtrArray ready, int rank, int world, unsigned epoch) {
  const int i = threadIdx.x;
  if (i >= world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(static_cast<unsigned*>(ready.p[i]) + rank), "r"(epoch)
               : "memory");
}

extern "C" int otb_cp_publish(void* const* ready, int rank, int world, unsigned epoch, cudaStream_t stream) {
  if (world < 1 || world > CP_MAX_RANKS) return -9;
  PtrArray r;
  memset(&r, 0, sizeof(r));
  for (int i = 0; i < world; ++i) r.p[i] = ready[i];
  cp_publish_kernel<<<1, 32, 0, stream>>>(r, rank, world, epoch);
  return (int)cudaGetLastError();
}
