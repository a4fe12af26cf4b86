// Tensor-parallel linears fused with their collective over peer memory (NVLink / NVSwitch), sm_100a.
//
//   all-gather -> GEMM   (column-parallel linear on a sequence-sharded activation)
//       D[W*Ml, N] = concat_r(A_r[Ml, K]) * B[N, K]^T (+ bias)
//       Every rank keeps only its own rows A_r in a peer-visible buffer.  A copier warp in every CTA pulls
//       the peers' rows across NVLink exactly once, 16 KB at a time (bulk async copy peer -> shared ->
//       local gathered buffer, two copies in flight per CTA), and counts finished pieces per 128-row
//       block; the TMA producer warp starts a remote row block as soon as its count is complete, so the
//       link transfer of later blocks overlaps the tensor-core work on earlier ones.  (A tile is re-read
//       once per column block: reading it from the peer each time would multiply the link traffic,
//       because peer lines are not kept in the local L2.)  Own rows go first and are read in place; a
//       peer is touched only after it published its rows (ready flag, release/acquire at system scope).
//
//   GEMM -> reduce-scatter   (row-parallel linear that leaves a sequence-sharded result)
//       out_d[Ml, N] = sum_r A_r[rows of d, Kl] * B_r[N, Kl]^T (+ bias) (+ residual)
//       The epilogue converts each partial tile to bf16 in shared memory and sends it with TMA tensor
//       stores (full 128-byte lines) into the destination rank's staging buffer; tiles bound for remote
//       ranks are scheduled first, own rows last.  When a tile's stores have completed it bumps a per
//       (source, row-block) counter at the destination with a release-add.  The tail of the SAME kernel
//       waits, row-block by row-block, for all W sources and writes the fp32-summed result.
//
// Buffers that peers read or write are double-buffered by step parity by the caller; since each step of
// rank r waits for step-e data of every peer, no rank can be more than one step ahead, which makes the
// parity scheme race free without an extra barrier.
//
// All waits are bounded; on expiry the kernel records {kernel, stage, peer} and runs to its normal end.
// `phase_mask` lets a single-GPU test run the two halves of GEMM -> reduce-scatter as separate launches
// (bit 0: GEMM + peer stores, bit 1: reduce), because kernels that wait on one another must never share
// a GPU.
#include "common.cuh"

namespace otb {

constexpr int DBM = 128;
constexpr int DBK = 64;
constexpr int DUMMA_K = 16;
constexpr int DMAX_RANKS = 8;
constexpr unsigned KID_AG_GEMM = 20, KID_GEMM_RS = 21;

struct TmapArray {
  CUtensorMap m[DMAX_RANKS];
};
struct PtrArray {
  void* p[DMAX_RANKS];
};

__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(unsigned* p, unsigned v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
// untiled bulk copies: global -> shared (mbarrier completion) and shared -> global (bulk group)
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
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Bounded wait until *flag (written by a peer) has reached `target` (wrap-safe compare).
__device__ __forceinline__ bool wait_flag_ge(const unsigned* flag, unsigned target, volatile int* abort_flag,
                                             long long budget, KernelStatus* st, unsigned kid, unsigned stage,
                                             unsigned detail) {
  if ((int)(ld_acquire_sys_u32(flag) - target) >= 0) return true;
  const long long t0 = clock64();
  while (true) {
    if (*abort_flag) return false;
    if ((int)(ld_acquire_sys_u32(flag) - target) >= 0) return true;
    if (clock64() - t0 > budget) {
      *abort_flag = 1;
      report_timeout(st, kid, stage, detail);
      return false;
    }
    __nanosleep(200);
  }
}

struct DistParams {
  int Ml;          // rows owned by one rank
  int N, K;        // output columns and contraction length of THIS rank's GEMM
  int rank, world;
  unsigned epoch;  // step counter (>= 1), the value peers publish / count up to
  __nv_bfloat16* out;
  long long ldo;
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [Ml, N] or null (GEMM -> RS only)
  long long ldr;
  const unsigned* ready;  // AG: local flags[world], ready[r] >= epoch once rank r published its rows
  __nv_bfloat16* gathered;  // AG: local [world*Ml, K] buffer the peers' rows are copied into
  unsigned* gcount;         // AG: local [world][row blocks] count of 16 KB pieces that have landed (monotonic)
  unsigned* ticket;         // AG: local piece dispenser (monotonic)
  int phase_mask;
  long long budget;
  KernelStatus* status;
};

constexpr int XBUF_BYTES = 16384;  // one copier piece / one 128 x 64 bf16 store chunk

template <int BN, int STAGES>
struct DistSmem {
  static constexpr int A_BYTES = DBM * DBK * 2;
  static constexpr int B_BYTES = BN * DBK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int XBUF_OFFSET = STAGES * STAGE_BYTES;       // 2 x 16 KB, 1024-byte aligned
  static constexpr int BAR_OFFSET = XBUF_OFFSET + 2 * XBUF_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 6) * 8 + 16 + 1024;
};
static_assert(DistSmem<256, 4>::TOTAL <= 232448, "shared memory budget");
static_assert(DistSmem<128, 6>::TOTAL <= 232448, "shared memory budget");

// tile -> (segment, m block inside the segment, n block); n fastest inside groups of 8 m blocks so
// that CTAs working at the same time share B tiles in L2.
__device__ __forceinline__ void dist_tile_coords(int tile, int m_per_seg, int num_n, int& seg, int& mi, int& ni) {
  const int per_seg = m_per_seg * num_n;
  seg = tile / per_seg;
  int r = tile - seg * per_seg;
  constexpr int GROUP = 8;
  const int group_size = GROUP * num_n;
  const int g = r / group_size;
  const int first_m = g * GROUP;
  const int gm = min(m_per_seg - first_m, GROUP);
  r -= g * group_size;
  mi = first_m + r % gm;
  ni = r / gm;
}

// pieces of 16 KB in row block `mb` of a shard of Ml rows x K columns
__device__ __forceinline__ int pieces_in_block(int mb, int Ml, int K) {
  const long long bytes = (long long)min(DBM, Ml - mb * DBM) * K * 2;
  return (int)((bytes + XBUF_BYTES - 1) / XBUF_BYTES);
}

// MODE 0: all-gather -> GEMM.  MODE 1: GEMM -> reduce-scatter.
// tma_a.m[0]: MODE 0 own shard [Ml, K] / MODE 1 the local activation [W*Ml, Kl]; tma_a.m[1]: MODE 0 the gathered
// buffer [W*Ml, K].  st_maps.m[d] (MODE 1): staging of rank d as a 3-D tensor (N, Ml, W sources).
template <int MODE, int BN, int STAGES>
__global__ void __launch_bounds__(224, 1)
gemm_dist_kernel(const __grid_constant__ TmapArray tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ TmapArray st_maps, const __grid_constant__ PtrArray peers,
                 const __grid_constant__ PtrArray counters, DistParams p) {
  using L = DistSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* xbuf = smem + L::XBUF_OFFSET;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint64_t* copy_bar = tempty_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(copy_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int W = p.world;
  const int m_per_seg = (p.Ml + DBM - 1) / DBM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = (MODE == 1 && !(p.phase_mask & 1)) ? 0 : W * m_per_seg * num_n;
  const int num_kb = (p.K + DBK - 1) / DBK;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr unsigned KID = MODE == 0 ? KID_AG_GEMM : KID_GEMM_RS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 128);
      mbar_init(&copy_bar[b], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage_i = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        if (*abort_flag) break;  // a wait gave up: issue no further copies
        int seg, mi, ni;
        dist_tile_coords(tile, m_per_seg, num_n, seg, mi, ni);
        const int n0 = ni * BN;
        const CUtensorMap* amap;
        int a_row;
        if (MODE == 0) {
          const int src = (p.rank + seg) % W;  // own rows first, then the peers in ring order
          if (seg == 0) {
            amap = &tma_a.m[0];
            a_row = mi * DBM;
          } else {
            // rows of a peer: wait until the copier warps have landed every piece of this row block
            const unsigned target = p.epoch * (unsigned)pieces_in_block(mi, p.Ml, p.K);
            const unsigned* cnt = p.gcount + src * m_per_seg + mi;
            if ((int)(ld_acquire_gpu_u32(cnt) - target) < 0) {
              const long long t0 = clock64();
              while ((int)(ld_acquire_gpu_u32(cnt) - target) < 0) {
                if (*abort_flag) break;
                if (clock64() - t0 > p.budget) {
                  *abort_flag = 1;
                  report_timeout(p.status, KID, 7, (unsigned)(src * m_per_seg + mi));
                  break;
                }
                __nanosleep(100);
              }
            }
            fence_proxy_async_all();  // the pieces were written through the async proxy by other CTAs
            amap = &tma_a.m[1];
            a_row = src * p.Ml + mi * DBM;
          }
        } else {
          const int dst = (p.rank + 1 + seg) % W;  // remote destinations first, own rows last
          amap = &tma_a.m[0];
          a_row = dst * p.Ml + mi * DBM;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&empty_bar[stage_i], phase ^ 1, abort_flag, p.status, KID, 1, stage_i);
          uint8_t* sa = smem + stage_i * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage_i], L::STAGE_BYTES);
          tma_load_2d(sa, amap, &full_bar[stage_i], kb * DBK, a_row);
          tma_load_2d(sb, &tma_b, &full_bar[stage_i], kb * DBK, n0);
          if (++stage_i == STAGES) {
            stage_i = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_bf16(DBM, BN, 0, 0);
      int stage_i = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        if (*abort_flag) break;
        mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, KID, 2, acc);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&full_bar[stage_i], phase, abort_flag, p.status, KID, 3, stage_i);
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage_i * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < DBK / DUMMA_K; ++k) {
            uint64_t ad = make_smem_desc(sa + k * 32u, 16u, 1024);
            uint64_t bd = make_smem_desc(sb + k * 32u, 16u, 1024);
            umma_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage_i]);
          if (++stage_i == STAGES) {
            stage_i = 0;
            phase ^= 1;
          }
        }
        umma_commit(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------------ copier (all-gather only)
    if (MODE == 0 && W > 1 && elect_one()) {
      // pieces in consumption order: peer segments 1..W-1, row blocks, 16 KB pieces
      const long long shard_bytes = (long long)p.Ml * p.K * 2;
      const long long block_bytes = (long long)DBM * p.K * 2;
      const int ppb = (int)((block_bytes + XBUF_BYTES - 1) / XBUF_BYTES);  // pieces per full row block
      const long long total = (long long)(W - 1) * m_per_seg * ppb;
      unsigned seen = 0;
      uint32_t ph[2] = {0, 0};
      long long pend_u = -1;   // piece whose store was issued but not yet counted
      long long loaded_u = -1; // piece whose load is in flight
      int loaded_buf = 0;
      uint32_t loaded_bytes = 0;
      // decode piece u -> src, mb, byte offset in the shard, size (0 = piece does not exist in a short last block)
      auto decode = [&](long long u, int& src, int& mb, long long& off, uint32_t& bytes) {
        const int seg = (int)(u / ((long long)m_per_seg * ppb));
        const int r = (int)(u - (long long)seg * m_per_seg * ppb);
        mb = r / ppb;
        const int c = r - mb * ppb;
        src = (p.rank + 1 + seg) % W;
        off = (long long)mb * block_bytes + (long long)c * XBUF_BYTES;
        const long long end = min(shard_bytes, (long long)(mb + 1) * block_bytes);
        const long long left = end - off;
        bytes = left <= 0 ? 0u : (uint32_t)min((long long)XBUF_BYTES, left);
      };
      auto count_piece = [&](long long u) {
        int src, mb;
        long long off;
        uint32_t bytes;
        decode(u, src, mb, off, bytes);
        fence_proxy_async_all();
        red_release_gpu_add(p.gcount + src * m_per_seg + mb, 1u);
      };
      int nbuf = 0;
      // pieces are handed out by a ticket counter, so the CTAs that are running copy everything even when
      // part of the grid is still waiting for an SM; every CTA draws exactly one ticket past the end
      const unsigned per_step = (unsigned)total + gridDim.x;
      const unsigned base = (p.epoch - 1u) * per_step;
      while (true) {
        if (*abort_flag) break;
        const unsigned tk = atomicAdd(p.ticket, 1u) - base;
        if (tk >= (unsigned)total) break;
        const long long u = tk;
        int src, mb;
        long long off;
        uint32_t bytes;
        decode(u, src, mb, off, bytes);
        if (bytes == 0) continue;
        if (!(seen & (1u << src))) {
          wait_flag_ge(p.ready + src, p.epoch, abort_flag, p.budget, p.status, KID, 5, (unsigned)src);
          seen |= 1u << src;
          if (*abort_flag) break;
        }
        // the buffer about to be refilled was last read by the store of the piece before the one in flight
        if (pend_u >= 0) {
          bulk_wait<0>();
          count_piece(pend_u);
          pend_u = -1;
        }
        const int b = nbuf;
        nbuf ^= 1;
        mbar_expect_tx(&copy_bar[b], bytes);
        bulk_load(xbuf + b * XBUF_BYTES, static_cast<const uint8_t*>(peers.p[src]) + off, bytes, &copy_bar[b]);
        if (loaded_u >= 0) {
          // finish the previous piece: wait for its load, push it to the gathered buffer
          mbar_wait(&copy_bar[loaded_buf], ph[loaded_buf], abort_flag, p.status, KID, 8, loaded_buf);
          ph[loaded_buf] ^= 1;
          int s2, m2;
          long long o2;
          uint32_t b2;
          decode(loaded_u, s2, m2, o2, b2);
          bulk_store(reinterpret_cast<uint8_t*>(p.gathered) + (long long)s2 * shard_bytes + o2,
                     xbuf + loaded_buf * XBUF_BYTES, loaded_bytes);
          bulk_commit();
          pend_u = loaded_u;
        }
        loaded_u = u;
        loaded_buf = b;
        loaded_bytes = bytes;
      }
      if (loaded_u >= 0) {
        if (pend_u >= 0) {
          bulk_wait<0>();
          count_piece(pend_u);
          pend_u = -1;
        }
        mbar_wait(&copy_bar[loaded_buf], ph[loaded_buf], abort_flag, p.status, KID, 8, loaded_buf);
        int s2, m2;
        long long o2;
        uint32_t b2;
        decode(loaded_u, s2, m2, o2, b2);
        bulk_store(reinterpret_cast<uint8_t*>(p.gathered) + (long long)s2 * shard_bytes + o2,
                   xbuf + loaded_buf * XBUF_BYTES, loaded_bytes);
        bulk_commit();
        pend_u = loaded_u;
      }
      if (pend_u >= 0) {
        bulk_wait<0>();
        count_piece(pend_u);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    const int et = quad * 32 + lane;  // 0..127 inside the epilogue group
    int acc = 0;
    uint32_t acc_phase = 0;
    int xb = 0;  // staging chunk buffer in use (MODE 1)
    unsigned* prev_cnt = nullptr;  // counter of the last tile whose stores may still be in flight (thread et == 0)
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int seg, mi, ni;
      dist_tile_coords(tile, m_per_seg, num_n, seg, mi, ni);
      const int n0 = ni * BN;
      const int lrow = mi * DBM + quad * 32 + lane;  // row inside the segment
      const bool row_ok = lrow < p.Ml;
      mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, KID, 4, acc);
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + acc * BN;
      if (MODE == 0) {
        const int src = (p.rank + seg) % W;
        __nv_bfloat16* dst_row = p.out + ((long long)src * p.Ml + lrow) * p.ldo;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          __syncwarp();
          uint32_t r[32];
          tmem_ld_x32(taddr + c * 32, r);
          tmem_wait_ld();
          const int col0 = n0 + c * 32;
          if (row_ok && col0 < p.N) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = col0 + j * 8;
              if (col >= p.N) break;
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j * 8 + e]);
              if (p.bias != nullptr) {
                uint4 bb = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
                float2 f;
                f = unpack_bf16(bb.x); v[0] += f.x; v[1] += f.y;
                f = unpack_bf16(bb.y); v[2] += f.x; v[3] += f.y;
                f = unpack_bf16(bb.z); v[4] += f.x; v[5] += f.y;
                f = unpack_bf16(bb.w); v[6] += f.x; v[7] += f.y;
              }
              uint4 o;
              o.x = pack_bf16(v[0], v[1]);
              o.y = pack_bf16(v[2], v[3]);
              o.z = pack_bf16(v[4], v[5]);
              o.w = pack_bf16(v[6], v[7]);
              *reinterpret_cast<uint4*>(dst_row + col) = o;
            }
          }
        }
        tc_fence_before();
        mbar_arrive(&tempty_bar[acc]);
      } else {
        // partial tile -> bf16 in shared memory (128-byte swizzle) -> TMA store into the destination's staging
        const int peer = (p.rank + 1 + seg) % W;
        const int trow = quad * 32 + lane;  // row inside the tile
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          __syncwarp();
          uint32_t r[32], r2[32];
          tmem_ld_x32(taddr + c * 64, r);
          tmem_ld_x32(taddr + c * 64 + 32, r2);
          tmem_wait_ld();
          if (c == BN / 64 - 1) {
            tc_fence_before();
            mbar_arrive(&tempty_bar[acc]);  // accumulator fully read: the MMA warp may reuse it
          }
          // the chunk buffer was last read by the store issued two chunks ago
          if (et == 0) bulk_wait_read<1>();
          epi_bar_sync();
          uint8_t* rowp = xbuf + xb * XBUF_BYTES + trow * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t* rr = j < 4 ? r + j * 8 : r2 + (j - 4) * 8;
            uint4 o;
            o.x = pack_bf16(__uint_as_float(rr[0]), __uint_as_float(rr[1]));
            o.y = pack_bf16(__uint_as_float(rr[2]), __uint_as_float(rr[3]));
            o.z = pack_bf16(__uint_as_float(rr[4]), __uint_as_float(rr[5]));
            o.w = pack_bf16(__uint_as_float(rr[6]), __uint_as_float(rr[7]));
            *reinterpret_cast<uint4*>(rowp + ((j ^ (trow & 7)) << 4)) = o;
          }
          fence_async_smem();
          epi_bar_sync();
          const int col0 = n0 + c * 64;
          if (et == 0) {
            if (col0 < p.N) tma_store_3d(&st_maps.m[peer], xbuf + xb * XBUF_BYTES, col0, mi * DBM, p.rank);
            bulk_commit();  // always one group per chunk, so group counts identify tiles
          }
          xb ^= 1;
        }
        // count the PREVIOUS tile at its destination: its stores are complete once at most this tile's
        // BN/64 groups are still pending, so the wait rarely stalls
        if (et == 0) {
          if (prev_cnt != nullptr) {
            bulk_wait<BN / 64>();
            fence_proxy_async_all();
            __threadfence_system();
            red_release_sys_add(prev_cnt, 1u);
          }
          prev_cnt = static_cast<unsigned*>(counters.p[peer]) + p.rank * m_per_seg + mi;
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }

    if (MODE == 1 && et == 0 && prev_cnt != nullptr) {
      bulk_wait<0>();
      fence_proxy_async_all();
      __threadfence_system();
      red_release_sys_add(prev_cnt, 1u);
    }

    if (MODE == 1 && (p.phase_mask & 2)) {
      // -------------------------------------------------------------- reduce tail: my rows, all sources
      // units of 128 rows x 256 columns spread over all CTAs; 4 independent 16-byte columns per thread and
      // source are in flight at a time
      const __nv_bfloat16* my_stage = static_cast<const __nv_bfloat16*>(peers.p[p.rank]);
      const unsigned* my_cnt = static_cast<const unsigned*>(counters.p[p.rank]);
      const unsigned target = p.epoch * (unsigned)num_n;
      constexpr int RW = 256;  // columns per unit
      const int ncu = (p.N + RW - 1) / RW;
      const int units = m_per_seg * ncu;
      int waited_mb = -1;
      for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int mb = u / ncu, cb = u - mb * ncu;
        if (mb != waited_mb) {
          if (et < W) wait_flag_ge(my_cnt + et * m_per_seg + mb, target, abort_flag, p.budget, p.status, KID, 6, et);
          epi_bar_sync();
          waited_mb = mb;
        }
        const int rows = min(DBM, p.Ml - mb * DBM);
        const int c0 = cb * RW;
        const int vecs = (min(RW, p.N - c0)) >> 3;  // 16-byte vectors per row in this unit (<= 32)
        // thread -> (row offset, vector): a warp covers one row's 32 vectors; 4 rows per pass per warp
        const int v = lane;
        for (int r0 = quad; r0 < rows; r0 += 16) {
          float a[4][8];
          bool ok[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            ok[i] = (r0 + 4 * i) < rows && v < vecs;
#pragma unroll
            for (int e = 0; e < 8; ++e) a[i][e] = 0.f;
          }
          for (int s = 0; s < W; ++s) {
            uint4 uu[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              if (ok[i]) {
                const int row = mb * DBM + r0 + 4 * i;
                uu[i] = __ldcg(reinterpret_cast<const uint4*>(my_stage + ((long long)s * p.Ml + row) * p.N + c0 + v * 8));
              } else {
                uu[i] = make_uint4(0, 0, 0, 0);
              }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float2 f;
              f = unpack_bf16(uu[i].x); a[i][0] += f.x; a[i][1] += f.y;
              f = unpack_bf16(uu[i].y); a[i][2] += f.x; a[i][3] += f.y;
              f = unpack_bf16(uu[i].z); a[i][4] += f.x; a[i][5] += f.y;
              f = unpack_bf16(uu[i].w); a[i][6] += f.x; a[i][7] += f.y;
            }
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (!ok[i]) continue;
            const int row = mb * DBM + r0 + 4 * i;
            const int col = c0 + v * 8;
            if (p.bias != nullptr) {
              uint4 bb = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
              float2 f;
              f = unpack_bf16(bb.x); a[i][0] += f.x; a[i][1] += f.y;
              f = unpack_bf16(bb.y); a[i][2] += f.x; a[i][3] += f.y;
              f = unpack_bf16(bb.z); a[i][4] += f.x; a[i][5] += f.y;
              f = unpack_bf16(bb.w); a[i][6] += f.x; a[i][7] += f.y;
            }
            if (p.residual != nullptr) {
              uint4 bb = *reinterpret_cast<const uint4*>(p.residual + (long long)row * p.ldr + col);
              float2 f;
              f = unpack_bf16(bb.x); a[i][0] += f.x; a[i][1] += f.y;
              f = unpack_bf16(bb.y); a[i][2] += f.x; a[i][3] += f.y;
              f = unpack_bf16(bb.z); a[i][4] += f.x; a[i][5] += f.y;
              f = unpack_bf16(bb.w); a[i][6] += f.x; a[i][7] += f.y;
            }
            uint4 o;
            o.x = pack_bf16(a[i][0], a[i][1]);
            o.y = pack_bf16(a[i][2], a[i][3]);
            o.z = pack_bf16(a[i][4], a[i][5]);
            o.w = pack_bf16(a[i][6], a[i][7]);
            *reinterpret_cast<uint4*>(p.out + (long long)row * p.ldo + col) = o;
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let copies / MMAs in flight land
    }
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Publishes "my rows for step `epoch` are written": stores epoch into ready[rank] of every rank.
__global__ void publish_kernel(PtrArray ready, int rank, int world, unsigned epoch) {
  const int i = threadIdx.x;
  if (i >= world) return;
  __threadfence_system();
  st_release_sys_u32(static_cast<unsigned*>(ready.p[i]) + rank, epoch);
}

// ------------------------------------------------------------------------------------------ host
static int g_dist_sms = 0;

template <int MODE, int BN, int STAGES>
static int launch_dist(const TmapArray& ta, const CUtensorMap& tb, const TmapArray& st_maps, const PtrArray& peers,
                       const PtrArray& counters, const DistParams& p, cudaStream_t stream) {
  using L = DistSmem<BN, STAGES>;
  static bool configured = false;
  auto kern = gemm_dist_kernel<MODE, BN, STAGES>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int m_per_seg = (p.Ml + DBM - 1) / DBM;
  const int num_tiles = p.world * m_per_seg * ((p.N + BN - 1) / BN);
  int grid = num_tiles < g_dist_sms ? num_tiles : g_dist_sms;
  kern<<<grid, 224, L::TOTAL, stream>>>(ta, tb, st_maps, peers, counters, p);
  return (int)cudaGetLastError();
}

static int dist_common_checks(int Ml, int N, int K, int rank, int world) {
  if (Ml <= 0 || N <= 0 || K <= 0) return -2;
  if ((N % 8) || (K % 8)) return -3;
  if (world < 1 || world > DMAX_RANKS || rank < 0 || rank >= world) return -9;
  if (g_dist_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_dist_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_dist_sms <= 0) return -7;
  }
  return 0;
}

static int pick_bn(int Ml, int N, int world) {
  const long long m_tiles = (long long)world * ((Ml + DBM - 1) / DBM);
  if (m_tiles * ((N + 255) / 256) >= g_dist_sms || N >= 4096) return 256;
  return 128;
}

}  // namespace otb

using namespace otb;

// a_shards[r]: rank r's contiguous [Ml, K] rows as mapped into THIS process; B: [N, K] local weight shard;
// out: [world*Ml, N].  ready: local unsigned[world], ready[r] >= epoch once rank r published its rows.
// gathered: local scratch [world*Ml, K] bf16; gcount: local unsigned[world * ceil(Ml/128) + 1] (piece counts
// per row block, then the piece dispenser), zeroed once and owned by this call site: both count monotonically
// across steps of the same shape, and `epoch` must go 1, 2, 3, ... on it.
extern "C" int otb_ag_gemm_bf16(void* const* a_shards, const void* B, void* out, int Ml, int N, int K, long long ldb,
                                long long ldo, const void* bias, const void* ready, void* gathered, void* gcount,
                                int rank, int world, unsigned epoch, long long budget, void* status,
                                cudaStream_t stream) {
  int rc = dist_common_checks(Ml, N, K, rank, world);
  if (rc) return rc;
  if ((ldb % 8) || (ldo % 8)) return -3;
  if (world > 1 && (gathered == nullptr || gcount == nullptr || ready == nullptr)) return -10;
  const int bn = pick_bn(Ml, N, world);
  TmapArray ta, none_maps;
  memset(&none_maps, 0, sizeof(none_maps));
  CUtensorMap tb;
  uint64_t dims[2], strides[1];
  uint32_t box[2];
  PtrArray peers, none;
  memset(&peers, 0, sizeof(peers));
  memset(&none, 0, sizeof(none));
  for (int r = 0; r < world; ++r) {
    if (reinterpret_cast<uintptr_t>(a_shards[r]) & 15) return -4;
    peers.p[r] = a_shards[r];
  }
  dims[0] = K; dims[1] = Ml; box[0] = 64; box[1] = DBM;
  strides[0] = (uint64_t)K * 2;
  int e = make_tmap_bf16(&ta.m[0], a_shards[rank], 2, dims, strides, box);
  if (e) return 1000 + e;
  for (int r = 1; r < DMAX_RANKS; ++r) ta.m[r] = ta.m[0];
  if (world > 1) {
    dims[1] = (uint64_t)world * Ml;
    e = make_tmap_bf16(&ta.m[1], gathered, 2, dims, strides, box);
    if (e) return 1100 + e;
  }
  dims[0] = K; dims[1] = N; box[0] = 64; box[1] = bn;
  strides[0] = (uint64_t)ldb * 2;
  e = make_tmap_bf16(&tb, B, 2, dims, strides, box);
  if (e) return 2000 + e;
  DistParams p;
  memset(&p, 0, sizeof(p));
  p.Ml = Ml; p.N = N; p.K = K; p.rank = rank; p.world = world; p.epoch = epoch;
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.ready = static_cast<const unsigned*>(ready);
  p.gathered = static_cast<__nv_bfloat16*>(gathered);
  p.gcount = static_cast<unsigned*>(gcount);
  p.ticket = p.gcount + (size_t)world * ((Ml + DBM - 1) / DBM);
  p.phase_mask = 3; p.budget = budget; p.status = static_cast<KernelStatus*>(status);
  if (bn == 256) return launch_dist<0, 256, 4>(ta, tb, none_maps, peers, none, p, stream);
  return launch_dist<0, 128, 6>(ta, tb, none_maps, peers, none, p, stream);
}

// A: [world*Ml, Kl] local activation (all rows, this rank's slice of the contraction); B: [N, Kl];
// stage[r] / counters[r]: rank r's staging [world][Ml][N] bf16 and counters [world][ceil(Ml/128)] u32 as mapped
// into this process (this step's parity); out: [Ml, N] this rank's rows of the reduced result.
extern "C" int otb_gemm_rs_bf16(const void* A, const void* B, void* out, int Ml, int N, int Kl, long long lda,
                                long long ldb, long long ldo, const void* bias, const void* residual, long long ldr,
                                void* const* stage, void* const* counters, int rank, int world, unsigned epoch,
                                int phase_mask, long long budget, void* status, cudaStream_t stream) {
  int rc = dist_common_checks(Ml, N, Kl, rank, world);
  if (rc) return rc;
  if ((lda % 8) || (ldb % 8) || (ldo % 8) || (residual && (ldr % 8))) return -3;
  if (reinterpret_cast<uintptr_t>(A) & 15) return -4;
  if (N < 64) return -11;
  const int bn = pick_bn(Ml, N, world);
  TmapArray ta;
  CUtensorMap tb;
  uint64_t dims[2], strides[1];
  uint32_t box[2];
  dims[0] = Kl; dims[1] = (uint64_t)world * Ml; box[0] = 64; box[1] = DBM;
  strides[0] = (uint64_t)lda * 2;
  int e = make_tmap_bf16(&ta.m[0], A, 2, dims, strides, box);
  if (e) return 1000 + e;
  for (int r = 1; r < DMAX_RANKS; ++r) ta.m[r] = ta.m[0];
  dims[0] = Kl; dims[1] = N; box[0] = 64; box[1] = bn;
  strides[0] = (uint64_t)ldb * 2;
  e = make_tmap_bf16(&tb, B, 2, dims, strides, box);
  if (e) return 2000 + e;
  PtrArray st, ct;
  TmapArray st_maps;
  memset(&st, 0, sizeof(st));
  memset(&ct, 0, sizeof(ct));
  memset(&st_maps, 0, sizeof(st_maps));
  for (int r = 0; r < world; ++r) {
    st.p[r] = stage[r];
    ct.p[r] = counters[r];
    // staging of rank r seen as (N, Ml, world sources): stores are clipped at the shard's row count
    uint64_t d3[3] = {(uint64_t)N, (uint64_t)Ml, (uint64_t)world};
    uint64_t s3[2] = {(uint64_t)N * 2, (uint64_t)Ml * N * 2};
    uint32_t b3[3] = {64, DBM, 1};
    if (reinterpret_cast<uintptr_t>(stage[r]) & 15) return -4;
    int e3 = make_tmap_bf16(&st_maps.m[r], stage[r], 3, d3, s3, b3);
    if (e3) return 3000 + e3;
  }
  for (int r = world; r < DMAX_RANKS; ++r) st_maps.m[r] = st_maps.m[0];
  DistParams p;
  memset(&p, 0, sizeof(p));
  p.Ml = Ml; p.N = N; p.K = Kl; p.rank = rank; p.world = world; p.epoch = epoch;
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.phase_mask = phase_mask; p.budget = budget; p.status = static_cast<KernelStatus*>(status);
  if (bn == 256) return launch_dist<1, 256, 4>(ta, tb, st_maps, st, ct, p, stream);
  return launch_dist<1, 128, 6>(ta, tb, st_maps, st, ct, p, stream);
}

extern "C" int otb_dist_publish(void* const* ready, int rank, int world, unsigned epoch, cudaStream_t stream) {
  if (world < 1 || world > DMAX_RANKS) return -9;
  PtrArray r;
  memset(&r, 0, sizeof(r));
  for (int i = 0; i < world; ++i) r.p[i] = ready[i];
  publish_kernel<<<1, 32, 0, stream>>>(r, rank, world, epoch);
  return (int)cudaGetLastError();
}
