// Tensor-parallel linears fused with their collective over peer memory (NVLink / NVSwitch), sm_100a.
//
//   all-gather -> GEMM   (column-parallel linear on a sequence-sharded activation)
//       D[W*Ml, N] = concat_r(A_r[Ml, K]) * B[N, K]^T (+ bias)
//       Every rank keeps only its own rows A_r in a peer-visible buffer.  The TMA producer warp reads the
//       A tile of segment r straight out of rank r's memory through a per-rank tensor map (plain tiled
//       loads, no multicast), so the gather is never materialised and the link transfer of segment r+1
//       overlaps the tensor-core work on segment r.  Local rows go first; a remote segment is touched
//       only after its owner published it (per-source ready flag, release/acquire at system scope).
//
//   GEMM -> reduce-scatter   (row-parallel linear that leaves a sequence-sharded result)
//       out_d[Ml, N] = sum_r A_r[rows of d, Kl] * B_r[N, Kl]^T (+ bias) (+ residual)
//       The epilogue stores each bf16 partial tile directly into the destination rank's staging buffer
//       (peer stores; tiles bound for remote ranks are scheduled first, own rows last) and bumps a per
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
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

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
  int phase_mask;
  long long budget;
  KernelStatus* status;
};

template <int BN, int STAGES>
struct DistSmem {
  static constexpr int A_BYTES = DBM * DBK * 2;
  static constexpr int B_BYTES = BN * DBK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;
};

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

// MODE 0: all-gather -> GEMM.  MODE 1: GEMM -> reduce-scatter.
template <int MODE, int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_dist_kernel(const __grid_constant__ TmapArray tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ PtrArray stage, const __grid_constant__ PtrArray counters, DistParams p) {
  using L = DistSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
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
      unsigned seen = 1u << p.rank;  // sources whose ready flag was already observed
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        if (*abort_flag) break;  // a wait gave up: issue no further copies
        int seg, mi, ni;
        dist_tile_coords(tile, m_per_seg, num_n, seg, mi, ni);
        const int n0 = ni * BN;
        const CUtensorMap* amap;
        int a_row;
        if (MODE == 0) {
          const int src = (p.rank + seg) % W;  // own rows first, then the peers in ring order
          if (!(seen & (1u << src))) {
            wait_flag_ge(p.ready + src, p.epoch, abort_flag, p.budget, p.status, KID, 5, (unsigned)src);
            seen |= 1u << src;
          }
          amap = &tma_a.m[src];
          a_row = mi * DBM;  // row inside rank src's shard
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
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;
    const int et = quad * 32 + lane;  // 0..127 inside the epilogue group
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int seg, mi, ni;
      dist_tile_coords(tile, m_per_seg, num_n, seg, mi, ni);
      const int n0 = ni * BN;
      const int lrow = mi * DBM + quad * 32 + lane;  // row inside the segment
      const bool row_ok = lrow < p.Ml;
      __nv_bfloat16* dst_row;
      int peer = 0;
      if (MODE == 0) {
        const int src = (p.rank + seg) % W;
        dst_row = p.out + ((long long)src * p.Ml + lrow) * p.ldo;
      } else {
        peer = (p.rank + 1 + seg) % W;
        // staging of rank `peer`: [W sources][Ml][N]
        dst_row = static_cast<__nv_bfloat16*>(stage.p[peer]) + ((long long)p.rank * p.Ml + lrow) * p.N;
      }
      mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, KID, 4, acc);
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + acc * BN;
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
            if (MODE == 0 && p.bias != nullptr) {
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
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
      if (MODE == 1) {
        // make this tile's peer stores visible, then count it at the destination
        __threadfence_system();
        epi_bar_sync();
        if (et == 0) {
          unsigned* cnt = static_cast<unsigned*>(counters.p[peer]) + p.rank * m_per_seg + mi;
          red_release_sys_add(cnt, 1u);
        }
      }
    }

    if (MODE == 1 && (p.phase_mask & 2)) {
      // -------------------------------------------------------------- reduce tail: my rows, all sources
      const __nv_bfloat16* my_stage = static_cast<const __nv_bfloat16*>(stage.p[p.rank]);
      const unsigned* my_cnt = static_cast<const unsigned*>(counters.p[p.rank]);
      const unsigned target = p.epoch * (unsigned)num_n;
      const int vec_per_row = p.N >> 3;
      for (int mb = blockIdx.x; mb < m_per_seg; mb += gridDim.x) {
        // the 4 epilogue warps of this CTA reduce row block `mb`; wait for every source first
        if (et < W) wait_flag_ge(my_cnt + et * m_per_seg + mb, target, abort_flag, p.budget, p.status, KID, 6, et);
        epi_bar_sync();
        const int rows = min(DBM, p.Ml - mb * DBM);
        const long long total = (long long)rows * vec_per_row;
        for (long long t = et; t < total; t += 128) {
          const int rr = (int)(t / vec_per_row);
          const int cv = (int)(t - (long long)rr * vec_per_row);
          const int row = mb * DBM + rr;
          const int col = cv * 8;
          float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          for (int s = 0; s < W; ++s) {
            const uint4 u = __ldcg(reinterpret_cast<const uint4*>(my_stage + ((long long)s * p.Ml + row) * p.N + col));
            float2 f;
            f = unpack_bf16(u.x); a[0] += f.x; a[1] += f.y;
            f = unpack_bf16(u.y); a[2] += f.x; a[3] += f.y;
            f = unpack_bf16(u.z); a[4] += f.x; a[5] += f.y;
            f = unpack_bf16(u.w); a[6] += f.x; a[7] += f.y;
          }
          if (p.bias != nullptr) {
            uint4 bb = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
            float2 f;
            f = unpack_bf16(bb.x); a[0] += f.x; a[1] += f.y;
            f = unpack_bf16(bb.y); a[2] += f.x; a[3] += f.y;
            f = unpack_bf16(bb.z); a[4] += f.x; a[5] += f.y;
            f = unpack_bf16(bb.w); a[6] += f.x; a[7] += f.y;
          }
          if (p.residual != nullptr) {
            uint4 bb = *reinterpret_cast<const uint4*>(p.residual + (long long)row * p.ldr + col);
            float2 f;
            f = unpack_bf16(bb.x); a[0] += f.x; a[1] += f.y;
            f = unpack_bf16(bb.y); a[2] += f.x; a[3] += f.y;
            f = unpack_bf16(bb.z); a[4] += f.x; a[5] += f.y;
            f = unpack_bf16(bb.w); a[6] += f.x; a[7] += f.y;
          }
          uint4 o;
          o.x = pack_bf16(a[0], a[1]);
          o.y = pack_bf16(a[2], a[3]);
          o.z = pack_bf16(a[4], a[5]);
          o.w = pack_bf16(a[6], a[7]);
          *reinterpret_cast<uint4*>(p.out + (long long)row * p.ldo + col) = o;
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
static int launch_dist(const TmapArray& ta, const CUtensorMap& tb, const PtrArray& stage, const PtrArray& counters,
                       const DistParams& p, cudaStream_t stream) {
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
  kern<<<grid, 192, L::TOTAL, stream>>>(ta, tb, stage, counters, p);
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

// a_shards[r]: rank r's [Ml, K] rows (lda elements per row) as mapped into THIS process; B: [N, K] local
// weight shard; out: [world*Ml, N].  ready: local unsigned[world]; ready[r] >= epoch once rank r published.
extern "C" int otb_ag_gemm_bf16(void* const* a_shards, const void* B, void* out, int Ml, int N, int K, long long lda,
                                long long ldb, long long ldo, const void* bias, const void* ready, int rank, int world,
                                unsigned epoch, long long budget, void* status, cudaStream_t stream) {
  int rc = dist_common_checks(Ml, N, K, rank, world);
  if (rc) return rc;
  if ((lda % 8) || (ldb % 8) || (ldo % 8)) return -3;
  const int bn = pick_bn(Ml, N, world);
  TmapArray ta;
  CUtensorMap tb;
  uint64_t dims[2], strides[1];
  uint32_t box[2];
  for (int r = 0; r < world; ++r) {
    if (reinterpret_cast<uintptr_t>(a_shards[r]) & 15) return -4;
    dims[0] = K; dims[1] = Ml; box[0] = 64; box[1] = DBM;
    strides[0] = (uint64_t)lda * 2;
    int e = make_tmap_bf16(&ta.m[r], a_shards[r], 2, dims, strides, box);
    if (e) return 1000 + e;
  }
  for (int r = world; r < DMAX_RANKS; ++r) ta.m[r] = ta.m[0];
  dims[0] = K; dims[1] = N; box[0] = 64; box[1] = bn;
  strides[0] = (uint64_t)ldb * 2;
  int e = make_tmap_bf16(&tb, B, 2, dims, strides, box);
  if (e) return 2000 + e;
  PtrArray none;
  memset(&none, 0, sizeof(none));
  DistParams p;
  memset(&p, 0, sizeof(p));
  p.Ml = Ml; p.N = N; p.K = K; p.rank = rank; p.world = world; p.epoch = epoch;
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.ready = static_cast<const unsigned*>(ready);
  p.phase_mask = 3; p.budget = budget; p.status = static_cast<KernelStatus*>(status);
  if (bn == 256) return launch_dist<0, 256, 4>(ta, tb, none, none, p, stream);
  return launch_dist<0, 128, 6>(ta, tb, none, none, p, stream);
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
  memset(&st, 0, sizeof(st));
  memset(&ct, 0, sizeof(ct));
  for (int r = 0; r < world; ++r) {
    st.p[r] = stage[r];
    ct.p[r] = counters[r];
  }
  DistParams p;
  memset(&p, 0, sizeof(p));
  p.Ml = Ml; p.N = N; p.K = Kl; p.rank = rank; p.world = world; p.epoch = epoch;
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.phase_mask = phase_mask; p.budget = budget; p.status = static_cast<KernelStatus*>(status);
  if (bn == 256) return launch_dist<1, 256, 4>(ta, tb, st, ct, p, stream);
  return launch_dist<1, 128, 6>(ta, tb, st, ct, p, stream);
}

extern "C" int otb_dist_publish(void* const* ready, int rank, int world, unsigned epoch, cudaStream_t stream) {
  if (world < 1 || world > DMAX_RANKS) return -9;
  PtrArray r;
  memset(&r, 0, sizeof(r));
  for (int i = 0; i < world; ++i) r.p[i] = ready[i];
  publish_kernel<<<1, 32, 0, stream>>>(r, rank, world, epoch);
  return (int)cudaGetLastError();
}
