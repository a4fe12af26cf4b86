// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory ring -> tcgen05.mma with the
// accumulator in tensor memory -> fused epilogue.
//
//   D[M,N] = A * B  (fp32 accumulate), then optionally  + bias[N], + residual[M,N], += D_old,
//   or the gated-MLP epilogue  out2[M,N/2] = act(gate) * up  on block-interleaved columns.
//
// Operand layouts (bf16, row-major storage):
//   A "K-major"  : stored [M][K]            A "MN-major": stored [K][M]
//   B "K-major"  : stored [N][K]            B "MN-major": stored [K][N]
// which covers  x @ W^T (NT), dY @ W (NN) and dY^T @ X (TN) without any transposed copy.
//
// One CTA per SM, 6 warps: warp 0 issues TMA loads, warp 1 issues MMAs (one elected lane each),
// warps 2..5 drain the accumulator (TMEM lanes 32*(warp%4) ..) while the MMA warp already works on
// the next tile in the second accumulator buffer.
#include "common.cuh"

namespace otb {

constexpr int BM = 128;
constexpr int BK = 64;   // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr unsigned KID_GEMM = 1;

enum EpiFlags {
  EPI_BIAS = 1,        // + bias[N] (bf16)
  EPI_RESIDUAL = 2,    // + residual[M,N] (bf16)
  EPI_ACCUM = 4,       // out += result (read-modify-write of out)
  EPI_OUT_F32 = 8,     // out is fp32 instead of bf16
  EPI_GLU_GELU = 16,   // out2[:, j] = gelu_tanh(gate_j) * up_j, columns interleaved in blocks of 32
  EPI_GLU_SILU = 32,   // same with silu
  EPI_BIAS_F32 = 64,   // bias is fp32
  EPI_NO_OUT = 128,    // skip the plain store of D (GLU inference: only out2 is wanted)
  EPI_ACT_GELU = 256,  // out = gelu_tanh(result + bias)
};

struct GemmParams {
  int M, N, K;
  int a_mn_major, b_mn_major;
  void* out;
  long long ldo;
  const void* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  __nv_bfloat16* out2;
  long long ldo2;
  int flags;
  KernelStatus* status;
};

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;  // + alignment slack
};

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_idx, int& n_idx) {
  constexpr int GROUP = 8;
  int group_size = GROUP * num_n;
  int g = tile / group_size;
  int first_m = g * GROUP;
  int gm = min(num_m - first_m, GROUP);
  int r = tile - g * group_size;
  m_idx = first_m + r % gm;
  n_idx = r / gm;
}

// Epilogue of one 128 x BN accumulator tile: warp `quad` (TMEM lanes 32*quad ..) drains its 32 rows, 32 columns at a
// time, and applies the fused epilogue (bias / activation / residual / accumulate / gated-MLP forward).
template <int BN>
__device__ __forceinline__ void epilogue_tile(const GemmParams& p, const int flags, const bool glu, const int m0,
                                              const int n0, const int quad, const int lane, const uint32_t tmem_base,
                                              const int acc) {
  const int row = m0 + quad * 32 + lane;
  const bool row_ok = row < p.M;
  const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + acc * BN;
#pragma unroll 1
  for (int c = 0; c < BN / 32; c += (glu ? 2 : 1)) {
    __syncwarp();
    uint32_t r[32];
    tmem_ld_x32(taddr + c * 32, r);
    uint32_t r2[32];
    if (glu) tmem_ld_x32(taddr + (c + 1) * 32, r2);
    tmem_wait_ld();
    const int col0 = n0 + c * 32;
    const bool active = row_ok && col0 < p.N;
    if (active && !(flags & EPI_NO_OUT)) {
      const int nchunks = glu ? 2 : 1;
      for (int h = 0; h < nchunks; ++h) {
        uint32_t* rr = h ? r2 : r;
        const int cbase = col0 + h * 32;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int col = cbase + j * 8;
          if (col >= p.N) break;
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(rr[j * 8 + e]);
          if (flags & EPI_BIAS) {
            if (flags & EPI_BIAS_F32) {
              const float4* bp = reinterpret_cast<const float4*>(static_cast<const float*>(p.bias) + col);
              float4 b0 = __ldg(bp), b1 = __ldg(bp + 1);
              v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
              v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
            } else {
              uint4 bb = __ldg(reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.bias) + col));
              float2 f;
              f = unpack_bf16(bb.x); v[0] += f.x; v[1] += f.y;
              f = unpack_bf16(bb.y); v[2] += f.x; v[3] += f.y;
              f = unpack_bf16(bb.z); v[4] += f.x; v[5] += f.y;
              f = unpack_bf16(bb.w); v[6] += f.x; v[7] += f.y;
            }
          }
          if (flags & EPI_ACT_GELU) {
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = gelu_tanh_f(v[e]);
          }
          if (flags & EPI_RESIDUAL) {
            uint4 bb = *reinterpret_cast<const uint4*>(p.residual + (long long)row * p.ldr + col);
            float2 f;
            f = unpack_bf16(bb.x); v[0] += f.x; v[1] += f.y;
            f = unpack_bf16(bb.y); v[2] += f.x; v[3] += f.y;
            f = unpack_bf16(bb.z); v[4] += f.x; v[5] += f.y;
            f = unpack_bf16(bb.w); v[6] += f.x; v[7] += f.y;
          }
          if (flags & EPI_OUT_F32) {
            float4* op = reinterpret_cast<float4*>(static_cast<float*>(p.out) + (long long)row * p.ldo + col);
            if (flags & EPI_ACCUM) {
              float4 o0 = op[0], o1 = op[1];
              v[0] += o0.x; v[1] += o0.y; v[2] += o0.z; v[3] += o0.w;
              v[4] += o1.x; v[5] += o1.y; v[6] += o1.z; v[7] += o1.w;
            }
            op[0] = make_float4(v[0], v[1], v[2], v[3]);
            op[1] = make_float4(v[4], v[5], v[6], v[7]);
          } else {
            uint4* op = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + (long long)row * p.ldo + col);
            if (flags & EPI_ACCUM) {
              uint4 bb = *op;
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
            *op = o;
          }
        }
      }
    }
    if (active && glu) {
      // gate = r (columns col0..col0+31), up = r2; output column = col0/2 .. +31
      const int ocol0 = col0 >> 1;
      __nv_bfloat16* op = p.out2 + (long long)row * p.ldo2 + ocol0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float g = __uint_as_float(r[j * 8 + e]);
          float u = __uint_as_float(r2[j * 8 + e]);
          // match the unfused path: gate/up are rounded to bf16 before the activation
          g = __bfloat162float(__float2bfloat16(g));
          u = __bfloat162float(__float2bfloat16(u));
          float a = (flags & EPI_GLU_GELU) ? gelu_tanh_f(g) : silu_f(g);
          v[e] = a * u;
        }
        uint4 o;
        o.x = pack_bf16(v[0], v[1]);
        o.y = pack_bf16(v[2], v[3]);
        o.z = pack_bf16(v[4], v[5]);
        o.w = pack_bf16(v[6], v[7]);
        *reinterpret_cast<uint4*>(op + j * 8) = o;
      }
    }
  }
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
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
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 128 / 256 / 512: powers of two >= 32

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
    tma_prefetch_desc(&tma_a);
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
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        int mi, ni;
        tile_coords(tile, num_m, num_n, mi, ni);
        const int m0 = mi * BM, n0 = ni * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, KID_GEMM, 1, stage);
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
          const int k0 = kb * BK;
          if (!p.a_mn_major) {
            tma_load_2d(sa, &tma_a, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * 8192, &tma_a, &full_bar[stage], m0 + 64 * i, k0);
          }
          if (!p.b_mn_major) {
            tma_load_2d(sb, &tma_b, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * 8192, &tma_b, &full_bar[stage], n0 + 64 * i, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn_major, p.b_mn_major);
      const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u, b_lbo = p.b_mn_major ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn_major ? 2048u : 32u, b_kstep = p.b_mn_major ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, KID_GEMM, 2, acc);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&full_bar[stage], phase, abort_flag, p.status, KID_GEMM, 3, stage);
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t ad = make_smem_desc(sa + k * a_kstep, a_lbo, 1024);
            uint64_t bd = make_smem_desc(sb + k * b_kstep, b_lbo, 1024);
            umma_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
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
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    const int flags = p.flags;
    const bool glu = (flags & (EPI_GLU_GELU | EPI_GLU_SILU)) != 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int mi, ni;
      tile_coords(tile, num_m, num_n, mi, ni);
      const int m0 = mi * BM, n0 = ni * BN;
      mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, KID_GEMM, 4, acc);
      tc_fence_after();
      epilogue_tile<BN>(p, flags, glu, m0, n0, quad, lane, tmem_base, acc);
      tc_fence_before();
      mbar_arrive(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      // a wait gave up: let TMA copies and MMAs still in flight finish before releasing resources
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------ CTA-pair kernel
// Two CTAs of a cluster (two SMs) work on ONE 256 x 256 output tile with `tcgen05.mma.cta_group::2`: CTA r of the
// pair owns rows [128 r, 128 r + 128) of the tile (its own A tile, its own accumulator in its own tensor memory) and
// loads only HALF of the B tile (columns [128 r, 128 r + 128)); the tensor cores of both SMs read both halves.  Per
// CTA that is 256 operand rows per 128 x 256 of output instead of 384: a third less traffic from L2 into shared
// memory, and six pipeline stages of 32 KB instead of four of 48 KB.
//
// Protocol (rank 0 of the pair = leader; barriers sit at the same shared-memory offsets in both CTAs):
//   full[s]   (leader's only)  armed by the leader's producer with the bytes of BOTH CTAs' loads; every TMA load of
//                              either CTA completes on it (the non-leader addresses it through the pair's window).
//   empty[s]  (one per CTA)    the leader's MMA thread commits to both with one multicast commit.
//   tfull[b]  (one per CTA)    same multicast commit once a tile's last MMA is issued: both epilogues start.
//   tempty[b] (leader's only)  256 arrivals: the 128 epilogue threads of each CTA, the peer's by a remote arrive.
// Loads are plain (no multicast).  All waits are bounded as in the single-CTA kernel.
constexpr unsigned KID_GEMM2 = 6;
constexpr uint32_t PEER_BIT_MASK = 0xFEFFFFFFu;      // clears the CTA-rank bit of a shared-window address: rank 0's

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 2-D tiled load whose completion is counted on the LEADER CTA's barrier at the same offset as `bar`.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar) & PEER_BIT_MASK), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive, once all MMAs issued so far have completed, on the barrier at `bar`'s offset in BOTH CTAs of the pair.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}
// Arrive on the leader's barrier at `bar`'s offset (local for the leader, remote for its peer).
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & PEER_BIT_MASK) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

template <int STAGES>
struct SmemLayout2 {
  static constexpr int A_BYTES = BM * BK * 2;          // this CTA's 128 rows of A
  static constexpr int B_BYTES = 128 * BK * 2;         // this CTA's half (128 columns) of the 256-wide B tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;
};

template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, GemmParams p) {
  constexpr int BN = 256, BM2 = 2 * BM;
  using L = SmemLayout2<STAGES>;
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
  const uint32_t rank = cluster_ctarank();             // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_m = (p.M + BM2 - 1) / BM2;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 256);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                  // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int tile = pair; tile < num_tiles; tile += num_pairs) {
        int mi, ni;
        tile_coords(tile, num_m, num_n, mi, ni);
        const int m0 = mi * BM2 + (int)rank * BM, n0 = ni * BN + (int)rank * 128;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, KID_GEMM2, 1, stage);
          uint8_t* sa = smem + stage * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * L::STAGE_BYTES);
          const int k0 = kb * BK;
          if (!p.a_mn_major) {
            tma_load_2d_pair(sa, &tma_a, &full_bar[stage], k0, m0);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d_pair(sa + i * 8192, &tma_a, &full_bar[stage], m0 + 64 * i, k0);
          }
          if (!p.b_mn_major) {
            tma_load_2d_pair(sb, &tma_b, &full_bar[stage], k0, n0);
          } else {
#pragma unroll
            for (int i = 0; i < 2; ++i) tma_load_2d_pair(sb + i * 8192, &tma_b, &full_bar[stage], n0 + 64 * i, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && elect_one()) {
      const uint32_t idesc = make_idesc_bf16(BM2, BN, p.a_mn_major, p.b_mn_major);
      const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u, b_lbo = p.b_mn_major ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn_major ? 2048u : 32u, b_kstep = p.b_mn_major ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int tile = pair; tile < num_tiles; tile += num_pairs) {
        mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag, p.status, KID_GEMM2, 2, acc);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&full_bar[stage], phase, abort_flag, p.status, KID_GEMM2, 3, stage);
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t ad = make_smem_desc(sa + k * a_kstep, a_lbo, 1024);
            uint64_t bd = make_smem_desc(sb + k * b_kstep, b_lbo, 1024);
            umma_ss_pair(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage]);          // frees the stage in BOTH CTAs once these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        umma_commit_pair(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int flags = p.flags;
    const bool glu = (flags & (EPI_GLU_GELU | EPI_GLU_SILU)) != 0;
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      int mi, ni;
      tile_coords(tile, num_m, num_n, mi, ni);
      const int m0 = mi * BM2 + (int)rank * BM, n0 = ni * BN;
      mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, p.status, KID_GEMM2, 4, acc);
      tc_fence_after();
      epilogue_tile<BN>(p, flags, glu, m0, n0, quad, lane, tmem_base, acc);
      tc_fence_before();
      mbar_arrive_leader(&tempty_bar[acc]);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                  // nobody leaves while its peer may still signal its barriers or read its tiles
  if (warp == 1) {
    if (*abort_flag) {
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------ host
static int g_num_sms = 0;
static int g_pair_default = 1;     // products that do not name a tile use the CTA-pair kernel when they are large

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  using L = SmemLayout<BN, STAGES>;
  static bool configured = false;
  auto kern = gemm_bf16_kernel<BN, STAGES>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  int num_tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  int grid = num_tiles < g_num_sms ? num_tiles : g_num_sms;
  kern<<<grid, 192, L::TOTAL, stream>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

template <int STAGES>
static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t stream) {
  using L = SmemLayout2<STAGES>;
  static bool configured = false;
  auto kern = gemm2_bf16_kernel<STAGES>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int num_tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + 255) / 256);
  int pairs = g_num_sms / 2;
  if (num_tiles < pairs) pairs = num_tiles;
  kern<<<2 * pairs, 192, L::TOTAL, stream>>>(ta, tb, p);     // cluster size 2 comes from __cluster_dims__
  return (int)cudaGetLastError();
}

}  // namespace otb

using namespace otb;

// Returns 0 on success, a CUDA/driver error code, or a negative argument-check code.
extern "C" int otb_gemm_bf16(const void* A, const void* B, void* out, int M, int N, int K, long long lda,
                             long long ldb, long long ldo, int a_mn_major, int b_mn_major, const void* bias,
                             const void* residual, long long ldr, void* out2, long long ldo2, int flags,
                             int bn_override, void* status, cudaStream_t stream) {
  // bn_override: 0 = choose; 64 / 128 / 256 = that column tile on one CTA; 512 = the CTA-pair kernel (256 x 256 tiles)
  if (M <= 0 || N <= 0 || K <= 0) return -2;
  if ((lda % 8) || (ldb % 8) || (ldo % 8) || (N % 8)) return -3;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out)) & 15) return -4;
  if ((flags & EPI_RESIDUAL) && ((ldr % 8) || (reinterpret_cast<uintptr_t>(residual) & 15))) return -5;
  if ((flags & (EPI_GLU_GELU | EPI_GLU_SILU)) && ((N % 64) || (ldo2 % 8) || out2 == nullptr)) return -6;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) return -7;
  }
  int bn = bn_override;
  // Big products: two SMs per 256 x 256 tile (measured 1.10 - 1.26x the single-CTA kernel on the training shapes).
  // The exception is a weight gradient with a narrow output (both operands MN-major, N <= 2048), where it measured
  // 0.97x.
  if (bn == 0 && g_pair_default && M >= 1024 && N >= 1024 && (long long)((M + 255) / 256) * ((N + 255) / 256) >= 74 &&
      !(a_mn_major && b_mn_major && N <= 2048))
    bn = 512;
  if (bn == 0) {
    int m_tiles = (M + BM - 1) / BM;
    if ((long long)m_tiles * ((N + 255) / 256) >= g_num_sms || N >= 4096) bn = 256;
    else if ((long long)m_tiles * ((N + 127) / 128) >= g_num_sms / 2 || N >= 1024) bn = 128;
    else bn = 64;
    if (N <= 64) bn = 64;
    else if (N <= 128 && bn > 128) bn = 128;
  }
  CUtensorMap ta, tb;
  {
    uint64_t dims[2], strides[1];
    uint32_t box[2];
    if (!a_mn_major) { dims[0] = K; dims[1] = M; box[0] = 64; box[1] = BM; }
    else { dims[0] = M; dims[1] = K; box[0] = 64; box[1] = 64; }
    strides[0] = (uint64_t)lda * 2;
    int r = make_tmap_bf16(&ta, A, 2, dims, strides, box);
    if (r) return 1000 + r;
    if (!b_mn_major) { dims[0] = K; dims[1] = N; box[0] = 64; box[1] = bn == 512 ? 128 : bn; }
    else { dims[0] = N; dims[1] = K; box[0] = 64; box[1] = 64; }
    strides[0] = (uint64_t)ldb * 2;
    r = make_tmap_bf16(&tb, B, 2, dims, strides, box);
    if (r) return 2000 + r;
  }
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.out = out; p.ldo = ldo;
  p.bias = bias;
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.out2 = static_cast<__nv_bfloat16*>(out2); p.ldo2 = ldo2;
  p.flags = flags;
  p.status = static_cast<KernelStatus*>(status);
  switch (bn) {
    case 256: return launch_gemm<256, 4>(ta, tb, p, stream);
    case 128: return launch_gemm<128, 6>(ta, tb, p, stream);
    case 64: return launch_gemm<64, 8>(ta, tb, p, stream);
    case 512: return launch_gemm_pair<6>(ta, tb, p, stream);
    default: return -8;
  }
}

// Switches the CTA-pair kernel on / off as the default for large products (benchmarks compare the two).
extern "C" void otb_gemm_set_pair_default(int on) { g_pair_default = on ? 1 : 0; }
