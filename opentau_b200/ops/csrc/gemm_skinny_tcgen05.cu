// Weight-streaming bf16 GEMM for few rows (inference: a 51-token action suffix, a ~200-token prefix, a few hundred
// vision patches) on sm_100a:   out[M,N] = X[M,K] * W[N,K]^T   with M small.
//
// The persistent 128 x BN GEMM turns such a product into N/BN tiles: 8..40 CTAs stream the whole weight matrix while
// a hundred SMs idle, and the weights of an M = 2-tile problem are fetched once per row tile.  Here the operands are
// swapped and the reduction dimension is split:
//
//   * the WEIGHT rows are the 128-row M operand of tcgen05.mma, the tokens are the N operand (64 / 128 / 256 wide),
//     so every weight element crosses shared memory exactly once per 256 tokens and the accumulator
//     D^T[128 weight rows, tokens] sits in TMEM with one weight row per lane;
//   * K is split over the CTAs of a thread-block cluster (1 to 8): grid = (N/128, splits, token chunks), so even
//     an N = 1024 projection puts 64 CTAs to work.  Each CTA leaves its fp32 partial tile in its own shared memory
//     (the TMA ring is free by then), the cluster synchronises, and every CTA reduces 1/splits of the tile over
//     distributed shared memory in fixed rank order (deterministic, no global workspace, no atomics) and applies the
//     epilogue: bias, GELU, residual, bf16 / fp32 store, or the gated-MLP product on block-interleaved rows.
//
// Warp roles as in the big GEMM: warp 0 TMA producer, warp 1 MMA issuer, warps 2..5 TMEM readers; all six warps take
// part in the cluster reduction.  Every wait is bounded; a CTA whose wait gave up still arrives at both cluster
// barriers, so its peers are never left waiting.
#include "common.cuh"

namespace otb {

constexpr unsigned KID_SKINNY = 4;
constexpr int SK_BW = 128;  // weight rows per CTA (UMMA M)
constexpr int SK_BK = 64;
constexpr int SK_UMMA_K = 16;

enum SkinnyFlags {  // same values as the big GEMM's epilogue flags
  SK_BIAS = 1,
  SK_RESIDUAL = 2,
  SK_OUT_F32 = 8,
  SK_GLU_GELU = 16,
  SK_GLU_SILU = 32,
  SK_BIAS_F32 = 64,
  SK_NO_OUT = 128,
  SK_ACT_GELU = 256,
  SK_GATE = 512,       // with SK_RESIDUAL: out = residual + gate * result (adaptive-norm gate of the residual branch)
};

struct SkinnyParams {
  int M, N, K;
  void* out;
  long long ldo;
  const void* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  __nv_bfloat16* out2;
  long long ldo2;
  const __nv_bfloat16* gate;      // rows of N gates; row (m / rows_per_gate), row stride gate_stride
  long long gate_stride;
  int rows_per_gate;
  int flags;
  int splits;
  KernelStatus* status;
};

template <int NT, int STAGES>
struct SkinnySmem {
  static constexpr int W_BYTES = SK_BW * SK_BK * 2;
  static constexpr int X_BYTES = NT * SK_BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int PARTIAL_BYTES = NT * SK_BW * 4;   // fp32 partial tile, overlays the ring after the last MMA
  static_assert(PARTIAL_BYTES <= BAR_OFFSET, "partial tile does not fit in the ring");
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 1) * 8 + 16 + 1024;
};

__device__ __forceinline__ void cluster_sync_all() {
  __syncwarp();   // the role branches above diverge inside warps 0 and 1; the aligned barrier wants whole warps
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// sum of one partial-tile element over the S ranks of the cluster, in rank order; the loads are issued together
__device__ __forceinline__ float reduce_ranks(uint32_t local_addr, int S) {
  float v[8];
#pragma unroll
  for (int s = 0; s < 8; ++s) v[s] = s < S ? ld_dsmem_f32(local_addr, (uint32_t)s) : 0.f;
  float acc = v[0];
#pragma unroll
  for (int s = 1; s < 8; ++s) acc += v[s];
  return acc;
}

// bias / activation / residual / store of one element
__device__ __forceinline__ void skinny_store(const SkinnyParams& p, int m, int n, float v) {
  const int flags = p.flags;
  if (flags & SK_BIAS) {
    v += (flags & SK_BIAS_F32) ? __ldg(static_cast<const float*>(p.bias) + n)
                               : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n]);
  }
  if (flags & SK_ACT_GELU) v = gelu_tanh_f(v);
  if (flags & SK_RESIDUAL) {
    if (flags & SK_GATE) v *= __bfloat162float(p.gate[(long long)(m / p.rows_per_gate) * p.gate_stride + n]);
    v += __bfloat162float(p.residual[(long long)m * p.ldr + n]);
  }
  if (flags & SK_OUT_F32) {
    static_cast<float*>(p.out)[(long long)m * p.ldo + n] = v;
  } else {
    static_cast<__nv_bfloat16*>(p.out)[(long long)m * p.ldo + n] = __float2bfloat16(v);
  }
}

template <int NT, int STAGES>
__global__ void __launch_bounds__(192, NT <= 128 ? 2 : 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x,
                   SkinnyParams p) {
  using L = SkinnySmem<NT, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* partial = reinterpret_cast<float*>(smem);   // [token][128 weight rows], valid after the last MMA retired

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = p.splits;
  const int split = (int)cluster_ctarank();          // the cluster spans gridDim.y == S
  const int n0 = blockIdx.x * SK_BW;
  const int m_base = blockIdx.z * NT;
  const int m_valid = min(NT, p.M - m_base);
  const int num_kb = (p.K + SK_BK - 1) / SK_BK;
  const int per = (num_kb + S - 1) / S;
  const int kb0 = split * per;
  const int kb1 = min(num_kb, kb0 + per);
  const int nkb = max(kb1 - kb0, 0);
  const bool glu = (p.flags & (SK_GLU_GELU | SK_GLU_SILU)) != 0;
  const bool direct = S == 1 && !glu;                // straight from TMEM to global memory

  const int early = min(STAGES, nkb);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tfull_bar, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_x);
    // The weights do not depend on the preceding kernel: the first ring of weight tiles is requested at once, before
    // the TMEM allocation, the block barrier and the dependency wait, so that their HBM latency overlaps all three
    // (and, under programmatic dependent launch, the predecessor's tail).  Activations follow after the wait.
    for (int i = 0; i < early; ++i) {
      mbar_expect_tx(&full_bar[i], L::STAGE_BYTES);
      tma_load_2d(smem + i * L::STAGE_BYTES, &tma_w, &full_bar[i], (kb0 + i) * SK_BK, n0);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, NT);   // 64 / 128 / 256 columns
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();                 // after the TMEM allocation (see common.cuh)

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      pdl_wait();
      for (int i = 0; i < early; ++i)
        tma_load_2d(smem + i * L::STAGE_BYTES + L::W_BYTES, &tma_x, &full_bar[i], (kb0 + i) * SK_BK, m_base);
      int stage = early == STAGES ? 0 : early;
      uint32_t phase = early == STAGES ? 1 : 0;
      for (int kb = kb0 + early; kb < kb1; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, KID_SKINNY, 1, stage)) break;
        uint8_t* sw = smem + stage * L::STAGE_BYTES;
        uint8_t* sx = sw + L::W_BYTES;
        mbar_expect_tx(&full_bar[stage], L::STAGE_BYTES);
        tma_load_2d(sw, &tma_w, &full_bar[stage], kb * SK_BK, n0);
        tma_load_2d(sx, &tma_x, &full_bar[stage], kb * SK_BK, m_base);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_bf16(SK_BW, NT, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      for (int i = 0; i < nkb; ++i) {
        if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, KID_SKINNY, 2, stage)) break;
        tc_fence_after();
        const uint32_t sw = smem_u32(smem + stage * L::STAGE_BYTES);
        const uint32_t sx = sw + L::W_BYTES;
#pragma unroll
        for (int k = 0; k < SK_BK / SK_UMMA_K; ++k) {
          uint64_t wd = make_smem_desc(sw + k * 32u, 16u, 1024);
          uint64_t xd = make_smem_desc(sx + k * 32u, 16u, 1024);
          umma_ss(tmem_base, wd, xd, idesc, (i | k) != 0 ? 1u : 0u);
        }
        umma_commit(&empty_bar[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      umma_commit(tfull_bar);   // fires when every MMA above has retired (at once if there was none)
    }
  } else {
    // ------------------------------------------------------------------ TMEM readers (warps 2..5)
    pdl_wait();                                       // residual / gate / output buffers belong to the predecessor
    const int quad = warp & 3;                        // TMEM lane quadrant this warp may read
    const int wrow = quad * 32 + lane;                // weight row inside the tile
    const int n = n0 + wrow;
    bool ok = mbar_wait(tfull_bar, 0, abort_flag, p.status, KID_SKINNY, 3, 0);
    tc_fence_after();
    const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16);
    const int nchunk = (m_valid + 31) / 32;
#pragma unroll 1
    for (int c = 0; c < nchunk; ++c) {
      uint32_t r[32];
      if (nkb > 0 && ok) {
        __syncwarp();
        tmem_ld_x32(taddr + c * 32, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = 0u;       // this split owns no k-block (or gave up): contributes zeros
      }
      if (direct) {
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int m = c * 32 + j;
            if (m < m_valid) skinny_store(p, m_base + m, n, __uint_as_float(r[j]));
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int m = c * 32 + j;
          if (m < m_valid) partial[m * SK_BW + wrow] = __uint_as_float(r[j]);
        }
      }
    }
    tc_fence_before();
  }

  // ---------------------------------------------------------------------- cluster reduction + epilogue
  cluster_sync_all();                                 // every CTA's partial tile is complete and visible
  pdl_wait();                                         // warps 0 / 1 join the reduction: they write outputs too
  if (!direct && !*abort_flag) {
    const uint32_t pbase = smem_u32(partial);
    if (!(p.flags & SK_NO_OUT)) {
      // plain output: this rank reduces weight rows [r0, r0 + rows) (the last rank takes the remainder)
      const int rows_per = (SK_BW + S - 1) / S, r0 = split * rows_per;
      const int rows = max(0, min(rows_per, SK_BW - r0));
      for (int i = threadIdx.x; i < m_valid * rows; i += blockDim.x) {
        const int m = i / rows, wr = r0 + i % rows;
        if (n0 + wr >= p.N) continue;
        skinny_store(p, m_base + m, n0 + wr, reduce_ranks(pbase + (uint32_t)(m * SK_BW + wr) * 4u, S));
      }
    }
    if (glu) {
      // rows come in blocks of 32: [gate | up | gate | up]; 64 output columns per tile, split evenly over the ranks
      const int units_per = (64 + S - 1) / S, u0 = split * units_per;
      const int units = max(0, min(units_per, 64 - u0));
      for (int i = threadIdx.x; i < m_valid * units; i += blockDim.x) {
        const int m = i / units, u = u0 + i % units;
        const int gr = (u >> 5) * 64 + (u & 31);      // gate row inside the tile; its up row is 32 further
        if (n0 + (u >> 5) * 64 >= p.N) continue;
        float g = reduce_ranks(pbase + (uint32_t)(m * SK_BW + gr) * 4u, S);
        float up = reduce_ranks(pbase + (uint32_t)(m * SK_BW + gr + 32) * 4u, S);
        // match the unfused path: gate / up are rounded to bf16 before the activation
        g = __bfloat162float(__float2bfloat16(g));
        up = __bfloat162float(__float2bfloat16(up));
        const float a = (p.flags & SK_GLU_GELU) ? gelu_tanh_f(g) : silu_f(g);
        p.out2[(long long)(m_base + m) * p.ldo2 + (n0 >> 1) + u] = __float2bfloat16(a * up);
      }
    }
  }
  cluster_sync_all();                                 // nobody leaves while a peer may still read its shared memory

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);   // let TMA copies / MMAs in flight finish
    }
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, NT);
  }
}

static int g_sk_sms = 0;

template <int NT, int STAGES>
static int launch_skinny(const CUtensorMap& tw, const CUtensorMap& tx, const SkinnyParams& p, int n_tiles, int chunks,
                         cudaStream_t stream) {
  using L = SkinnySmem<NT, STAGES>;
  static bool configured = false;
  auto kern = gemm_skinny_kernel<NT, STAGES>;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaError_t e = launch_pdl(kern, dim3((unsigned)n_tiles, (unsigned)p.splits, (unsigned)chunks), dim3(192, 1, 1),
                             (size_t)L::TOTAL, stream, (unsigned)p.splits, tw, tx, p);
  return (int)e;
}

}  // namespace otb

using namespace otb;

// out[M,N] = X[M,K] W[N,K]^T (+ epilogue).  Returns 0, a CUDA / driver error code, or a negative argument-check code.
// `splits_override`: 0 = choose (see the rule at the selection below).
extern "C" int otb_gemm_skinny_bf16(const void* X, const void* W, void* out, int M, int N, int K, long long ldx,
                                    long long ldw, long long ldo, const void* bias, const void* residual,
                                    long long ldr, void* out2, long long ldo2, const void* gate,
                                    long long gate_stride, int rows_per_gate, int flags, int splits_override,
                                    void* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return -2;
  if ((ldx % 8) || (ldw % 8)) return -3;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W)) & 15) return -4;
  if (flags & 4) return -9;                                  // accumulate-into-output is the big GEMM's job
  if ((flags & SK_GATE) && (!(flags & SK_RESIDUAL) || gate == nullptr || rows_per_gate < 1)) return -10;
  const bool glu = (flags & (SK_GLU_GELU | SK_GLU_SILU)) != 0;
  if (glu && ((N % 64) || out2 == nullptr)) return -6;
  if (!(flags & SK_NO_OUT) && out == nullptr) return -6;
  if (g_sk_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sk_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_sk_sms <= 0) return -7;
  }
  const int nt = M <= 64 ? 64 : (M <= 128 ? 128 : 256);
  const int chunks = (M + nt - 1) / nt;
  const int n_tiles = (N + SK_BW - 1) / SK_BW;
  const int num_kb = (K + SK_BK - 1) / SK_BK;
  int splits = splits_override;
  if (splits == 0) {
    // OPENTAU_B200_SKINNY_SLOTS: CTAs the automatic choice may fill, per SM (default 2 for the <= 128-token tiles);
    // OPENTAU_B200_SKINNY_MAX_SPLITS caps the cluster size.  Tuning knobs for measurements.
    static int slots_per_sm = -1, max_splits = -1;
    if (slots_per_sm < 0) {
      const char* e = getenv("OPENTAU_B200_SKINNY_SLOTS");
      slots_per_sm = (e != nullptr && atoi(e) > 0) ? atoi(e) : 2;
      e = getenv("OPENTAU_B200_SKINNY_MAX_SPLITS");
      max_splits = (e != nullptr && atoi(e) >= 1 && atoi(e) <= 8) ? atoi(e) : 8;
    }
    // Largest cluster size whose grid is resident at once and leaves every CTA two k-blocks, with one refinement
    // measured on the action-expert chains: going beyond ONE CTA per SM only pays while each CTA still streams four
    // k-blocks; a 256-CTA launch of two-k-block CTAs fills every SM twice and keeps the next kernel of the chain
    // (programmatic dependent launch) from becoming resident early.
    const long long slots = (long long)g_sk_sms * (nt <= 128 ? slots_per_sm : 1);
    splits = 1;
    for (int s = 2; s <= max_splits; ++s) {
      const long long ctas = (long long)n_tiles * chunks * s;
      if (ctas <= slots && num_kb / s >= 2 && (ctas <= g_sk_sms || num_kb / s >= 4)) splits = s;
    }
  }
  if (splits < 1 || splits > 8) return -8;
  CUtensorMap tw, tx;
  {
    uint64_t dims[2], strides[1];
    uint32_t box[2];
    dims[0] = (uint64_t)K; dims[1] = (uint64_t)N; box[0] = 64; box[1] = SK_BW;
    strides[0] = (uint64_t)ldw * 2;
    int r = make_tmap_bf16(&tw, W, 2, dims, strides, box);
    if (r) return 1000 + r;
    dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; box[0] = 64; box[1] = (uint32_t)nt;
    strides[0] = (uint64_t)ldx * 2;
    r = make_tmap_bf16(&tx, X, 2, dims, strides, box);
    if (r) return 2000 + r;
  }
  SkinnyParams p;
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo;
  p.bias = bias;
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.out2 = static_cast<__nv_bfloat16*>(out2); p.ldo2 = ldo2;
  p.gate = static_cast<const __nv_bfloat16*>(gate); p.gate_stride = gate_stride; p.rows_per_gate = rows_per_gate;
  p.flags = flags;
  p.splits = splits;
  p.status = static_cast<KernelStatus*>(status);
  switch (nt) {
    case 64: return launch_skinny<64, 4>(tw, tx, p, n_tiles, chunks, stream);
    case 128: return launch_skinny<128, 3>(tw, tx, p, n_tiles, chunks, stream);
    default: return launch_skinny<256, 4>(tw, tx, p, n_tiles, chunks, stream);
  }
}
