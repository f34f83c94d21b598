// Prefill GEMM on CTA pairs: C[M,N] = A[M,K] * W[N,K]^T (+ residual), bf16 or int8 (W8A8), 256-row tiles.
//
// Two CTAs of a cluster (two SMs) work on one 256 x TILE_N output tile with tcgen05.mma
// cta_group::2: each CTA stages only its own 128 rows of A and HALF of the tile's weight rows, the
// even CTA issues the MMAs and the tensor cores of both SMs read both halves.  Per k-block a CTA
// therefore moves 16 KB + TILE_N/2 x 128 B into shared memory for 128 x TILE_N x 64 multiply-adds -
// half the weight traffic of the one-CTA kernel, whose narrow tiles were paced by the L2 -> shared
// memory loads, not by the tensor pipe.  TILE_N is one MMA of N = 256 or two MMAs of N = 144 / 160 that share
// the A tile (256 x 288 tiles cut a 2048 x 2560 product into 72 tiles for the 74 SM pairs: one round).
//
// Roles per CTA (192 threads): warp 0 TMA producer (plain single-destination loads into its own
// shared memory; the completion bytes of both CTAs are counted on the even CTA's barrier), warp 1
// MMA issuer (even CTA only) and tensor-memory owner, warps 2-5 epilogue (tcgen05.ld of the CTA's own
// 128 accumulator rows).  tcgen05.commit signals the "stage free" and "accumulator ready" barriers of
// both CTAs; the epilogue warps of both CTAs arrive on the even CTA's "accumulator free" barrier.
// Every wait is bounded (2 s) and reports through the status word; an abort is forwarded to the
// other CTA of the pair so that both unwind, meet at the cluster barrier and free tensor memory.
// Replaces the reference's linear_prefill (backends/corex/__init__.py:1612-1701).
#include "sm100.cuh"
#include "tp.cuh"

namespace {

using namespace sm100;

constexpr int kThreadsPair = 192;
constexpr int PM = 128;            // rows of A per CTA (256 per pair)

struct PairArgs {
  bf16* C; int64_t ldc;
  const bf16* residual; int64_t ldr;
  const float* row_scale;          // int8: [M] activation scales
  const float* col_scale;          // int8: [N] weight scales
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;  // m_tiles counts 256-row tiles
  int* status;
  const TpPfDev* pf; unsigned pf_seq;   // tensor-parallel prefill: rows go to this rank's peer-visible buffer (tp.cuh)
  int up_off;                      // SwiGLU form: W is [gate rows | up rows], the up rows start here; N counts outputs
};

__device__ __forceinline__ uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool wait_bar2(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = now_ns();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (now_ns() - t0 > 2000000000ull) return false;
  }
}

// SWIGLU (one MMA of N = 256, bf16): the even CTA stages 128 gate rows of W, the odd CTA the 128 up rows
// of the same output columns, so accumulator columns [0, 128) hold the gate and [128, 256) the up
// projection of one 128-column output tile; the epilogue writes silu(gate) * up and the [M, 2I]
// intermediate never reaches memory.
template <int BNI, int NI, int STAGES, bool I8, bool SWIGLU = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsPair, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const PairArgs a) {
  constexpr int TILE_N = BNI * NI;
  constexpr int BH = BNI / 2;                       // weight rows of one MMA held by this CTA
  constexpr int A_BYTES = PM * 128, BJ_BYTES = BH * 128, STAGE_BYTES = A_BYTES + NI * BJ_BYTES;
  constexpr int ACC_BUFS = 2 * TILE_N <= 512 ? 2 : 1;
  constexpr uint32_t TMEM_COLS = ACC_BUFS * TILE_N <= 256 ? 256 : 512;
  constexpr uint32_t IDESC = umma_idesc(256, BNI, 1, I8 ? 2 : 1);
  constexpr int BK = I8 ? 128 : 64;                 // elements per 128-byte k-block
  constexpr int OUT_N = SWIGLU ? TILE_N / 2 : TILE_N;   // output columns of a tile
  static_assert(BNI % 16 == 0 && BNI <= 256 && BH % 8 == 0 && TILE_N % 32 == 0, "tile shape");
  static_assert(!SWIGLU || NI == 1, "the SwiGLU form is one MMA per k-step");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 8); }
    abort_s = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(&tmem_base_s, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // both CTAs' barriers exist before either signals the other
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t peer_abort = map_to_cta(smem_u32(&abort_s), rank ^ 1);
  griddep_launch();
  griddep_wait();

  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int total = a.m_tiles * a.n_tiles;
  if (warp == 0) {
    // ------------------------------- TMA producer (both CTAs) -------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = pair; tile < total && !*abort_flag; tile += npairs) {
        const int m0 = (tile % a.m_tiles) * 256 + (int)rank * PM, n0 = (tile / a.m_tiles) * OUT_N;
        const int brow = SWIGLU ? n0 + (int)rank * a.up_off : n0 + (int)rank * BH;
        for (int kb = 0; kb < a.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!wait_bar2(&empty_bar[s], ph ^ 1, abort_flag)) {
            atomicExch(a.status, 81); abort_s = 1; st_cluster_u32(peer_abort, 1); break;
          }
          if (leader) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
          const uint32_t fb = map_to_cta(smem_u32(&full_bar[s]), 0);
          unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
          tma_load_2d_pair(st, &tmA, fb, kb * BK, m0);
#pragma unroll
          for (int j = 0; j < NI; ++j)
            tma_load_2d_pair(st + A_BYTES + j * BJ_BYTES, &tmB, fb, kb * BK, brow + j * BNI);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (even CTA) ----------------------------------
    if (lane == 0 && leader) {
      uint32_t it = 0, tcount = 0;
      for (int tile = pair; tile < total && !*abort_flag; tile += npairs, ++tcount) {
        const uint32_t acc = tcount % ACC_BUFS, aph = (tcount / ACC_BUFS) & 1;
        if (!wait_bar2(&acc_empty[acc], aph ^ 1, abort_flag)) {
          atomicExch(a.status, 82); abort_s = 1; st_cluster_u32(peer_abort, 1); break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TILE_N;
        bool ok = true;
        for (int kb = 0; kb < a.k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!wait_bar2(&full_bar[s], ph, abort_flag)) {
            atomicExch(a.status, 83); abort_s = 1; st_cluster_u32(peer_abort, 1); ok = false; break;
          }
          tc_fence_after();
          const unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
          const uint64_t ad = umma_desc_sw128(st);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
#pragma unroll
            for (int j = 0; j < NI; ++j) {
              const uint64_t bd = umma_desc_sw128(st + A_BYTES + j * BJ_BYTES);
              if (I8) umma_i8_pair(d_tmem + j * BNI, ad + 2 * k, bd + 2 * k, IDESC, (kb | k) != 0);
              else umma_f16_pair(d_tmem + j * BNI, ad + 2 * k, bd + 2 * k, IDESC, (kb | k) != 0);
            }
          }
          umma_commit_pair(&empty_bar[s], 3);
        }
        if (!ok) break;
        umma_commit_pair(&acc_full[acc], 3);
      }
    }
  } else {
    // ------------------------------- epilogue (both CTAs) -----------------------------------
    const int q = warp & 3;
    uint32_t tcount = 0;
    const uint32_t ae0 = map_to_cta(smem_u32(&acc_empty[0]), 0), ae1 = map_to_cta(smem_u32(&acc_empty[1]), 0);
    for (int tile = pair; tile < total && !*abort_flag; tile += npairs, ++tcount) {
      const int m0 = (tile % a.m_tiles) * 256 + (int)rank * PM, n0 = (tile / a.m_tiles) * OUT_N;
      const uint32_t acc = tcount % ACC_BUFS, aph = (tcount / ACC_BUFS) & 1;
      const int row = m0 + q * 32 + lane;
      const bool rowok = row < a.M;
      // The residual rows are requested while the tile is still being multiplied, RPF column chunks ahead of
      // the accumulator reads: the latency of their 64-byte pieces would otherwise sit between two
      // tcgen05.ld of a tile whose epilogue nothing hides (one round of 256 x 288 tiles).
      constexpr int NCH = TILE_N / 32, RPF = 4;
      const bf16* rbase = (!SWIGLU && a.residual && !a.pf && rowok) ? a.residual + (int64_t)row * a.ldr + n0 : nullptr;
      uint4 rbuf[RPF][4];
      auto fetch = [&](int ci, uint4* dst) {
        if (rbase) {
#pragma unroll
          for (int v = 0; v < 4; ++v)
            if (n0 + ci * 32 + v * 8 < a.N) dst[v] = *reinterpret_cast<const uint4*>(rbase + ci * 32 + v * 8);
        }
      };
#pragma unroll
      for (int ci = 0; ci < RPF && ci < NCH; ++ci) fetch(ci, rbuf[ci]);
      if (!wait_bar2(&acc_full[acc], aph, abort_flag)) {
        if (lane == 0) { atomicExch(a.status, 84); abort_s = 1; st_cluster_u32(peer_abort, 1); }
        break;
      }
      tc_fence_after();
      const float rs = (I8 && rowok) ? a.row_scale[row] : 1.f;
      if (SWIGLU) {
#pragma unroll 1
        for (int c0 = 0; c0 < OUT_N; c0 += 32) {
          uint32_t rg[32], ru[32];
          const uint32_t ta = tmem_base + acc * TILE_N + ((uint32_t)(q * 32) << 16) + c0;
          tmem_ld32(ta, rg);
          tmem_ld32(ta + OUT_N, ru);
          tmem_ld_wait();
          const int col0 = n0 + c0;
          if (row < a.M && col0 < a.N) {
            bf16* cp = a.C + (int64_t)row * a.ldc + col0;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 >= a.N) break;  // N is a multiple of 8
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                if (I8) {
                  const int cc = col0 + v * 8 + i;
                  f[i] = silu_f((float)(int)rg[v * 8 + i] * rs * a.col_scale[cc]) *
                         ((float)(int)ru[v * 8 + i] * rs * a.col_scale[a.up_off + cc]);
                } else {
                  f[i] = silu_f(__uint_as_float(rg[v * 8 + i])) * __uint_as_float(ru[v * 8 + i]);
                }
              }
              *reinterpret_cast<uint4*>(cp + v * 8) = float_to_bf16x8(f);
            }
          }
        }
      } else {
#pragma unroll
        for (int ci = 0; ci < NCH; ++ci) {
          const int c0 = ci * 32;
          uint32_t r[32];
          tmem_ld32(tmem_base + acc * TILE_N + ((uint32_t)(q * 32) << 16) + c0, r);
          tmem_ld_wait();
          const int col0 = n0 + c0;
          if (rowok && col0 < a.N) {
            bf16* cp;
            if (a.pf) {
              const int rpr = a.pf->rows_per_rank;
              cp = a.pf->inbox[a.pf->rank] + (int64_t)row * a.pf->width + col0;      // stays at home: the owner pulls it
            } else {
              cp = a.C + (int64_t)row * a.ldc + col0;
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 >= a.N) break;  // N is a multiple of 8
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                if (I8) f[i] = (float)(int)r[v * 8 + i] * rs * a.col_scale[col0 + v * 8 + i];
                else f[i] = __uint_as_float(r[v * 8 + i]);
              }
              if (rbase) {
                float g[8];
                bf16x8_to_float(rbuf[ci % RPF][v], g);
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] += g[i];
              }
              *reinterpret_cast<uint4*>(cp + v * 8) = float_to_bf16x8(f);
            }
          }
          if (ci + RPF < NCH) fetch(ci + RPF, rbuf[ci % RPF]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? ae1 : ae0);
    }
    if (a.pf) {
      __threadfence_system();
      asm volatile("bar.sync 1, 128;" ::: "memory");      // the four epilogue warps
      if (warp == 2 && lane == 0) tp_pf_publish(a.pf, 1, a.pf_seq, gridDim.x);
    }
  }
  // ------------------------------- teardown ---------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (abort_s) {  // give copies and MMAs still in flight time to land before anything is released
    const uint64_t t0 = now_ns();
    while (now_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  cluster_sync_all();   // the other CTA's tensor cores read this CTA's shared memory until its last MMA
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

int g_pair_sms = 0;
int pair_sm_count() {
  if (!g_pair_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_pair_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_pair_sms <= 0) g_pair_sms = 148;
  }
  return g_pair_sms;
}

template <int BNI, int NI, int STAGES, bool I8, bool SWIGLU = false>
int launch_pair(const void* A, int64_t lda, const void* W, int64_t ldw, PairArgs a, cudaStream_t st) {
  constexpr int TILE_N = BNI * NI;
  const CUtensorMapDataType dt = I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  constexpr int ES = I8 ? 1 : 2;
  CUtensorMap tmA, tmB;
  int rc = cb_make_tmap_2d(&tmA, dt, ES, A, (uint64_t)a.M, (uint64_t)a.K, (uint64_t)lda, PM, 128 / ES);
  if (rc) return rc;
  const uint64_t w_rows = SWIGLU ? (uint64_t)a.up_off + (uint64_t)a.N : (uint64_t)a.N;
  rc = cb_make_tmap_2d(&tmB, dt, ES, W, w_rows, (uint64_t)a.K, (uint64_t)ldw, BNI / 2, 128 / ES);
  if (rc) return rc;
  a.k_blocks = (a.K * ES + 127) / 128;
  constexpr int OUT_N = SWIGLU ? TILE_N / 2 : TILE_N;
  a.n_tiles = (a.N + OUT_N - 1) / OUT_N;
  const size_t smem = (size_t)STAGES * (PM * 128 + NI * (BNI / 2) * 128) + 1024;
  auto kern = gemm_tc_pair_kernel<BNI, NI, STAGES, I8, SWIGLU>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int total = a.m_tiles * a.n_tiles, pairs = pair_sm_count() / 2;
  const int grid = 2 * (total < pairs ? total : pairs);
  return (int)cb_launch(kern, dim3((unsigned)grid), dim3(kThreadsPair), smem, st, tmA, tmB, a);
}

int g_pair_enabled = 1;

}  // namespace

// Width of the pair kernel's tile for an [M, N] product, or 0 when the one-CTA kernel should run:
// the width with the fewest rounds x width over the SM pairs.
int cb_gemm_pair_plan(int64_t M, int64_t N) {
  if (!g_pair_enabled || M <= 256 || N < 256) return 0;
  const int pairs = pair_sm_count() / 2;
  const int64_t mt = (M + 255) / 256;
  const int cand[3] = {256, 288, 320};
  int best = 0;
  int64_t bc = INT64_MAX;
  for (int i = 0; i < 3; ++i) {
    const int64_t tiles = mt * ((N + cand[i] - 1) / cand[i]);
    const int64_t rounds = (tiles + pairs - 1) / pairs;
    // tiles wider than 256 columns have one accumulator: from the second round on their epilogue is not
    // hidden behind the next tile's products (measured: +25 % on a six-round product)
    const int64_t cost = rounds * cand[i] * (cand[i] > 256 && rounds > 1 ? 5 : 4);
    if (cost < bc) { bc = cost; best = cand[i]; }
  }
  return best;
}

// tile: 256, 288 or 320 (0 = choose).  row_scale / col_scale given: int8 operands (contract of cb_gemm_i8), else
// bf16 (contract of cb_gemm_bf16).
int cb_gemm_pair_run(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc, const void* residual,
                     int64_t ldr, const void* row_scale, const void* col_scale, int64_t M, int64_t N, int64_t K, int tile,
                     const void* pf, int64_t pf_seq, void* status, void* stream) {
  PairArgs a;
  a.C = (bf16*)C; a.ldc = ldc; a.residual = (const bf16*)residual; a.ldr = ldr;
  a.row_scale = (const float*)row_scale; a.col_scale = (const float*)col_scale;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.m_tiles = (int)((M + 255) / 256); a.n_tiles = 0;
  a.k_blocks = (int)((K + 63) / 64); a.status = (int*)status;
  a.pf = (const TpPfDev*)pf; a.pf_seq = (unsigned)pf_seq; a.up_off = 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (!tile) tile = cb_gemm_pair_plan(M, N);
  if (row_scale) {
    if (tile == 256) return launch_pair<256, 1, 6, true>(A, lda, W, ldw, a, st);
    if (tile == 288) return launch_pair<144, 2, 6, true>(A, lda, W, ldw, a, st);
    if (tile == 320) return launch_pair<160, 2, 6, true>(A, lda, W, ldw, a, st);
    return CB_ERR_ARG;
  }
  if (tile == 256) return launch_pair<256, 1, 6, false>(A, lda, W, ldw, a, st);
  if (tile == 288) return launch_pair<144, 2, 6, false>(A, lda, W, ldw, a, st);
  if (tile == 320) return launch_pair<160, 2, 6, false>(A, lda, W, ldw, a, st);
  return CB_ERR_ARG;
}

// C[M, I] = silu(A W[0:I]^T) * (A W[up_off:up_off+I]^T), bf16: the gate|up projection with its SwiGLU product
// in the epilogue.  More than 256 rows (smaller products: cb_gemm_bf16 + cb_swiglu).  K % 8 == 0, I % 8 == 0.
CB_EXPORT int cb_gemm_bf16_swiglu(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc,
                                  int64_t M, int64_t I, int64_t up_off, int64_t K, void* status, void* stream) {
  if (M < 1 || I < 1 || K < 1 || up_off < I) return CB_ERR_SHAPE;
  if (K % 8 || I % 8 || ldc % 8 || !status) return CB_ERR_SHAPE;
  PairArgs a;
  a.C = (bf16*)C; a.ldc = ldc; a.residual = nullptr; a.ldr = 0; a.row_scale = nullptr; a.col_scale = nullptr;
  a.M = (int)M; a.N = (int)I; a.K = (int)K; a.m_tiles = (int)((M + 255) / 256); a.n_tiles = 0;
  a.k_blocks = 0; a.status = (int*)status; a.pf = nullptr; a.pf_seq = 0; a.up_off = (int)up_off;
  return launch_pair<256, 1, 6, false, true>(A, lda, W, ldw, a, (cudaStream_t)stream);
}

// int8 form: A_q [M, K] int8 with row scales, W_q [up_off + I, K] int8 with column scales (gate rows, then up rows).
CB_EXPORT int cb_gemm_i8_swiglu(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc,
                                const void* row_scale, const void* col_scale, int64_t M, int64_t I, int64_t up_off,
                                int64_t K, void* status, void* stream) {
  if (M < 1 || I < 1 || K < 1 || up_off < I || !row_scale || !col_scale) return CB_ERR_SHAPE;
  if (K % 16 || I % 8 || ldc % 8 || lda % 16 || ldw % 16 || !status) return CB_ERR_SHAPE;
  PairArgs a;
  a.C = (bf16*)C; a.ldc = ldc; a.residual = nullptr; a.ldr = 0;
  a.row_scale = (const float*)row_scale; a.col_scale = (const float*)col_scale;
  a.M = (int)M; a.N = (int)I; a.K = (int)K; a.m_tiles = (int)((M + 255) / 256); a.n_tiles = 0;
  a.k_blocks = 0; a.status = (int*)status; a.pf = nullptr; a.pf_seq = 0; a.up_off = (int)up_off;
  return launch_pair<256, 1, 6, true, true>(A, lda, W, ldw, a, (cudaStream_t)stream);
}

// 0: every bf16 product runs on the one-CTA kernel.
CB_EXPORT int cb_set_gemm_pair(int64_t on) { g_pair_enabled = on ? 1 : 0; return 0; }
