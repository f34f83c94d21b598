// Prefill GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * W[N,K]^T (+ residual).
//
// Persistent, warp-specialised, one CTA per SM:
//   warp 0   : TMA producer  - 128B-swizzled [128 x 64] A tiles and [BN x 64] W tiles into a
//              STAGES-deep shared-memory ring, completion on per-stage "full" mbarriers;
//   warp 1   : MMA issuer    - one elected thread issues tcgen05.mma (cta_group::1, 128 x BN x 16)
//              straight from the swizzled tiles, accumulating in TMEM; tcgen05.commit releases
//              each stage ("empty") and, after the last k-block, publishes the accumulator;
//   warps 2-5: epilogue      - tcgen05.ld the fp32 accumulator (one TMEM lane quadrant per warp),
//              add the optional residual, convert and store; the accumulator is double-buffered
//              in TMEM so the next tile's MMAs overlap this tile's epilogue.
// bf16 (kind::f16) and int8 (kind::i8, int32 accumulate, per-row x per-column scales) share the
// pipeline.  Both operands are K-major, i.e. the checkpoint's [N, K] weight layout is used as is.
// Every CTA fetches its own tiles with plain (single-destination) TMA loads.
// Replaces the reference's linear_prefill (torch matmul / cublasGemmEx + epilogue kernel,
// backends/corex/__init__.py:1612-1701, kernels/w8a8.cu:196-366, w8a8_tcu.cu:327-776).
#include "sm100.cuh"
#include "tp.cuh"

namespace {

using namespace sm100;

constexpr int BM = 128, BK_BYTES = 128;
constexpr int kThreadsGemm = 192;

struct GemmArgs {
  void* C; int64_t ldc;            // bf16 [M, ldc]
  const bf16* residual; int64_t ldr;  // optional, added before the store
  const float* row_scale;          // int8: [M] activation scales
  const float* col_scale;          // int8: [N] weight scales
  int M, N, K;
  int m_tiles, n_tiles, k_blocks;
  int* status;                     // device status word: set to a non-zero code if a wait ran out
  // tensor-parallel prefill: instead of C, every output row goes (bf16) into this rank's own peer-visible
  // buffer, from which the rank that owns the row pulls it; the last CTA publishes the sequence number (tp.cuh)
  const TpPfDev* pf; unsigned pf_seq;
  // grouped (expert-major) mode: the m-tile list lives in device memory, written by the dispatch
  // kernel of the same step.  Tile i covers rows [g_row0[i], g_row0[i] + g_rows[i]) of A and C and
  // multiplies them by expert g_expert[i]'s [N, K] block of the weight stack.
  const int* g_count; const int* g_row0; const int* g_rows; const int* g_expert;
  // split-K for products with few rows (batched decode): `splits` CTAs share one output tile, each
  // multiplies a K slice and leaves an fp32 partial tile in `ws`; the last one to arrive (ticket)
  // adds the partials in slice order and writes the result, so the sum does not depend on timing.
  int splits; float* ws; unsigned* tickets;
};
struct TileCoord { int m0, row_end, n0, brow; };
template <int BN>
__device__ __forceinline__ TileCoord tile_coord(const GemmArgs& a, int tile, int m_tiles) {
  const int mt = tile % m_tiles, nt = tile / m_tiles;
  TileCoord c;
  c.n0 = nt * BN;
  if (a.g_count) {
    c.m0 = a.g_row0[mt];
    c.row_end = c.m0 + a.g_rows[mt];
    c.brow = a.g_expert[mt] * a.N + c.n0;
  } else {
    c.m0 = mt * BM;
    c.row_end = a.M;
    c.brow = c.n0;
  }
  return c;
}

__device__ __forceinline__ uint64_t gtime_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// wall-clock bounded wait (2 s)
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = gtime_ns();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (gtime_ns() - t0 > 2000000000ull) return false;
  }
}

template <int BN, int STAGES, bool I8>
__global__ void __launch_bounds__(kThreadsGemm, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmArgs a) {
  constexpr int A_BYTES = BM * BK_BYTES, B_BYTES = BN * BK_BYTES, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int ESIZE = I8 ? 1 : 2, BK = BK_BYTES / ESIZE, UK = 32 / ESIZE;  // elements per k-block / per MMA
  // two accumulators; an allocation is a power of two >= 32 columns
  constexpr uint32_t TMEM_COLS = 2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512);
  constexpr uint32_t IDESC = umma_idesc(BM, BN, 1, I8 ? 2 : 1);
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  __shared__ bool split_last_s;
  volatile int* abort_flag = &abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    abort_s = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  griddep_launch();
  griddep_wait();

  int m_tiles = a.m_tiles;
  if (a.g_count) { m_tiles = *a.g_count; if (m_tiles > a.m_tiles) m_tiles = a.m_tiles; }   // a.m_tiles: list capacity
  const int splits = a.splits > 1 ? a.splits : 1;
  const int kper = (a.k_blocks + splits - 1) / splits;            // k-blocks per slice
  const int total = m_tiles * a.n_tiles * splits;                  // work item = (tile, K slice), slice fastest
  if (warp == 0) {
    // ------------------------------- TMA producer -----------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < total && !*abort_flag; tile += gridDim.x) {
        const TileCoord tc = tile_coord<BN>(a, tile / splits, m_tiles);
        const int kb0 = (tile % splits) * kper, kb1 = min(a.k_blocks, kb0 + kper);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!wait_bar(&empty_bar[s], ph ^ 1, abort_flag)) { atomicExch(a.status, 1); abort_s = 1; break; }
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
          tma_load_2d(st, &tmA, &full_bar[s], kb * BK, tc.m0);
          tma_load_2d(st + A_BYTES, &tmB, &full_bar[s], kb * BK, tc.brow);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------------------
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < total && !*abort_flag; tile += gridDim.x, ++tcount) {
        const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
        if (!wait_bar(&acc_empty[acc], aph ^ 1, abort_flag)) { atomicExch(a.status, 2); abort_s = 1; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        const int kb0 = (tile % splits) * kper, kb1 = min(a.k_blocks, kb0 + kper);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!wait_bar(&full_bar[s], ph, abort_flag)) { atomicExch(a.status, 3); abort_s = 1; ok = false; break; }
          tc_fence_after();
          const unsigned char* st = tiles + (size_t)s * STAGE_BYTES;
          const uint64_t ad = umma_desc_sw128(st), bd = umma_desc_sw128(st + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            // advance 32 bytes along K inside the 128-byte swizzle atom: +2 in 16-byte units
            if (I8) umma_i8(d_tmem, ad + 2 * k, bd + 2 * k, IDESC, ((kb - kb0) | k) != 0);
            else umma_f16(d_tmem, ad + 2 * k, bd + 2 * k, IDESC, ((kb - kb0) | k) != 0);
          }
          umma_commit(&empty_bar[s]);
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
      }
    }
  } else {
    // ------------------------------- epilogue ---------------------------------------------
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < total && !*abort_flag; tile += gridDim.x, ++tcount) {
      const int otile = tile / splits, ksl = tile % splits;
      const TileCoord tc = tile_coord<BN>(a, otile, m_tiles);
      const int m0 = tc.m0, n0 = tc.n0, row_end = tc.row_end;
      const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
      if (!wait_bar(&acc_full[acc], aph, abort_flag)) { if (lane == 0) { atomicExch(a.status, 4); abort_s = 1; } break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const float rs = (I8 && row < row_end) ? a.row_scale[row] : 1.f;
      // weight scales of this tile's columns: the grouped form keeps one [N] vector per expert, back to back
      const float* cscale = I8 ? a.col_scale + (tc.brow - n0) : nullptr;
      if (splits > 1) {
        // ---- K slice: park the fp32 partial tile, the last slice to arrive reduces all of them ----
        float* mine = a.ws + ((size_t)tile * BM + q * 32 + lane) * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(tmem_base + acc * BN + ((uint32_t)(q * 32) << 16) + c0, r);
          tmem_ld_wait();
          if (row < row_end && n0 + c0 < a.N) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              float4 f;
              if (I8) f = make_float4((float)(int)r[4 * v], (float)(int)r[4 * v + 1], (float)(int)r[4 * v + 2], (float)(int)r[4 * v + 3]);
              else f = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
              __stcg(reinterpret_cast<float4*>(mine + c0) + v, f);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          const unsigned prev = atomicAdd(a.tickets + otile, 1u);
          split_last_s = prev == (unsigned)splits - 1;
          if (split_last_s) a.tickets[otile] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (split_last_s) {
          __threadfence();
          // all 128 epilogue threads walk the tile's valid rows as float4 columns (coalesced), adding
          // the slices in slice order
          const int et = (warp - 2) * 32 + lane;
          const int nrow = min(BM, row_end - m0), ncol4 = min(BN, a.N - n0) >> 2;
          const float* base = a.ws + (size_t)otile * splits * BM * BN;
#pragma unroll 2
          for (int e = et; e < nrow * ncol4; e += 128) {
            const int r = e / ncol4, c = (e % ncol4) * 4;
            float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int sidx = 0; sidx < splits; ++sidx) {
              const float4 x = __ldcg(reinterpret_cast<const float4*>(base + ((size_t)sidx * BM + r) * BN + c));
              f.x += x.x; f.y += x.y; f.z += x.z; f.w += x.w;
            }
            const int grow = m0 + r, gcol = n0 + c;
            if (I8) {
              const float rsr = a.row_scale[grow];
              f.x *= rsr * a.col_scale[gcol]; f.y *= rsr * a.col_scale[gcol + 1];
              f.z *= rsr * a.col_scale[gcol + 2]; f.w *= rsr * a.col_scale[gcol + 3];
            }
            if (a.residual) {
              const uint2 rr = *reinterpret_cast<const uint2*>(a.residual + (int64_t)grow * a.ldr + gcol);
              f.x += __uint_as_float(rr.x << 16); f.y += __uint_as_float(rr.x & 0xffff0000u);
              f.z += __uint_as_float(rr.y << 16); f.w += __uint_as_float(rr.y & 0xffff0000u);
            }
            const __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y), hi = __floats2bfloat162_rn(f.z, f.w);
            uint2 o;
            o.x = *reinterpret_cast<const uint32_t*>(&lo);
            o.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(a.C) + (int64_t)grow * a.ldc + gcol) = o;
          }
        }
        (void)ksl;
        continue;
      }
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + acc * BN + ((uint32_t)(q * 32) << 16) + c0, r);
        tmem_ld_wait();
        const int col0 = n0 + c0;
        if (row < row_end && col0 < a.N) {
          bf16* cp;
          if (a.pf) {
            const int rpr = a.pf->rows_per_rank;
            cp = a.pf->inbox[a.pf->rank] + (int64_t)row * a.pf->width + col0;      // stays at home: the owner pulls it
          } else {
            cp = reinterpret_cast<bf16*>(a.C) + (int64_t)row * a.ldc + col0;
          }
          const bf16* rp = (a.residual && !a.pf) ? a.residual + (int64_t)row * a.ldr + col0 : nullptr;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col0 + v * 8 >= a.N) break;  // N is a multiple of 8
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (I8) f[i] = (float)(int)r[v * 8 + i] * rs * cscale[col0 + v * 8 + i];
              else f[i] = __uint_as_float(r[v * 8 + i]);
            }
            if (rp) {
              float g[8];
              bf16x8_to_float(*reinterpret_cast<const uint4*>(rp + v * 8), g);
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] += g[i];
            }
            *reinterpret_cast<uint4*>(cp + v * 8) = float_to_bf16x8(f);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
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
  if (abort_s) {  // give copies still in flight time to land before the shared memory is released
    const uint64_t t0 = gtime_ns();
    while (gtime_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, int STAGES, bool I8>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmArgs a, int sms, cudaStream_t st) {
  a.n_tiles = (a.N + BN - 1) / BN;
  const size_t smem = (size_t)STAGES * (BM + BN) * BK_BYTES + 1024;
  auto kern = gemm_tc_kernel<BN, STAGES, I8>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  const int total = a.m_tiles * a.n_tiles * (a.splits > 1 ? a.splits : 1);
  const int grid = total < sms ? total : sms;
  return (int)cb_launch(kern, dim3((unsigned)grid), dim3(kThreadsGemm), smem, st, tmA, tmB, a);
}

int g_sms = 0;
int sm_count() {
  if (!g_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_sms <= 0) g_sms = 148;
  }
  return g_sms;
}

// Relative time of an [M, N] product with BN-wide tiles: waves of tiles over the SMs times the cost
// of one tile.  A tile's cost is its width times a factor measured on B200 for K = 2560..9216: a
// narrow tile re-reads the A tile from L2 for fewer flops and the loads, not the tensor pipe, set
// its pace (128 x 256 tiles ran at 1.3 PFLOP/s machine-wide, 128 x 128 at 0.79).
double tile_cost(int M, int N, int bn, int sms) {
  const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
  const int waves = (tiles + sms - 1) / sms;
  const double f = bn >= 256 ? 1.0 : (bn >= 160 ? 1.3 : (bn >= 128 ? 1.7 : 2.5));
  return (double)waves * bn * f;
}
int pick_bn(int M, int N, int sms, bool allow64) {
  const int cand[4] = {256, 160, 128, 64};
  int best = 256;
  double bc = 1e300;
  for (int i = 0; i < (allow64 ? 4 : 3); ++i) {
    const double c = tile_cost(M, N, cand[i], sms);
    if (c < bc) { bc = c; best = cand[i]; }
  }
  return best;
}

}  // namespace

// CTA-pair kernel (gemm_tc2.cu): tile width it would use for [M, N], or 0 for "not this product".
int cb_gemm_pair_plan(int64_t M, int64_t N);
int cb_gemm_pair_run(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc, const void* residual,
                     int64_t ldr, const void* row_scale, const void* col_scale, int64_t M, int64_t N, int64_t K, int tile,
                     const void* pf, int64_t pf_seq, void* status, void* stream);

// C[M,N] (bf16) = A[M,K] (bf16) x W[N,K]^T (bf16) (+ residual[M,N]).  K % 8 == 0, N % 8 == 0.
// bn_hint: 0 = choose (CTA pairs for more than 256 rows), 64/128/160/256 = one-CTA kernel with that tile
// width, 1256/1288/1320 = CTA-pair kernel with a 256 x 256 / 256 x 288 / 256 x 320 tile.
CB_EXPORT int cb_gemm_bf16(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc,
                           const void* residual, int64_t ldr, int64_t M, int64_t N, int64_t K,
                           int64_t bn_hint, const void* pf, int64_t pf_seq, void* status, void* stream) {
  if (M < 1 || N < 1 || K < 1) return CB_ERR_SHAPE;
  if (K % 8 || N % 8 || (!pf && ldc % 8) || (residual && ldr % 8) || !status) return CB_ERR_SHAPE;
  const int sms = sm_count();
  int bn = (int)bn_hint;
  if (bn == 0 || bn >= 1000) {
    const int tile = bn >= 1000 ? bn - 1000 : cb_gemm_pair_plan(M, N);
    if (tile) return cb_gemm_pair_run(A, lda, W, ldw, C, ldc, residual, ldr, nullptr, nullptr, M, N, K, tile, pf, pf_seq, status, stream);
  }
  if (!bn) bn = pick_bn((int)M, (int)N, sms, true);
  CUtensorMap tmA, tmB;
  int rc = cb_make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, 64);
  if (rc) return rc;
  rc = cb_make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, (uint32_t)bn, 64);
  if (rc) return rc;
  GemmArgs a;
  a.C = C; a.ldc = ldc; a.residual = (const bf16*)residual; a.ldr = ldr; a.row_scale = nullptr; a.col_scale = nullptr;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.m_tiles = (int)((M + BM - 1) / BM); a.n_tiles = 0;
  a.k_blocks = (int)((K + 63) / 64); a.status = (int*)status;
  a.pf = (const TpPfDev*)pf; a.pf_seq = (unsigned)pf_seq;
  a.g_count = a.g_row0 = a.g_rows = a.g_expert = nullptr;
  a.splits = 1; a.ws = nullptr; a.tickets = nullptr;
  cudaStream_t st = (cudaStream_t)stream;
  if (bn == 256) return launch_gemm<256, 4, false>(tmA, tmB, a, sms, st);
  if (bn == 160) return launch_gemm<160, 5, false>(tmA, tmB, a, sms, st);
  if (bn == 128) return launch_gemm<128, 6, false>(tmA, tmB, a, sms, st);
  if (bn == 64) return launch_gemm<64, 8, false>(tmA, tmB, a, sms, st);
  return CB_ERR_ARG;
}

// C[M,N] (bf16) = (A_q[M,K] int8 x W_q[N,K]^T int8) * row_scale[m] * col_scale[n] (+ residual). K % 16 == 0.
CB_EXPORT int cb_gemm_i8(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc,
                         const void* residual, int64_t ldr, const void* row_scale, const void* col_scale,
                         int64_t M, int64_t N, int64_t K, int64_t bn_hint, const void* pf, int64_t pf_seq,
                         void* status, void* stream) {
  if (M < 1 || N < 1 || K < 1) return CB_ERR_SHAPE;
  if (K % 16 || N % 8 || (!pf && ldc % 8) || lda % 16 || ldw % 16 || (residual && ldr % 8) || !status || !row_scale || !col_scale)
    return CB_ERR_SHAPE;
  const int sms = sm_count();
  int bn = (int)bn_hint;
  if (bn == 0 || bn >= 1000) {
    const int tile = bn >= 1000 ? bn - 1000 : cb_gemm_pair_plan(M, N);
    if (tile)
      return cb_gemm_pair_run(A, lda, W, ldw, C, ldc, residual, ldr, row_scale, col_scale, M, N, K, tile, pf, pf_seq, status, stream);
  }
  if (!bn) bn = pick_bn((int)M, (int)N, sms, false);
  CUtensorMap tmA, tmB;
  int rc = cb_make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, 128);
  if (rc) return rc;
  rc = cb_make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, (uint32_t)bn, 128);
  if (rc) return rc;
  GemmArgs a;
  a.C = C; a.ldc = ldc; a.residual = (const bf16*)residual; a.ldr = ldr;
  a.row_scale = (const float*)row_scale; a.col_scale = (const float*)col_scale;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.m_tiles = (int)((M + BM - 1) / BM); a.n_tiles = 0;
  a.k_blocks = (int)((K + 127) / 128); a.status = (int*)status;
  a.pf = (const TpPfDev*)pf; a.pf_seq = (unsigned)pf_seq;
  a.g_count = a.g_row0 = a.g_rows = a.g_expert = nullptr;
  a.splits = 1; a.ws = nullptr; a.tickets = nullptr;
  cudaStream_t st = (cudaStream_t)stream;
  if (bn == 256) return launch_gemm<256, 4, true>(tmA, tmB, a, sms, st);
  if (bn == 160) return launch_gemm<160, 5, true>(tmA, tmB, a, sms, st);
  if (bn == 128) return launch_gemm<128, 6, true>(tmA, tmB, a, sms, st);
  return CB_ERR_ARG;
}

// Grouped (expert-major) product for routed-MoE prefill: rows of A sorted by expert, W a stack
// [E, N, K]; C[r, :] = A[r, :] x W[expert(r)]^T for the rows the tile list covers.  The list
// (g_count m-tiles of at most 128 rows, never crossing an expert boundary) is produced on the device
// by cb_moe_dispatch, so no count travels to the host; max_tiles bounds it and sizes the grid.
// Replaces the reference's expert-major grouped GEMMs (kernels/w8a8_tcu.cu:962, moe_grouped_i8.cu:1283).
CB_EXPORT int cb_gemm_bf16_grouped(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc,
                                   int64_t rows, int64_t E, int64_t N, int64_t K, const void* g_count,
                                   const void* g_row0, const void* g_rows, const void* g_expert, int64_t max_tiles,
                                   void* status, void* stream) {
  if (rows < 1 || N < 1 || K < 1 || E < 1 || max_tiles < 1) return CB_ERR_SHAPE;
  if (K % 8 || N % 8 || ldc % 8 || !status || !g_count || !g_row0 || !g_rows || !g_expert) return CB_ERR_SHAPE;
  const int sms = sm_count();
  const int bn = N % 256 == 0 || N > 1024 ? 256 : (N % 160 == 0 ? 160 : 128);
  CUtensorMap tmA, tmB;
  int rc = cb_make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, (uint64_t)rows, (uint64_t)K, (uint64_t)lda, BM, 64);
  if (rc) return rc;
  rc = cb_make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, (uint64_t)(E * N), (uint64_t)K, (uint64_t)ldw, (uint32_t)bn, 64);
  if (rc) return rc;
  GemmArgs a;
  a.C = C; a.ldc = ldc; a.residual = nullptr; a.ldr = 0; a.row_scale = nullptr; a.col_scale = nullptr;
  a.M = (int)rows; a.N = (int)N; a.K = (int)K; a.m_tiles = (int)max_tiles; a.n_tiles = 0;
  a.k_blocks = (int)((K + 63) / 64); a.status = (int*)status;
  a.pf = nullptr; a.pf_seq = 0;
  a.g_count = (const int*)g_count; a.g_row0 = (const int*)g_row0; a.g_rows = (const int*)g_rows; a.g_expert = (const int*)g_expert;
  a.splits = 1; a.ws = nullptr; a.tickets = nullptr;
  cudaStream_t st = (cudaStream_t)stream;
  if (bn == 256) return launch_gemm<256, 4, false>(tmA, tmB, a, sms, st);
  if (bn == 160) return launch_gemm<160, 5, false>(tmA, tmB, a, sms, st);
  return launch_gemm<128, 6, false>(tmA, tmB, a, sms, st);
}

// The same grouped product from int8 stacks (W8A8 routed experts): A int8 [rows, K] with one scale per row
// (the gathered activation rows, quantised per token), W int8 [E, N, K] with col_scale [E, N];
// C = (A x W[expert]^T) * row_scale * col_scale[expert] on the kind::i8 path.  K % 16 == 0.
CB_EXPORT int cb_gemm_i8_grouped(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc,
                                 const void* row_scale, const void* col_scale, int64_t rows, int64_t E, int64_t N,
                                 int64_t K, const void* g_count, const void* g_row0, const void* g_rows,
                                 const void* g_expert, int64_t max_tiles, void* status, void* stream) {
  if (rows < 1 || N < 1 || K < 1 || E < 1 || max_tiles < 1) return CB_ERR_SHAPE;
  if (K % 16 || N % 8 || ldc % 8 || lda % 16 || ldw % 16) return CB_ERR_SHAPE;
  if (!status || !row_scale || !col_scale || !g_count || !g_row0 || !g_rows || !g_expert) return CB_ERR_ARG;
  const int sms = sm_count();
  const int bn = N % 256 == 0 || N > 1024 ? 256 : (N % 160 == 0 ? 160 : 128);
  CUtensorMap tmA, tmB;
  int rc = cb_make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, (uint64_t)rows, (uint64_t)K, (uint64_t)lda, BM, 128);
  if (rc) return rc;
  rc = cb_make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, (uint64_t)(E * N), (uint64_t)K, (uint64_t)ldw, (uint32_t)bn, 128);
  if (rc) return rc;
  GemmArgs a;
  a.C = C; a.ldc = ldc; a.residual = nullptr; a.ldr = 0;
  a.row_scale = (const float*)row_scale; a.col_scale = (const float*)col_scale;
  a.M = (int)rows; a.N = (int)N; a.K = (int)K; a.m_tiles = (int)max_tiles; a.n_tiles = 0;
  a.k_blocks = (int)((K + 127) / 128); a.status = (int*)status;
  a.pf = nullptr; a.pf_seq = 0;
  a.g_count = (const int*)g_count; a.g_row0 = (const int*)g_row0; a.g_rows = (const int*)g_rows; a.g_expert = (const int*)g_expert;
  a.splits = 1; a.ws = nullptr; a.tickets = nullptr;
  cudaStream_t st = (cudaStream_t)stream;
  if (bn == 256) return launch_gemm<256, 4, true>(tmA, tmB, a, sms, st);
  if (bn == 160) return launch_gemm<160, 5, true>(tmA, tmB, a, sms, st);
  return launch_gemm<128, 6, true>(tmA, tmB, a, sms, st);
}

// Skinny product for batched decode (M <= 128 rows: one m-tile): C = A x W^T (+ residual) with the K
// dimension split over CTAs so that the whole machine streams the weights even when N gives only a
// few 256-wide tiles (N = 2560: 10 tiles x 14 slices).  ws holds the fp32 partial tiles
// (cb_gemm_splitk_ws_bytes), tickets one zero-initialised counter per output tile; both may be
// shared by all calls of a stream.  Falls back to the plain kernel when splitting does not pay.
namespace {
// Tile width and slice count for a product of at most 128 rows.  Every (tile, slice) gets its own CTA
// in a single wave; the estimate is the bytes one CTA moves into shared memory (its slice of W and of
// the valid rows of A) plus what the last slice re-reads to add the partial tiles.
// K is counted in bytes of a row (a k-block is 128 bytes); n_cand = 2 leaves out the 64-wide tile.
void plan_split(int64_t M, int64_t N, int64_t Kbytes, int* bn_out, int* s_out, int n_cand = 3) {
  const int sms = sm_count();
  const int64_t kb = (Kbytes + 127) / 128, K = Kbytes / 2;
  const int cand[3] = {256, 128, 64};
  double best = 1e300;
  *bn_out = 256; *s_out = 1;
  for (int i = 0; i < n_cand; ++i) {
    const int bn = cand[i];
    const int64_t tiles = (N + bn - 1) / bn;
    int64_t s = sms / tiles;
    if (s > kb / 4) s = kb / 4;          // at least four k-blocks per slice
    if (s > 32) s = 32;
    if (s < 1) s = 1;
    for (;;) {                           // no slice may be empty: s = ceil(kb / ceil(kb / s))
      const int64_t kper = (kb + s - 1) / s, s2 = (kb + kper - 1) / kper;
      if (s2 == s) break;
      s = s2;
    }
    const int64_t waves = (tiles * s + sms - 1) / sms;
    const double stream = (double)waves * (bn + M) * ((double)K / s) * 2.0 / 130e3;        // us at ~130 GB/s per SM
    const double reduce = s > 1 ? (double)s * M * bn * 4.0 / 100e3 + 2.0 : 0.0;
    const double cost = stream + reduce;
    if (cost < best) { best = cost; *bn_out = bn; *s_out = (int)s; }
  }
}
}  // namespace

// (slices, or 1 when the plain kernel is used) and the workspace a call needs
CB_EXPORT int64_t cb_gemm_splitk_plan(int64_t M, int64_t N, int64_t K) {
  if (M > BM) return 1;
  int bn, s;
  plan_split(M, N, K * 2, &bn, &s);
  return s;
}
CB_EXPORT int64_t cb_gemm_splitk_ws_bytes(int64_t M, int64_t N, int64_t K) {
  if (M > BM) return 0;
  int bn, s;
  plan_split(M, N, K * 2, &bn, &s);
  return s < 2 ? 0 : ((N + bn - 1) / bn) * s * BM * bn * (int64_t)sizeof(float);
}
CB_EXPORT int cb_gemm_bf16_splitk(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc,
                                  const void* residual, int64_t ldr, int64_t M, int64_t N, int64_t K, void* ws,
                                  int64_t ws_bytes, void* tickets, int64_t n_tickets, void* status, void* stream) {
  if (M < 1 || M > BM || N < 1 || K < 1) return CB_ERR_SHAPE;
  if (K % 8 || N % 8 || ldc % 8 || (residual && ldr % 8) || !status) return CB_ERR_SHAPE;
  int bn, splits;
  plan_split(M, N, K * 2, &bn, &splits);
  if (splits < 2) return cb_gemm_bf16(A, lda, W, ldw, C, ldc, residual, ldr, M, N, K, bn, nullptr, 0, status, stream);
  const int64_t tiles = (N + bn - 1) / bn;
  if (!ws || !tickets || ws_bytes < cb_gemm_splitk_ws_bytes(M, N, K) || n_tickets < tiles) return CB_ERR_ARG;
  const int sms = sm_count();
  CUtensorMap tmA, tmB;
  int rc = cb_make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, 64);
  if (rc) return rc;
  rc = cb_make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, (uint32_t)bn, 64);
  if (rc) return rc;
  GemmArgs a;
  a.C = C; a.ldc = ldc; a.residual = (const bf16*)residual; a.ldr = ldr; a.row_scale = nullptr; a.col_scale = nullptr;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.m_tiles = 1; a.n_tiles = 0;
  a.k_blocks = (int)((K + 63) / 64); a.status = (int*)status;
  a.pf = nullptr; a.pf_seq = 0;
  a.g_count = a.g_row0 = a.g_rows = a.g_expert = nullptr;
  a.splits = splits; a.ws = (float*)ws; a.tickets = (unsigned*)tickets;
  cudaStream_t st = (cudaStream_t)stream;
  if (bn == 256) return launch_gemm<256, 4, false>(tmA, tmB, a, sms, st);
  if (bn == 128) return launch_gemm<128, 6, false>(tmA, tmB, a, sms, st);
  return launch_gemm<64, 8, false>(tmA, tmB, a, sms, st);
}

// int8 (W8A8) form of the split-K product: int32 partial sums are parked as fp32 (exact up to 2^24 per
// slice, then rounded like any fp32 sum) and the row x column scales are applied by the reducing slice.
CB_EXPORT int cb_gemm_i8_splitk(const void* A, int64_t lda, const void* W, int64_t ldw, void* C, int64_t ldc,
                                const void* residual, int64_t ldr, const void* row_scale, const void* col_scale,
                                int64_t M, int64_t N, int64_t K, void* ws, int64_t ws_bytes, void* tickets,
                                int64_t n_tickets, void* status, void* stream) {
  if (M < 1 || M > BM || N < 1 || K < 1) return CB_ERR_SHAPE;
  if (K % 16 || N % 8 || ldc % 8 || lda % 16 || ldw % 16 || (residual && ldr % 8) || !status || !row_scale || !col_scale)
    return CB_ERR_SHAPE;
  int bn, splits;
  plan_split(M, N, K, &bn, &splits, 2);
  if (splits < 2)
    return cb_gemm_i8(A, lda, W, ldw, C, ldc, residual, ldr, row_scale, col_scale, M, N, K, bn, nullptr, 0, status, stream);
  const int64_t tiles = (N + bn - 1) / bn;
  if (!ws || !tickets || ws_bytes < tiles * splits * BM * bn * (int64_t)sizeof(float) || n_tickets < tiles) return CB_ERR_ARG;
  const int sms = sm_count();
  CUtensorMap tmA, tmB;
  int rc = cb_make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, 128);
  if (rc) return rc;
  rc = cb_make_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, (uint32_t)bn, 128);
  if (rc) return rc;
  GemmArgs a;
  a.C = C; a.ldc = ldc; a.residual = (const bf16*)residual; a.ldr = ldr;
  a.row_scale = (const float*)row_scale; a.col_scale = (const float*)col_scale;
  a.M = (int)M; a.N = (int)N; a.K = (int)K; a.m_tiles = 1; a.n_tiles = 0;
  a.k_blocks = (int)((K + 127) / 128); a.status = (int*)status;
  a.pf = nullptr; a.pf_seq = 0;
  a.g_count = a.g_row0 = a.g_rows = a.g_expert = nullptr;
  a.splits = splits; a.ws = (float*)ws; a.tickets = (unsigned*)tickets;
  cudaStream_t st = (cudaStream_t)stream;
  if (bn == 256) return launch_gemm<256, 4, true>(tmA, tmB, a, sms, st);
  return launch_gemm<128, 6, true>(tmA, tmB, a, sms, st);
}
