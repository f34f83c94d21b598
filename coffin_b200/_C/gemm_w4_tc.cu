// Grouped (expert-major) prefill GEMM straight from int4 weight codes on the tensor cores:
//   C[r, :] = A[r, :] x dequant(Wq[expert(r)])^T     (optionally silu(gate) * up in the epilogue)
// A bf16 [rows, K] sorted by expert; Wq [E, N, K/2] uint8 (two codes per byte, low nibble = even k),
// scales [E, N, K/128] fp32: the layout the decode kernels stream, so a W4A8 checkpoint keeps ONE copy
// of its expert stacks.  A routed-MoE prefill reads every expert's weights for ~64 rows each: with a
// bf16 expansion of the stacks that is HBM-bound on 4x the bytes (and the expansion costs 4x the
// memory); here the codes travel (TMA, 8 KB per k-block and tile) and are expanded inside the CTA.
//
// Roles (6 + NDQ warps, one CTA per SM, persistent over the tile list of cb_moe_dispatch):
//   warp 0     TMA producer of the [128 x 64] bf16 A tiles (128B swizzle), one per k-block;
//   last warp  TMA producer of the codes, [256 rows x 64 B] per two k-blocks, into a ring of its own that runs
//              six k-blocks ahead (the codes come from HBM, the activations mostly from L2);
//   warps 6-   dequant, two groups of NDQ / 2 warps on alternate k-blocks: a thread owns RPT weight rows of the
//              tile and turns their 64 codes each into bf16 rows of the K-major 128B-swizzled B tile (ring of
//              BS stages): nibble -> 0x4300 | n (= 128 + n exactly in bf16), - 136, x scale;
//              fence.proxy.async; arrive on b_ready;
//   warp 1     MMA issuer: waits for the A tile (a_full) and the expanded B tile (b_ready), issues
//              tcgen05.mma (128 x 256 x 16, kind::f16) into one of two TMEM accumulators; tcgen05.commit
//              frees the A stage and the B stage;
//   warps 2-5  epilogue: tcgen05.ld, optional SwiGLU, bf16 store.
// Every wait is bounded (2 s) and reports through the status word.
// Replaces the reference's W4A8 expert-major grouped path (models/qwen35/moe.py:561-730,
// backends/corex/kernels/w8a8_tcu.cu:962).
#include <cuda_bf16.h>

#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int WM = 128, WN = 256, WAS = 3, WBS = 3, WCS = 3;   // A / expanded-B / code ring depths
constexpr int NDQ = 8;                           // dequant warps (two groups of NDQ / 2)
constexpr int RPT = WN / (NDQ * 16);             // weight rows of a tile per dequant thread
constexpr int kThreadsW4 = (7 + NDQ) * 32;         // the last warp feeds the code ring
constexpr int kMaxG = 20;          // groups of 128 along K a row may have (K <= 2560)
// a code stage holds 64 bytes (128 codes = two k-blocks) of each of the tile's 256 weight rows; the codes come
// from HBM (every weight tile is used once), so their ring is fed by a warp of its own, six k-blocks ahead
constexpr int A_BYTES_W = WM * 128, Q_BYTES_W = WN * 64, B_BYTES_W = WN * 128;

struct W4Args {
  bf16* C; int64_t ldc;
  const float* scale;              // [E, Nw, G]
  int rows, N, Nw, K, G;           // N: output columns; Nw: weight rows per expert (2N with SwiGLU)
  int n_tiles, k_blocks, max_tiles;
  int swiglu, up_off;              // SwiGLU: tile = 128 gate rows + the 128 up rows of the same outputs
  const int* g_count; const int* g_row0; const int* g_rows; const int* g_expert;
  int* status;
  unsigned long long* trace;     // optional: CTA 0 stamps %globaltimer per k-block (debugging aid), [k][4]
};

__device__ __forceinline__ uint64_t w4_now() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool w4_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = w4_now();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (w4_now() - t0 > 2000000000ull) return false;
  }
}
__device__ __forceinline__ void fence_async_smem_w4() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 8 codes (one 32-bit word: byte i = codes 2i, 2i+1) -> 8 bf16 (4 words), value (code - 8) * s
__device__ __forceinline__ void w4_expand(uint32_t w, __nv_bfloat162 s2, uint32_t* out) {
  const uint32_t lo = w & 0x0f0f0f0fu, hi = (w >> 4) & 0x0f0f0f0fu;
  const __nv_bfloat162 off = __floats2bfloat162_rn(136.f, 136.f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // bytes (lo.b_i, 0x43, hi.b_i, 0x43): two bf16 equal to 128 + code
    uint32_t p;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(p) : "r"(lo), "r"(hi), "r"((uint32_t)i | ((uint32_t)(4 + i) << 8)));
    p = (p & 0x00ff00ffu) | 0x43004300u;
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&p);
    v = __hmul2(__hsub2(v, off), s2);
    out[i] = *reinterpret_cast<uint32_t*>(&v);
  }
}

__global__ void __launch_bounds__(kThreadsW4, 1)
gemm_w4_grouped_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmQ, const W4Args a) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* codes = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* atiles = codes + WCS * Q_BYTES_W;
  unsigned char* btiles = atiles + WAS * A_BYTES_W;
  bf16* sc_s = reinterpret_cast<bf16*>(btiles + WBS * B_BYTES_W);      // [dequant group][G][256] scales of the current tile
  __shared__ uint64_t code_full[WCS], code_empty[WCS], a_full[WAS], a_empty[WAS], b_ready[WBS], b_empty[WBS], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < WCS; ++s) { mbar_init(&code_full[s], 1); mbar_init(&code_empty[s], NDQ); }
    for (int s = 0; s < WAS; ++s) { mbar_init(&a_full[s], 1); mbar_init(&a_empty[s], 1); }
    for (int s = 0; s < WBS; ++s) { mbar_init(&b_ready[s], NDQ / 2); mbar_init(&b_empty[s], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
    abort_s = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmQ);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  griddep_launch();
  griddep_wait();

  int m_tiles = *a.g_count;
  if (m_tiles > a.max_tiles) m_tiles = a.max_tiles;
  const int total = m_tiles * a.n_tiles;
  const int out_n = a.swiglu ? WN / 2 : WN;          // output columns per tile
  constexpr uint32_t IDESC = umma_idesc(WM, WN, 1, 1);

  if (warp == 0) {
    // ------------------------------- TMA producer -----------------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      // tile = (m-tile, n-tile) with the n-tiles of an m-tile consecutive: the CTAs that run side by side share
      // the activation tile through L2; every weight tile is read once anyway
      int m0n = 0;
      if ((int)blockIdx.x < total) m0n = a.g_row0[blockIdx.x / a.n_tiles];
      for (int tile = blockIdx.x; tile < total && !*abort_flag; tile += gridDim.x) {
        const int m0 = m0n;
        if (tile + (int)gridDim.x < total) m0n = a.g_row0[(tile + gridDim.x) / a.n_tiles];     // ahead of its use
        for (int kb = 0; kb < a.k_blocks; ++kb, ++it) {
          const int s = it % WAS;
          if (!w4_wait(&a_empty[s], ((it / WAS) & 1) ^ 1, abort_flag)) { atomicCAS(a.status, 0, 91); abort_s = 1; break; }
          mbar_expect_tx(&a_full[s], A_BYTES_W);
          tma_load_2d(atiles + (size_t)s * A_BYTES_W, &tmA, &a_full[s], kb * 64, m0);
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 6 + NDQ) {
    // ------------------------------- code producer ------------------------------------------
    if (lane == 0) {
      uint32_t ci = 0;
      int exn = 0;
      if ((int)blockIdx.x < total) exn = a.g_expert[blockIdx.x / a.n_tiles];
      for (int tile = blockIdx.x; tile < total && !*abort_flag; tile += gridDim.x) {
        const int wrow = exn * a.Nw + (tile % a.n_tiles) * out_n;
        if (tile + (int)gridDim.x < total) exn = a.g_expert[(tile + gridDim.x) / a.n_tiles];
        for (int kb = 0; kb < a.k_blocks; kb += 2, ++ci) {      // two boxes of 128 rows x 64 bytes
          const int cs = ci % WCS;
          if (!w4_wait(&code_empty[cs], ((ci / WCS) & 1) ^ 1, abort_flag)) { atomicCAS(a.status, 0, 90); abort_s = 1; break; }
          mbar_expect_tx(&code_full[cs], Q_BYTES_W);
          unsigned char* cst = codes + (size_t)cs * Q_BYTES_W;
          tma_load_2d(cst, &tmQ, &code_full[cs], kb * 32, wrow);
          tma_load_2d(cst + Q_BYTES_W / 2, &tmQ, &code_full[cs], kb * 32, wrow + (a.swiglu ? a.up_off : WN / 2));
        }
        if (*abort_flag) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------------------
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < total && !*abort_flag; tile += gridDim.x, ++tcount) {
        const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
        if (!w4_wait(&acc_empty[acc], aph ^ 1, abort_flag)) { atomicCAS(a.status, 0, 92); abort_s = 1; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * WN;
        bool ok = true;
        for (int kb = 0; kb < a.k_blocks; ++kb, ++it) {
          const int s = it % WAS, bs = it % WBS;
          if (!w4_wait(&a_full[s], (it / WAS) & 1, abort_flag) || !w4_wait(&b_ready[bs], (it / WBS) & 1, abort_flag)) {
            atomicCAS(a.status, 0, 93); abort_s = 1; ok = false; break;
          }
          tc_fence_after();
          if (a.trace && blockIdx.x == 0 && it < 96) a.trace[it * 4 + 3] = w4_now();
          const uint64_t ad = umma_desc_sw128(atiles + (size_t)s * A_BYTES_W), bd = umma_desc_sw128(btiles + (size_t)bs * B_BYTES_W);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(d_tmem, ad + 2 * k, bd + 2 * k, IDESC, (kb | k) != 0);
          umma_commit(&a_empty[s]);
          umma_commit(&b_empty[bs]);
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
      }
    }
  } else if (warp >= 6 && warp < 6 + NDQ) {
    // ------------------------------- dequant ----------------------------------------------------------
    // Two groups of four warps take alternate k-blocks, so a group has two k-block times for one tile and
    // the expansion of k-block n+1 overlaps that of n.  Thread tg of a group owns weight rows tg and tg + 128.
    const int grp = (warp - 6) / (NDQ / 2), tg = threadIdx.x - 6 * 32 - grp * (NDQ * 16);
    uint32_t it = 0;
    float4 sreg[RPT][kMaxG / 4];
    // weight row (inside its expert's block) of tile row r for n-tile nt, or -1 past the last output column
    auto row_of = [&](int nt, int r) {
      if (a.swiglu) return (nt * out_n + (r & (WN / 2 - 1)) < a.N) ? nt * out_n + (r < WN / 2 ? r : a.up_off + r - WN / 2) : -1;
      return nt * WN + r < a.N ? nt * WN + r : -1;
    };
    auto fetch_scales = [&](int tile) {
      const int ex = a.g_expert[tile / a.n_tiles], nt = tile % a.n_tiles;
#pragma unroll
      for (int h = 0; h < RPT; ++h) {
        const int wr = row_of(nt, tg + h * (NDQ * 16));
        if (wr >= 0) {
          const float4* sp = reinterpret_cast<const float4*>(a.scale + ((int64_t)ex * a.Nw + wr) * a.G);
#pragma unroll
          for (int i = 0; i < kMaxG / 4; ++i)
            if (i * 4 < a.G) sreg[h][i] = sp[i];
        }
      }
    };
    // scales as bf16 in shared memory, [dequant group][scale group][row]: the two dequant groups own the same
    // rows on alternate k-blocks and reach the end of a tile at different times, so each keeps its own copy
    // and a thread reads back only what it wrote
    auto store_scales = [&](int slot) {
#pragma unroll
      for (int h = 0; h < RPT; ++h) {
        bf16* dst = sc_s + (size_t)(slot + grp) * WN * a.G + tg + h * (NDQ * 16);
#pragma unroll
        for (int i = 0; i < kMaxG / 4; ++i) {
          if (i * 4 < a.G) {
            dst[(size_t)(4 * i) * WN] = __float2bfloat16(sreg[h][i].x);
            dst[(size_t)(4 * i + 1) * WN] = __float2bfloat16(sreg[h][i].y);
            dst[(size_t)(4 * i + 2) * WN] = __float2bfloat16(sreg[h][i].z);
            dst[(size_t)(4 * i + 3) * WN] = __float2bfloat16(sreg[h][i].w);
          }
        }
      }
    };
    if ((int)blockIdx.x < total) { fetch_scales(blockIdx.x); store_scales(0); }
    int tnum = 0;
    for (int tile = blockIdx.x; tile < total && !*abort_flag; tile += gridDim.x, ++tnum) {
      const int nt = tile % a.n_tiles;
      bool live[RPT];
#pragma unroll
      for (int h = 0; h < RPT; ++h) live[h] = row_of(nt, tg + h * (NDQ * 16)) >= 0;
      const bf16* scs = sc_s + (size_t)grp * WN * a.G + tg;
      if (tile + (int)gridDim.x < total) fetch_scales(tile + gridDim.x);     // stored after this tile
      bool ok = true;
      for (int kb = 0; kb < a.k_blocks; ++kb, ++it) {
        if ((int)(it & 1) != grp) continue;
        const uint32_t ci = it >> 1;
        const int cs = ci % WCS, bs = it % WBS, sub = it & 1;         // sub: which 32 bytes of the 64-byte code rows
        if (!w4_wait(&code_full[cs], (ci / WCS) & 1, abort_flag) || !w4_wait(&b_empty[bs], ((it / WBS) & 1) ^ 1, abort_flag)) {
          if (lane == 0) { atomicCAS(a.status, 0, 94); abort_s = 1; }
          ok = false; break;
        }
        const bool tr = a.trace && blockIdx.x == 0 && it < 96 && (tg == 0);
        if (tr) a.trace[it * 4 + 0] = w4_now();
#pragma unroll
        for (int h = 0; h < RPT; ++h) {
          const int r = tg + h * (NDQ * 16);
          const uint4* q = reinterpret_cast<const uint4*>(codes + (size_t)cs * Q_BYTES_W + r * 64 + sub * 32);
          const uint4 q0 = q[0], q1 = q[1];
          const bf16 sc = live[h] ? scs[(size_t)(kb >> 1) * WN + h * (NDQ * 16)] : __float2bfloat16(0.f);
          const __nv_bfloat162 s2 = __halves2bfloat162(sc, sc);
          unsigned char* brow = btiles + (size_t)bs * B_BYTES_W + r * 128;
          const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
          for (int c = 0; c < 8; ++c) {                    // word c = codes 8c .. 8c+7 = 16-byte chunk c of the row
            uint32_t o[4];
            w4_expand(words[c], s2, o);
            *reinterpret_cast<uint4*>(brow + ((c ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        if (tr) a.trace[it * 4 + 1] = w4_now();
        fence_async_smem_w4();
        __syncwarp();
        if (tr) a.trace[it * 4 + 2] = w4_now();
        if (lane == 0) {
          mbar_arrive(&b_ready[bs]);
          mbar_arrive(&code_empty[cs]);                        // this group's only read of the code stage
        }
      }
      if (!ok) break;
      store_scales(0);                                          // the next tile's scales over this tile's (own entries only)
    }
  } else {
    // ------------------------------- epilogue ---------------------------------------------
    const int q = warp & 3;
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < total && !*abort_flag; tile += gridDim.x, ++tcount) {
      const int mt = tile / a.n_tiles, nt = tile % a.n_tiles;
      const int m0 = a.g_row0[mt], row_end = m0 + a.g_rows[mt], n0 = nt * out_n;
      const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
      if (!w4_wait(&acc_full[acc], aph, abort_flag)) { if (lane == 0) { atomicCAS(a.status, 0, 95); abort_s = 1; } break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < out_n; c0 += 32) {
        uint32_t rg[32], ru[32];
        const uint32_t ta = tmem_base + acc * WN + ((uint32_t)(q * 32) << 16) + c0;
        tmem_ld32(ta, rg);
        if (a.swiglu) tmem_ld32(ta + WN / 2, ru);
        tmem_ld_wait();
        const int col0 = n0 + c0;
        if (row < row_end && col0 < a.N) {
          bf16* cp = a.C + (int64_t)row * a.ldc + col0;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col0 + v * 8 >= a.N) break;  // N is a multiple of 8
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float g = __uint_as_float(rg[v * 8 + i]);
              f[i] = a.swiglu ? silu_f(g) * __uint_as_float(ru[v * 8 + i]) : g;
            }
            *reinterpret_cast<uint4*>(cp + v * 8) = float_to_bf16x8(f);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
  }
  // ------------------------------- teardown ---------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (abort_s) {
    const uint64_t t0 = w4_now();
    while (w4_now() - t0 < 2000000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// codes viewed as a 2-D byte tensor [rows, K/2]: box [128 rows, 64 bytes], no swizzle
int make_code_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes) {
  cb_encode_tiled_fn enc = cb_get_encode();
  if (!enc) return CB_ERR_DRIVER;
  if (((uintptr_t)base & 15) || (row_bytes & 15)) return CB_ERR_SHAPE;
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : CB_ERR_DRIVER;
}

}  // namespace

// rows x K (bf16, sorted by expert) times the int4 stack Wq [E, Nw, K/2] with scales [E, Nw, K/128] (fp32).
// swiglu = 0: C [rows, N] with N = Nw.  swiglu = 1: Nw = 2N (gate rows, then up rows) and
// C [rows, N] = silu(gate) * up.  K % 128 == 0, N % 8 == 0.  The tile list comes from cb_moe_dispatch.
CB_EXPORT int cb_gemm_w4_grouped(const void* A, int64_t lda, const void* Wq, const void* wscale, void* C, int64_t ldc,
                                 int64_t rows, int64_t E, int64_t Nw, int64_t K, int64_t swiglu, const void* g_count,
                                 const void* g_row0, const void* g_rows, const void* g_expert, int64_t max_tiles,
                                 void* status, void* trace, void* stream) {
  if (rows < 1 || Nw < 1 || K < 1 || E < 1 || max_tiles < 1) return CB_ERR_SHAPE;
  const int64_t N = swiglu ? Nw / 2 : Nw;
  if (K / 128 > kMaxG || (K / 128) % 4 || K % 256) return CB_ERR_SHAPE;      // the scales of a row travel as float4, the codes four k-blocks at a time
  if (K % 128 || N % 8 || ldc % 8 || (swiglu && Nw % 2) || !status || !g_count || !g_row0 || !g_rows || !g_expert) return CB_ERR_SHAPE;
  CUtensorMap tmA, tmQ;
  int rc = cb_make_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, (uint64_t)rows, (uint64_t)K, (uint64_t)lda, WM, 64);
  if (rc) return rc;
  rc = make_code_map(&tmQ, Wq, (uint64_t)(E * Nw), (uint64_t)(K / 2));
  if (rc) return rc;
  W4Args a;
  a.C = (bf16*)C; a.ldc = ldc; a.scale = (const float*)wscale;
  a.rows = (int)rows; a.N = (int)N; a.Nw = (int)Nw; a.K = (int)K; a.G = (int)(K / 128);
  const int out_n = swiglu ? WN / 2 : WN;
  a.n_tiles = (int)((N + out_n - 1) / out_n); a.k_blocks = (int)(K / 64); a.max_tiles = (int)max_tiles;
  a.swiglu = swiglu ? 1 : 0; a.up_off = (int)N;
  a.g_count = (const int*)g_count; a.g_row0 = (const int*)g_row0; a.g_rows = (const int*)g_rows; a.g_expert = (const int*)g_expert;
  a.status = (int*)status; a.trace = (unsigned long long*)trace;
  const size_t smem = (size_t)WCS * Q_BYTES_W + (size_t)WAS * A_BYTES_W + (size_t)WBS * B_BYTES_W + (size_t)2 * WN * a.G * sizeof(bf16) + 1024;
  cudaError_t e = cudaFuncSetAttribute(gemm_w4_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t total = max_tiles * a.n_tiles;
  const int grid = (int)(total < sms ? total : sms);
  return (int)cb_launch(gemm_w4_grouped_kernel, dim3((unsigned)grid), dim3(kThreadsW4), smem, (cudaStream_t)stream, tmA, tmQ, a);
}
