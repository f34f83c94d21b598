// Causal flash attention for prefill chunks on the 5th-generation tensor cores.
//
// One CTA owns 128 consecutive query rows of one head and walks the sequence's KV pages (64 tokens
// each) from key 0 to the diagonal:
//   warp 0 (one thread)   TMA: Q once, then K and V pages into two-stage rings (page id from the block
//                         table; the pools are [slot, kv head, hd] so a page of one kv head is a
//                         [64 x hd] box, stored as hd/64 swizzled [64 x 128 B] blocks)
//   warp 1 (one thread)   tcgen05.mma: S_j = Q K_j^T into one of two TMEM accumulators (K-major
//                         operands), O += P_j V_j into a third (P from shared memory, V as an
//                         MN-major operand: the page is used as it lies in the pool, no transpose)
//   warps 2-5             softmax, one thread per query row: tcgen05.ld of the row's 64 scores, scale,
//                         causal mask, running sum, P = 2^(s - m_ref) as bf16 into shared memory
//                         in the swizzled K-major layout the MMA reads.  The reference maximum m_ref
//                         is raised (and the O accumulator in TMEM rescaled through tcgen05.ld/st)
//                         only when a row's maximum grew by more than 2^8 since it was set, so the
//                         rescale is rare after the first tiles; the final division by the running
//                         sum makes the result exact either way.
// S_{j+1} is issued before the softmax of S_j has finished, so the tensor core works under the
// exponentials.  The epilogue reads O from TMEM, divides by the row sum, applies the sigmoid output
// gate and stores bf16.  Every wait is bounded (2 s wall clock) and reports through the status word;
// TMEM is freed on every path.  Replaces, for bf16 pools and dense causal attention, the mma.sync
// kernel of attn.cu (reference role: models/qwen35/full_attn.py:658-789, flash prefill).
#include "sm100.cuh"

namespace {
using namespace sm100;

constexpr int kBQ = 128, kBKV = 64, kThreads = 192;

struct AttnTcArgs {
  const bf16* gate; int64_t ldg;   // gate of head h at gate[t*ldg + h*2*hd + hd + d] (null: no gate)
  const int* block_table;          // [pages] pool page ids of the sequence
  bf16* out; int64_t ldo;          // [T, nh*hd]
  int T, q_pos0, nh, nkv;
  float scale_log2;                // hd^-0.5 * log2(e)
  int* status;
};

__device__ __forceinline__ uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = now_ns();
  for (;;) {
    for (int i = 0; i < 128; ++i)
      if (mbar_try(bar, parity)) return true;
    if (*abort_flag) return false;
    if (now_ns() - t0 > 2000000000ull) return false;
  }
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// generic-proxy shared-memory writes -> visible to the tensor core's (async proxy) reads
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// MN-major operand written by TMA with 128-byte swizzle: [K rows of 128 bytes], 8-row groups 1024 bytes
// apart (stride offset), the next 64 elements of the MN dimension `chunk_bytes` further (leading offset).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(const void* smem_tile, uint32_t chunk_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(smem_tile) & 0x3FFFF) >> 4);
  d |= (uint64_t)(chunk_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

template <int HD>
__global__ void __launch_bounds__(kThreads, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const AttnTcArgs a) {
  constexpr int NC = HD / 64;                         // 64-element (128-byte) chunks of the head dimension
  constexpr int Q_BYTES = kBQ * HD * 2, KV_BYTES = kBKV * HD * 2, P_BYTES = kBQ * kBKV * 2;
  constexpr int QC = kBQ * 128, KC = kBKV * 128;      // bytes of one chunk block of Q / of a K or V page
  constexpr uint32_t TMEM_COLS = 2 * kBKV + HD <= 256 ? 256 : 512;
  constexpr uint32_t IDESC_S = umma_idesc(kBQ, kBKV, 1, 1);
  constexpr uint32_t IDESC_O = umma_idesc(kBQ, HD, 1, 1) | (1u << 16);     // B operand MN-major
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* Qs = base;
  unsigned char* Ks = Qs + Q_BYTES;                   // [2][KV_BYTES]
  unsigned char* Vs = Ks + 2 * KV_BYTES;
  unsigned char* Ps = Vs + 2 * KV_BYTES;              // [2][P_BYTES]
  __shared__ uint64_t q_full, k_full[2], v_full[2], k_free[2], v_free[2], s_full[2], s_free[2], p_full[2], p_free[2], o_full;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query tiles first: they walk the most pages
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y, kvh = h / (a.nh / a.nkv);
  const int row0 = qt * kBQ;
  const int last_row = min(a.T, row0 + kBQ) - 1;
  const int n_tiles = (a.q_pos0 + last_row) / kBKV + 1;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    mbar_init(&o_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&k_free[i], 1); mbar_init(&v_free[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 4); mbar_init(&p_full[i], 4); mbar_init(&p_free[i], 1);
    }
    abort_s = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t tmem_o = tmem_base + 2 * kBKV;       // S0 | S1 | O
  griddep_launch();
  griddep_wait();

  if (warp == 0) {
    // ------------------------------------ TMA producer ------------------------------------------
    if (lane == 0) {
      mbar_expect_tx(&q_full, Q_BYTES);
      for (int c = 0; c < NC; ++c) tma_load_2d(Qs + c * QC, &tmQ, &q_full, h * HD + c * 64, row0);
      for (int j = 0; j < n_tiles && !*abort_flag; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int slot0 = a.block_table[j] * kBKV;
        if (!wait_bar(&k_free[s], ph ^ 1, abort_flag)) { atomicCAS(a.status, 0, 65); abort_s = 1; break; }
        mbar_expect_tx(&k_full[s], KV_BYTES);
        for (int c = 0; c < NC; ++c) tma_load_2d(Ks + s * KV_BYTES + c * KC, &tmK, &k_full[s], kvh * HD + c * 64, slot0);
        if (!wait_bar(&v_free[s], ph ^ 1, abort_flag)) { atomicCAS(a.status, 0, 66); abort_s = 1; break; }
        mbar_expect_tx(&v_full[s], KV_BYTES);
        for (int c = 0; c < NC; ++c) tma_load_2d(Vs + s * KV_BYTES + c * KC, &tmV, &v_full[s], kvh * HD + c * 64, slot0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------ MMA issuer --------------------------------------------
    if (lane == 0) {
      bool ok = wait_bar(&q_full, 0, abort_flag);
      if (!ok) { atomicCAS(a.status, 0, 67); abort_s = 1; }
      // S_j = Q K_j^T
      auto issue_s = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!wait_bar(&k_full[s], ph, abort_flag)) { atomicCAS(a.status, 0, 68); abort_s = 1; return false; }
        if (!wait_bar(&s_free[s], ph ^ 1, abort_flag)) { atomicCAS(a.status, 0, 69); abort_s = 1; return false; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const uint64_t qd = umma_desc_sw128(Qs + c * QC), kd = umma_desc_sw128(Ks + s * KV_BYTES + c * KC);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(tmem_base + s * kBKV, qd + 2 * k, kd + 2 * k, IDESC_S, (c | k) != 0);
        }
        umma_commit(&k_free[s]);
        umma_commit(&s_full[s]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (!ok) break;
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!wait_bar(&p_full[s], ph, abort_flag)) { atomicCAS(a.status, 0, 70); abort_s = 1; break; }
        if (!wait_bar(&v_full[s], ph, abort_flag)) { atomicCAS(a.status, 0, 71); abort_s = 1; break; }
        tc_fence_after();
        const uint64_t pd = umma_desc_sw128(Ps + s * P_BYTES);
        const uint64_t vd = umma_desc_mn_sw128(Vs + s * KV_BYTES, KC);
#pragma unroll
        for (int k = 0; k < 4; ++k)      // 16 keys per instruction: +32 bytes along P's rows, +16 rows of V
          umma_f16(tmem_o, pd + 2 * k, vd + (uint64_t)(k * 16 * 128 >> 4), IDESC_O, (j | k) != 0);
        umma_commit(&v_free[s]);
        umma_commit(&p_free[s]);
      }
      if (ok) umma_commit(&o_full);
    }
  } else {
    // ------------------------------------ softmax + epilogue ------------------------------------
    const int q = warp & 3;                            // TMEM lane quadrant this warp may access
    const int r = q * 32 + lane;                       // query row of this thread inside the tile
    const int t = row0 + r, pos = a.q_pos0 + t;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!wait_bar(&s_full[s], ph, abort_flag)) { if (lane == 0) { atomicCAS(a.status, 0, 72); abort_s = 1; } ok = false; break; }
      tc_fence_after();
      uint32_t sv[64];
      tmem_ld32(tmem_base + lane_base + s * kBKV, sv);
      tmem_ld32(tmem_base + lane_base + s * kBKV + 32, sv + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[s]);          // the accumulator may take S_{j+2}
      const int key0 = j * kBKV;
      float mx = -INFINITY;
      if (key0 + kBKV - 1 > a.q_pos0 + row0) {         // the tile touches the diagonal
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const float x = key0 + c <= pos ? __uint_as_float(sv[c]) * a.scale_log2 : -INFINITY;
          sv[c] = __float_as_uint(x);
          mx = fmaxf(mx, x);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const float x = __uint_as_float(sv[c]) * a.scale_log2;
          sv[c] = __float_as_uint(x);
          mx = fmaxf(mx, x);
        }
      }
      if (j == 0) {
        m_ref = mx;                                    // key 0 is visible to every row: finite
      } else if (__any_sync(0xffffffffu, mx > m_ref + 8.f)) {
        // raise the reference maximum of this warp's rows and rescale their O rows in TMEM; every
        // product that wrote O has to be complete first (the one of this tile cannot start before P)
        if (!wait_bar(&p_free[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag)) {
          if (lane == 0) { atomicCAS(a.status, 0, 73); abort_s = 1; }
          ok = false;
          break;
        }
        tc_fence_after();
        const float m_new = fmaxf(m_ref, mx);
        const float f = ex2(m_ref - m_new);
        m_ref = m_new;
        l *= f;
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld32(tmem_o + lane_base + c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
          tmem_st32(tmem_o + lane_base + c0, o);
        }
        tmem_st_wait();
        tc_fence_before();
      }
      // P = 2^(s - m_ref) as bf16, running sum in fp32
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float p0 = ex2(__uint_as_float(sv[2 * c]) - m_ref), p1 = ex2(__uint_as_float(sv[2 * c + 1]) - m_ref);
        l += p0 + p1;
        const __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
        pk[c] = *reinterpret_cast<const uint32_t*>(&b);
      }
      if (j >= 2 && !wait_bar(&p_free[s], ((j - 2) >> 1) & 1, abort_flag)) {   // the product of tile j-2 has read this buffer
        if (lane == 0) { atomicCAS(a.status, 0, 74); abort_s = 1; }
        ok = false;
        break;
      }
      unsigned char* prow = Ps + s * P_BYTES + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)                      // 16-byte chunk c of row r lives at chunk c ^ (r % 8)
        *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[s]);
    }
    if (ok && !wait_bar(&o_full, 0, abort_flag)) { if (lane == 0) { atomicCAS(a.status, 0, 75); abort_s = 1; } ok = false; }
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l;
      const bf16* gp = a.gate ? a.gate + (int64_t)t * a.ldg + (int64_t)h * 2 * HD + HD : nullptr;
      bf16* op = a.out + (int64_t)t * a.ldo + (int64_t)h * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t o[32];
        tmem_ld32(tmem_o + lane_base + c0, o);         // warp-collective: rows beyond T load too
        tmem_ld_wait();
        if (t < a.T) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(o[v * 8 + i]) * inv;
            if (gp) {
              float g[8];
              bf16x8_to_float(*reinterpret_cast<const uint4*>(gp + c0 + v * 8), g);
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] *= 1.f / (1.f + __expf(-g[i]));
            }
            *reinterpret_cast<uint4*>(op + c0 + v * 8) = float_to_bf16x8(f);
          }
        }
      }
    }
  }
  // ------------------------------------ teardown --------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (abort_s) {  // give copies still in flight time to land before the shared memory is released
    const uint64_t t0 = now_ns();
    while (now_ns() - t0 < 2000000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int HD>
int launch_attn_tc(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnTcArgs& a, cudaStream_t st) {
  const size_t smem = (size_t)kBQ * HD * 2 + 4 * (size_t)kBKV * HD * 2 + 2 * (size_t)kBQ * kBKV * 2 + 1024;
  auto kern = attn_tc_kernel<HD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((unsigned)((a.T + kBQ - 1) / kBQ), (unsigned)a.nh);
  return (int)cb_launch(kern, grid, dim3(kThreads), smem, st, tmQ, tmK, tmV, a);
}
}  // namespace

// q [T, nh, hd] bf16 (normed, rotated); pools [slots, nkv, hd] bf16; causal; hd 64 or 256.
CB_EXPORT int cb_attn_prefill_tc(const void* q, const void* gate, int64_t ldg, const void* kpool, const void* vpool,
                                 int64_t slots, const void* block_table, void* out, int64_t ldo, int64_t T,
                                 int64_t q_pos0, int64_t nh, int64_t nkv, int64_t hd, void* status, void* stream) {
  if (T == 0) return 0;
  if (!q || !kpool || !vpool || !block_table || !out || !status || nh % nkv || (hd != 64 && hd != 256)) return CB_ERR_SHAPE;
  CUtensorMap tmQ, tmK, tmV;
  int rc = cb_make_tmap_2d(&tmQ, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, (uint64_t)T, (uint64_t)(nh * hd), (uint64_t)(nh * hd), kBQ, 64);
  if (rc) return rc;
  rc = cb_make_tmap_2d(&tmK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kpool, (uint64_t)slots, (uint64_t)(nkv * hd), (uint64_t)(nkv * hd), kBKV, 64);
  if (rc) return rc;
  rc = cb_make_tmap_2d(&tmV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, vpool, (uint64_t)slots, (uint64_t)(nkv * hd), (uint64_t)(nkv * hd), kBKV, 64);
  if (rc) return rc;
  AttnTcArgs a{(const bf16*)gate, ldg, (const int*)block_table, (bf16*)out, ldo, (int)T, (int)q_pos0, (int)nh, (int)nkv,
               1.4426950408889634f / sqrtf((float)hd), (int*)status};
  if (hd == 256) return launch_attn_tc<256>(tmQ, tmK, tmV, a, (cudaStream_t)stream);
  return launch_attn_tc<64>(tmQ, tmK, tmV, a, (cudaStream_t)stream);
}
