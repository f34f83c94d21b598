// Causal flash attention for prefill chunks on the 5th-generation tensor cores.
//
// One CTA owns 128 consecutive query rows of one head and walks the sequence's KV pages (64 tokens
// each) from key 0 to the diagonal:
//   warp 0 (one thread)   TMA: K and V pages into three-stage rings (page id from the block table; the
//                         pools are [slot, kv head, hd] so a page of one kv head is a [64 x hd] box,
//                         stored as hd/64 swizzled [64 x 128 B] blocks)
//   warps 1 and 10        (one thread each) tcgen05.mma: S_j = Q K_j^T into one of two TMEM accumulators with Q read from
//                         TENSOR MEMORY (the A operand; with Q in shared memory the 128 x 64 products were
//                         bound by the shared-memory port, 0.74 us instead of 0.27 us per page), O += P_j V_j
//                         into a third (P from shared memory, V as an MN-major operand: the page is used
//                         as it lies in the pool, no transpose)
//   warps 2-9             first store their Q rows into tensor memory (tcgen05.st), then softmax: two
//                         threads per query row (the two warps that share a TMEM lane quadrant take one
//                         half of the row's 64 scores each; maxima and sums meet in shared memory):
//                         tcgen05.ld, scale, causal mask, P = 2^(s - m_ref) as bf16 into shared memory in
//                         the swizzled K-major layout the MMA reads.  The reference maximum m_ref is raised
//                         (and the O accumulator in TMEM rescaled through tcgen05.ld/st) only when a row's
//                         maximum grew by more than 2^8 since it was set, so the rescale is rare after the
//                         first tiles; the final division by the running sum makes the result exact
//                         either way.
// S_{j+1} is issued before the softmax of S_j has finished, so the tensor core works under the
// exponentials.  The epilogue reads O from TMEM, divides by the row sum, applies the sigmoid output
// gate and stores bf16.  Every wait is an mbarrier wait bounded by 2 s of wall clock that reports through
// the status word (no named barriers: a warp that gave up cannot strand its partner); TMEM is freed on
// every path.  Replaces, for bf16 pools and dense causal attention, the mma.sync
// kernel of attn.cu (reference role: models/qwen35/full_attn.py:658-789, flash prefill).
#include <cuda_fp16.h>

#include "sm100.cuh"

namespace {
using namespace sm100;

constexpr int kBQ = 128, kBKV = 64, kThreads = 352, kStages = 3;

struct AttnTcArgs {
  const bf16* q;                   // [T, nh, hd] normed and rotated queries
  const bf16* gate; int64_t ldg;   // gate of head h at gate[t*ldg + h*2*hd + hd + d] (null: no gate)
  const int* block_table;          // [pages] pool page ids of the sequence
  bf16* out; int64_t ldo;          // [T, nh*hd]
  int T, q_pos0, nh, nkv;
  float scale_log2;                // hd^-0.5 * log2(e)
  int* status;
  unsigned long long* trace;       // debugging: [tiles][8] %globaltimer stamps of CTA (0, 0), or null
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

// A operand read from tensor memory (lane = row, every 32-bit column holds two consecutive K elements).
__device__ __forceinline__ void umma_f16_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}

template <int HD>
__global__ void __launch_bounds__(kThreads, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const AttnTcArgs a) {
  constexpr int NC = HD / 64;                         // 64-element (128-byte) chunks of the head dimension
  constexpr int KV_BYTES = kBKV * HD * 2, P_BYTES = kBQ * kBKV * 2;
  constexpr int KC = kBKV * 128;                      // bytes of one chunk block of a K or V page
  constexpr int QCOLS = HD / 2;                       // TMEM columns of the Q tile (two bf16 per column)
  constexpr uint32_t TMEM_COLS = 2 * kBKV + HD + QCOLS <= 256 ? 256 : 512;
  constexpr uint32_t IDESC_S = umma_idesc(kBQ, kBKV, 1, 1);
  constexpr uint32_t IDESC_O = umma_idesc(kBQ, HD, 1, 1) | (1u << 16);     // B operand MN-major
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* Ks = base;                           // [kStages][KV_BYTES]
  unsigned char* Vs = Ks + kStages * KV_BYTES;
  unsigned char* Ps = Vs + kStages * KV_BYTES;        // [2][P_BYTES]
  __shared__ uint64_t q_full, k_full[kStages], v_full[kStages], k_free[kStages], v_free[kStages], s_full[2], s_free[2],
      p_full[2], p_free[2], o_full, pair_bar[4];
  __shared__ __half xch[2][2][kBQ];                   // [tile parity][column half][row]: half-row maxima (both halves read
                                                      // the same rounded values, so they agree on the reference)
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;
  volatile int* abort_flag = &abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query tiles first: they walk the most pages
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y, kvh = h / (a.nh / a.nkv);
  const int row0 = qt * kBQ;
  const bool traced = a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
  // stamp slots per tile: 0 K landed (seen by the MMA thread), 1 S issued, 2 S complete (seen by softmax),
  // 3 P published, 4 P and V seen by the MMA thread, 5 PV issued, 6 K requested, 7 V requested
  auto stamp = [&](int j, int slot) { if (traced) a.trace[j * 8 + slot] = now_ns(); };
  const int last_row = min(a.T, row0 + kBQ) - 1;
  const int n_tiles = (a.q_pos0 + last_row) / kBKV + 1;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 8);
    mbar_init(&o_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&k_free[i], 1); mbar_init(&v_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 8); mbar_init(&p_full[i], 8); mbar_init(&p_free[i], 1);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], 64);
    abort_s = 0;
    mbar_fence_init();
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
  const uint32_t tmem_o = tmem_base + 2 * kBKV;       // S0 | S1 | O | Q
  const uint32_t tmem_q = tmem_o + HD;
  griddep_launch();
  griddep_wait();

  if (warp == 0) {
    // ------------------------------------ TMA producer ------------------------------------------
    if (lane == 0) {
      for (int j = 0; j < n_tiles && !*abort_flag; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        const int slot0 = a.block_table[j] * kBKV;
        if (!wait_bar(&k_free[s], ph ^ 1, abort_flag)) { atomicCAS(a.status, 0, 65); abort_s = 1; break; }
        mbar_expect_tx(&k_full[s], KV_BYTES);
        stamp(j, 6);
        for (int c = 0; c < NC; ++c) tma_load_2d(Ks + s * KV_BYTES + c * KC, &tmK, &k_full[s], kvh * HD + c * 64, slot0);
        if (!wait_bar(&v_free[s], ph ^ 1, abort_flag)) { atomicCAS(a.status, 0, 66); abort_s = 1; break; }
        mbar_expect_tx(&v_full[s], KV_BYTES);
        stamp(j, 7);
        for (int c = 0; c < NC; ++c) tma_load_2d(Vs + s * KV_BYTES + c * KC, &tmV, &v_full[s], kvh * HD + c * 64, slot0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------ MMA issuer: S_j = Q K_j^T -----------------------------
    // Q from tensor memory, so only the K page crosses the shared-memory port.  The sixteen 128 x 64 x 16
    // products of a page are bound by this thread's issue rate, not by the tensor pipe, which is why
    // the O += P V products are issued by a thread of their own (warp 10).
    if (lane == 0) {
      bool ok = wait_bar(&q_full, 0, abort_flag);      // the softmax warps have stored Q into tensor memory
      if (!ok) { atomicCAS(a.status, 0, 67); abort_s = 1; }
      tc_fence_after();
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kStages, sb = j & 1;
        if (!wait_bar(&k_full[s], (j / kStages) & 1, abort_flag)) { atomicCAS(a.status, 0, 68); abort_s = 1; break; }
        stamp(j, 0);
        if (!wait_bar(&s_free[sb], ((j >> 1) & 1) ^ 1, abort_flag)) { atomicCAS(a.status, 0, 69); abort_s = 1; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const uint64_t kd = umma_desc_sw128(Ks + s * KV_BYTES + c * KC);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ta(tmem_base + sb * kBKV, tmem_q + c * 32 + k * 8, kd + 2 * k, IDESC_S, (c | k) != 0);
        }
        umma_commit(&k_free[s]);
        umma_commit(&s_full[sb]);
        stamp(j, 1);
      }
    }
  } else if (warp == 10) {
    // ------------------------------------ MMA issuer: O += P_j V_j ------------------------------
    if (lane == 0) {
      bool ok = true;
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kStages, sb = j & 1;
        if (!wait_bar(&p_full[sb], (j >> 1) & 1, abort_flag)) { atomicCAS(a.status, 0, 70); abort_s = 1; ok = false; break; }
        if (!wait_bar(&v_full[s], (j / kStages) & 1, abort_flag)) { atomicCAS(a.status, 0, 71); abort_s = 1; ok = false; break; }
        stamp(j, 4);
        tc_fence_after();
        const uint64_t pd = umma_desc_sw128(Ps + sb * P_BYTES);
        const uint64_t vd = umma_desc_mn_sw128(Vs + s * KV_BYTES, KC);
#pragma unroll
        for (int k = 0; k < 4; ++k)      // 16 keys per instruction: +32 bytes along P's rows, +16 rows of V
          umma_f16(tmem_o, pd + 2 * k, vd + (uint64_t)(k * 16 * 128 >> 4), IDESC_O, (j | k) != 0);
        umma_commit(&v_free[s]);
        umma_commit(&p_free[sb]);
        stamp(j, 5);
      }
      if (ok) umma_commit(&o_full);
    }
  } else {
    // ------------------------------------ softmax + epilogue ------------------------------------
    // Two warps share a TMEM lane quadrant (32 query rows): warp w takes the left half of every row's
    // 64 scores and of its O row, warp w + 4 the right half; row maxima and sums meet in shared memory.
    const int q = warp & 3, hf = (warp - 2) >> 2;
    const int r = q * 32 + lane;                       // query row of this thread inside the tile
    const int t = row0 + r, pos = a.q_pos0 + t;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    // ---- Q row -> tensor memory (64 elements per store; the two warps of a quadrant alternate)
    {
      const bf16* qrow = a.q + ((int64_t)min(t, a.T - 1) * a.nh + h) * HD;
#pragma unroll 1
      for (int i = hf; i < HD / 64; i += 2) {
        uint32_t w[32];
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          const uint4 x = *reinterpret_cast<const uint4*>(qrow + i * 64 + v * 8);
          w[4 * v] = x.x; w[4 * v + 1] = x.y; w[4 * v + 2] = x.z; w[4 * v + 3] = x.w;
        }
        tmem_st32(tmem_q + lane_base + i * 32, w);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_full);
    }
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    uint32_t xph = 0;                                  // phase of the pair barrier
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!wait_bar(&s_full[sb], ph, abort_flag)) { if (lane == 0) { atomicCAS(a.status, 0, 72); abort_s = 1; } ok = false; break; }
      tc_fence_after();
      if (warp == 2 && lane == 0) stamp(j, 2);
      uint32_t sv[32];
      tmem_ld32(tmem_base + lane_base + sb * kBKV + hf * 32, sv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[sb]);         // the accumulator may take S_{j+2}
      const int key0 = j * kBKV + hf * 32;
      float mx0 = -INFINITY, mx1 = -INFINITY;
      if (j * kBKV + kBKV - 1 > a.q_pos0 + row0) {     // the tile touches the diagonal
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float x0 = key0 + c <= pos ? __uint_as_float(sv[c]) * a.scale_log2 : -INFINITY;
          const float x1 = key0 + c + 1 <= pos ? __uint_as_float(sv[c + 1]) * a.scale_log2 : -INFINITY;
          sv[c] = __float_as_uint(x0); sv[c + 1] = __float_as_uint(x1);
          mx0 = fmaxf(mx0, x0); mx1 = fmaxf(mx1, x1);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float x0 = __uint_as_float(sv[c]) * a.scale_log2, x1 = __uint_as_float(sv[c + 1]) * a.scale_log2;
          sv[c] = __float_as_uint(x0); sv[c + 1] = __float_as_uint(x1);
          mx0 = fmaxf(mx0, x0); mx1 = fmaxf(mx1, x1);
        }
      }
      // the row maximum needs the other half
      xch[sb][hf][r] = __float2half_rd(fmaxf(mx0, mx1));
      mbar_arrive(&pair_bar[q]);
      if (!wait_bar(&pair_bar[q], xph, abort_flag)) { if (lane == 0) { atomicCAS(a.status, 0, 76); abort_s = 1; } ok = false; break; }
      xph ^= 1;
      const float mx = fmaxf(__half2float(xch[sb][0][r]), __half2float(xch[sb][1][r]));
      if (j == 0) {
        m_ref = mx;                                    // key 0 is visible to every row: finite
      } else if (__any_sync(0xffffffffu, mx > m_ref + 8.f)) {
        // raise the reference maximum of these rows and rescale this warp's half of their O rows in
        // TMEM; every product that wrote O has to be complete first (the one of this tile cannot
        // start before P).  Both warps of the quadrant see the same maxima and take the same branch.
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
        for (int c0 = hf * (HD / 2); c0 < (hf + 1) * (HD / 2); c0 += 32) {
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
      // P = 2^(s - m_ref) as bf16, running sum in fp32 (two chains)
      uint32_t pk[16];
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float p0 = ex2(__uint_as_float(sv[2 * c]) - m_ref), p1 = ex2(__uint_as_float(sv[2 * c + 1]) - m_ref);
        l0 += p0; l1 += p1;
        const __nv_bfloat162 b = __floats2bfloat162_rn(p0, p1);
        pk[c] = *reinterpret_cast<const uint32_t*>(&b);
      }
      l += l0 + l1;
      if (j >= 2 && !wait_bar(&p_free[sb], ((j - 2) >> 1) & 1, abort_flag)) {   // the product of tile j-2 has read this buffer
        if (lane == 0) { atomicCAS(a.status, 0, 74); abort_s = 1; }
        ok = false;
        break;
      }
      unsigned char* prow = Ps + sb * P_BYTES + r * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c)                      // 16-byte chunk c of row r lives at chunk c ^ (r % 8)
        *reinterpret_cast<uint4*>(prow + (((hf * 4 + c) ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[sb]);
      if (warp == 2 && lane == 0) stamp(j, 3);
    }
    if (ok && !wait_bar(&o_full, 0, abort_flag)) { if (lane == 0) { atomicCAS(a.status, 0, 75); abort_s = 1; } ok = false; }
    // the two halves of a row add their sums (through the P buffer, which no product reads any more)
    if (ok) {
      float* lx = reinterpret_cast<float*>(Ps);
      lx[hf * kBQ + r] = l;
      mbar_arrive(&pair_bar[q]);
      if (!wait_bar(&pair_bar[q], xph, abort_flag)) { if (lane == 0) { atomicCAS(a.status, 0, 77); abort_s = 1; } ok = false; }
      else l = lx[r] + lx[kBQ + r];
    }
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l;
      const bf16* gp = a.gate ? a.gate + (int64_t)t * a.ldg + (int64_t)h * 2 * HD + HD : nullptr;
      bf16* op = a.out + (int64_t)t * a.ldo + (int64_t)h * HD;
#pragma unroll 1
      for (int c0 = hf * (HD / 2); c0 < (hf + 1) * (HD / 2); c0 += 32) {
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
int launch_attn_tc(const CUtensorMap& tmK, const CUtensorMap& tmV, const AttnTcArgs& a, cudaStream_t st) {
  const size_t smem = 2 * (size_t)kStages * kBKV * HD * 2 + 2 * (size_t)kBQ * kBKV * 2 + 1024;
  auto kern = attn_tc_kernel<HD>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid((unsigned)((a.T + kBQ - 1) / kBQ), (unsigned)a.nh);
  return (int)cb_launch(kern, grid, dim3(kThreads), smem, st, tmK, tmV, a);
}
}  // namespace

// q [T, nh, hd] bf16 (normed, rotated); pools [slots, nkv, hd] bf16; causal; hd 64 or 256.
CB_EXPORT int cb_attn_prefill_tc(const void* q, const void* gate, int64_t ldg, const void* kpool, const void* vpool,
                                 int64_t slots, const void* block_table, void* out, int64_t ldo, int64_t T,
                                 int64_t q_pos0, int64_t nh, int64_t nkv, int64_t hd, void* status, void* trace, void* stream) {
  if (T == 0) return 0;
  if (!q || !kpool || !vpool || !block_table || !out || !status || nh % nkv || (hd != 64 && hd != 256)) return CB_ERR_SHAPE;
  if ((uintptr_t)q & 15) return CB_ERR_ARG;
  CUtensorMap tmK, tmV;
  int rc = cb_make_tmap_2d(&tmK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, kpool, (uint64_t)slots, (uint64_t)(nkv * hd), (uint64_t)(nkv * hd), kBKV, 64);
  if (rc) return rc;
  rc = cb_make_tmap_2d(&tmV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, vpool, (uint64_t)slots, (uint64_t)(nkv * hd), (uint64_t)(nkv * hd), kBKV, 64);
  if (rc) return rc;
  AttnTcArgs a{(const bf16*)q, (const bf16*)gate, ldg, (const int*)block_table, (bf16*)out, ldo, (int)T, (int)q_pos0, (int)nh, (int)nkv,
               1.4426950408889634f / sqrtf((float)hd), (int*)status, (unsigned long long*)trace};
  if (hd == 256) return launch_attn_tc<256>(tmK, tmV, a, (cudaStream_t)stream);
  return launch_attn_tc<64>(tmK, tmV, a, (cudaStream_t)stream);
}
