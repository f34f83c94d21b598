// Gated GQA softmax attention over a paged bf16 KV pool.
//
//  * attn_prep:    per-head q/k RMSNorm + partial rotary + K/V append to the pool (prefill rows).
//  * attn_prefill: causal flash attention, one CTA per (64-query tile, q head), tensor-core
//                  QK^T and PV (bf16 mma, fp32 softmax state), sigmoid output gate in the epilogue.
//                  Also serves speculative verification (a few queries per row, causal among them).
//  * attn_decode:  one query per row, split over key tiles; the CTA that owns the tile holding
//                  the current position also norms/rotates/appends this token's K/V, so a decode
//                  layer needs no separate rope / kv-store launches.
//    (the last split of a group to arrive merges the partials and applies the gate).
// The reference has decode kernels (backends/corex/kernels/attn.cu:370-566: slice + combine over
// an int8 cache through pos2slot) but prefill attention is torch code
// (models/qwen35/full_attn.py:658-789); rope, kv_quant and kv_pool_store are separate launches
// there (attn.cu:132,249,1200).  The pool here is [slots, nkv, hd] per layer, addressed through
// a per-row block table (block = 64 tokens).
#include "common.cuh"

namespace {

constexpr int kBlock = 64;  // tokens per KV block == key tile

// ---- int8 KV pool (optional) ------------------------------------------------------------------
// With scale pointers set, the pools hold int8 [slots, nkv, hd] and one fp32 scale per (slot, kv head):
// x ~= q * scale, scale = max|x| / 127 (floored at 1e-8), the reference's paged int8 cache
// (cache/paged_cache.py:78-141, kv_quant / kv_pool_store in backends/corex/kernels/attn.cu:132,1200).
// Every kernel converts on load into the bf16 form it already computes with, so the products and the
// softmax are unchanged; only the bytes read per key halve.
//
// Quantise a head row held as EPL consecutive values per lane; returns the scale and leaves the
// dequantised values in x (what later steps will read back).
template <int EPL>
__device__ __forceinline__ float quant_row_q8(float* x, int8_t* dst_row, int lane) {
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(x[e]));
  amax = warp_max(amax);
  const float sc = fmaxf(amax / 127.f, 1e-8f), inv = 1.f / sc;
  int q[EPL];
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    q[e] = max(-127, min(127, __float2int_rn(x[e] * inv)));
    x[e] = (float)q[e] * sc;
  }
  if (EPL == 8) {
    uint2 w;
    w.x = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    w.y = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
    *reinterpret_cast<uint2*>(dst_row + lane * EPL) = w;
  } else {
#pragma unroll
    for (int e = 0; e < EPL; ++e) dst_row[lane * EPL + e] = (int8_t)q[e];
  }
  return sc;
}
// 8 int8 (one 8-byte vector) times a scale -> 8 bf16 (one 16-byte vector)
__device__ __forceinline__ uint4 q8x8_to_bf16x8(uint2 w, float sc) {
  float f[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[i] = (float)(int8_t)((w.x >> (8 * i)) & 0xff) * sc;
    f[4 + i] = (float)(int8_t)((w.y >> (8 * i)) & 0xff) * sc;
  }
  return float_to_bf16x8(f);
}
// A 64-key tile of K and V of one kv head into shared memory as bf16 rows of LD elements: asynchronous
// 16-byte copies from a bf16 pool, or 8-byte loads + conversion from an int8 pool.
template <int HD, int NT>
__device__ __forceinline__ void load_kv_tile(bf16* Ks, bf16* Vs, int LD, const bf16* kpool, const bf16* vpool,
                                             const float* kscale, const float* vscale, int64_t slot0, int nkv, int kvh,
                                             int tid) {
  constexpr int CPR = HD / 8;
  if (kscale) {
    const int8_t* k8 = reinterpret_cast<const int8_t*>(kpool);
    const int8_t* v8 = reinterpret_cast<const int8_t*>(vpool);
    for (int idx = tid; idx < 64 * CPR; idx += NT) {
      const int r = idx / CPR, c = idx % CPR;
      const int64_t row = (slot0 + r) * nkv + kvh;
      const uint2 kq = *reinterpret_cast<const uint2*>(k8 + row * HD + c * 8);
      const uint2 vq = *reinterpret_cast<const uint2*>(v8 + row * HD + c * 8);
      *reinterpret_cast<uint4*>(Ks + r * LD + c * 8) = q8x8_to_bf16x8(kq, kscale[row]);
      *reinterpret_cast<uint4*>(Vs + r * LD + c * 8) = q8x8_to_bf16x8(vq, vscale[row]);
    }
    return;
  }
  for (int idx = tid; idx < 64 * CPR; idx += NT) {
    const int r = idx / CPR, c = idx % CPR;
    const int64_t off = ((slot0 + r) * nkv + kvh) * HD + c * 8;
    const uint32_t ka = (uint32_t)__cvta_generic_to_shared(Ks + r * LD + c * 8);
    const uint32_t va = (uint32_t)__cvta_generic_to_shared(Vs + r * LD + c * 8);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ka), "l"(kpool + off));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(va), "l"(vpool + off));
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
}

// ------------------------------------------------------------------------------------------
// q/k norm + rope (+ KV append) for prefill rows. One warp per (token, head).
struct PrepArgs {
  const bf16* proj; int64_t ldp;     // [T, ldp]: (q|gate) per head, then k heads, then v heads
  const float* qg; const float* kg;  // [hd] gains (1 + w)
  const float* cos; const float* sin;  // [rows, rot]
  const int* rope_idx;               // [T] row of cos/sin per token (null: t)
  const int* kv_slot;                // [T] flat pool slot per token
  bf16* q_out;                       // [T, nh, hd]
  bf16* kpool; bf16* vpool;          // [slots, nkv, hd]
  int T, nh, nkv, rot;
  float eps;
  float* kscale; float* vscale;      // int8 pools: [slots, nkv] scales (null: bf16 pools)
};

template <int HD>
__device__ __forceinline__ void norm_rope_lane(float* x, const float* gain, const float* cs, const float* sn,
                                               int rot, float eps, int lane) {
  // x: this lane's HD/32 contiguous elements [lane*EPL, ...)
  constexpr int EPL = HD / 32;
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) ss += x[e] * x[e];
  const float r = rsqrtf(warp_sum(ss) / (float)HD + eps);
#pragma unroll
  for (int e = 0; e < EPL; ++e) x[e] *= r * gain[lane * EPL + e];
  const int half = rot >> 1, plane = half / EPL;  // lanes per half
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const float other = __shfl_xor_sync(0xffffffffu, x[e], plane);
    const int i = lane * EPL + e;
    if (i < rot) {
      const float c = cs[i], s = sn[i];
      x[e] = (i < half) ? x[e] * c - other * s : x[e] * c + other * s;
    }
  }
}

template <int HD>
__global__ void __launch_bounds__(256) attn_prep_kernel(const PrepArgs a) {
  constexpr int EPL = HD / 32;
  griddep_launch();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  const int64_t task = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int per = a.nh + 2 * a.nkv;
  if (task >= (int64_t)a.T * per) return;
  const int t = task / per, hh = task % per;
  const bf16* prow = a.proj + (int64_t)t * a.ldp;
  const int ridx = a.rope_idx ? a.rope_idx[t] : t;
  const float* cs = a.cos + (int64_t)ridx * a.rot;
  const float* sn = a.sin + (int64_t)ridx * a.rot;
  float x[EPL];
  if (hh < a.nh) {
    const bf16* src = prow + (int64_t)hh * 2 * HD + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) x[e] = __bfloat162float(src[e]);
    norm_rope_lane<HD>(x, a.qg, cs, sn, a.rot, a.eps, lane);
    bf16* dst = a.q_out + ((int64_t)t * a.nh + hh) * HD + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) dst[e] = __float2bfloat16(x[e]);
  } else if (hh < a.nh + a.nkv) {
    const int kh = hh - a.nh;
    const bf16* src = prow + (int64_t)a.nh * 2 * HD + (int64_t)kh * HD + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) x[e] = __bfloat162float(src[e]);
    if (a.kv_slot[t] < 0) return;       // padding row of a batched verify: nothing to append
    norm_rope_lane<HD>(x, a.kg, cs, sn, a.rot, a.eps, lane);
    const int64_t krow = (int64_t)a.kv_slot[t] * a.nkv + kh;
    if (a.kscale) {
      const float sc = quant_row_q8<EPL>(x, reinterpret_cast<int8_t*>(a.kpool) + krow * HD, lane);
      if (lane == 0) a.kscale[krow] = sc;
      return;
    }
    bf16* dst = a.kpool + krow * HD + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) dst[e] = __float2bfloat16(x[e]);
  } else {
    const int vh = hh - a.nh - a.nkv;
    if (a.kv_slot[t] < 0) return;
    const bf16* src = prow + (int64_t)a.nh * 2 * HD + (int64_t)(a.nkv + vh) * HD + lane * EPL;
    const int64_t vrow = (int64_t)a.kv_slot[t] * a.nkv + vh;
    if (a.vscale) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) x[e] = __bfloat162float(src[e]);
      const float sc = quant_row_q8<EPL>(x, reinterpret_cast<int8_t*>(a.vpool) + vrow * HD, lane);
      if (lane == 0) a.vscale[vrow] = sc;
      return;
    }
    bf16* dst = a.vpool + vrow * HD + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) dst[e] = src[e];
  }
}

// ------------------------------------------------------------------------------------------
// Prefill flash attention (bf16 mma.m16n8k16, 4 warps x 16 query rows, 64-key tiles).
__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(addr), "l"(gmem));
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

struct PrefillArgs {
  const bf16* q;            // [T, nh, hd]
  const bf16* gate; int64_t ldg;  // gate of head h at gate[t*ldg + h*2*hd + hd + d]
  const bf16* kpool; const bf16* vpool;  // [slots, nkv, hd]
  const int* block_table;   // [nblocks] pool block ids of this sequence
  bf16* out; int64_t ldo;   // [T, nh*hd]
  int T, q_pos0, nh, nkv;
  float scale_log2;         // hd^-0.5 * log2(e)
  int causal;               // 1: key s visible to query position p when s <= p; 0: all kv_len keys (vision)
  int kv_len;               // non-causal: number of valid keys
  // block-selected attention: bit b of keep[t] says whether query t reads the block of (1 << ratio_log2)
  // tokens number b; tokens after a query's last complete block are always read.  null = dense.
  const unsigned* keep; int keep_words, ratio_log2;
  const float* kscale; const float* vscale;   // int8 pools: [slots, nkv] scales (null: bf16 pools)
};

template <int HD>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const PrefillArgs a) {
  constexpr int LD = HD + 8;  // padded row (bf16 elements): 16-byte odd multiple -> conflict-free ldmatrix
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);  // [64][LD]
  bf16* Ks = Qs + 64 * LD;
  bf16* Vs = Ks + 64 * LD;
  griddep_launch();
  griddep_wait();
  const int qt = blockIdx.x, h = blockIdx.y, kvh = h / (a.nh / a.nkv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3;
  constexpr int CPR = HD / 8;  // 16-byte chunks per row
  for (int idx = tid; idx < 64 * CPR; idx += 128) {
    const int r = idx / CPR, c = idx % CPR;
    const int t = qt * 64 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < a.T) v = *reinterpret_cast<const uint4*>(a.q + ((int64_t)t * a.nh + h) * HD + c * 8);
    *reinterpret_cast<uint4*>(Qs + r * LD + c * 8) = v;
  }
  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const int qpos_lo = a.q_pos0 + qt * 64 + warp * 16 + g;  // position of row g (row g+8: +8)
  const int last_q = min(a.T - 1, qt * 64 + 63);
  const int kv_end = a.causal ? a.q_pos0 + last_q + 1 : a.kv_len;   // keys visible to this tile: [0, kv_end)
  const int ntiles = (kv_end + kBlock - 1) / kBlock;

  for (int kt = 0; kt < ntiles; ++kt) {
    __syncthreads();  // previous tile fully consumed (also orders the Q store before first use)
    const int64_t slot0 = (int64_t)a.block_table[kt] * kBlock;
    load_kv_tile<HD, 128>(Ks, Vs, LD, a.kpool, a.vpool, a.kscale, a.vscale, slot0, a.nkv, kvh, tid);
    __syncthreads();
    // ---- S = Q K^T (16 x 64 per warp) --------------------------------------------------
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll 4
    for (int kk = 0; kk < HD / 16; ++kk) {
      uint32_t af[4];
      ldsm_x4(af[0], af[1], af[2], af[3], Qs + (warp * 16 + (lane & 15)) * LD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3, Ks + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * np], af, b0, b1);
        mma_bf16(s[2 * np + 1], af, b2, b3);
      }
    }
    // ---- mask + online softmax (base-2) --------------------------------------------------
    float mnew[2] = {mrow[0], mrow[1]};
    unsigned kbits[2] = {0xffffffffu, 0xffffffffu};
    if (a.keep) {
      const int fb = kt * (kBlock >> a.ratio_log2);          // first block of this tile
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int t = qt * 64 + warp * 16 + g + hh * 8;
        kbits[hh] = t < a.T ? a.keep[(int64_t)t * a.keep_words + (fb >> 5)] >> (fb & 31) : 0u;
      }
    }
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kt * kBlock + n * 8 + tq * 2 + (e & 1);
        const int qp = qpos_lo + ((e >> 1) << 3);
        bool vis = a.causal ? (key <= qp) : (key < a.kv_len);
        if (a.keep) {
          const int tail0 = ((qp + 1) >> a.ratio_log2) << a.ratio_log2;
          vis = vis && (key >= tail0 || ((kbits[e >> 1] >> ((n * 8 + tq * 2 + (e & 1)) >> a.ratio_log2)) & 1u));
        }
        const float v = vis ? s[n][e] * a.scale_log2 : -INFINITY;
        s[n][e] = v;
        mnew[e >> 1] = fmaxf(mnew[e >> 1], v);
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mnew[r] = fmaxf(mnew[r], __shfl_xor_sync(0xffffffffu, mnew[r], 1));
      mnew[r] = fmaxf(mnew[r], __shfl_xor_sync(0xffffffffu, mnew[r], 2));
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      msafe[r] = (mnew[r] == -INFINITY) ? 0.f : mnew[r];
      corr[r] = exp2f(mrow[r] - msafe[r]);  // mrow = -inf -> 0
      mrow[r] = mnew[r];
    }
    float lsum[2] = {0.f, 0.f};
    uint32_t pf[4][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float p0 = exp2f(s[n][0] - msafe[0]), p1 = exp2f(s[n][1] - msafe[0]);
      const float p2 = exp2f(s[n][2] - msafe[1]), p3 = exp2f(s[n][3] - msafe[1]);
      lsum[0] += p0 + p1;
      lsum[1] += p2 + p3;
      pf[n >> 1][(n & 1) * 2] = pack_bf162(p0, p1);
      pf[n >> 1][(n & 1) * 2 + 1] = pack_bf162(p2, p3);
    }
    lrow[0] = lrow[0] * corr[0] + lsum[0];
    lrow[1] = lrow[1] * corr[1] + lsum[1];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
    // ---- O += P V ----------------------------------------------------------------------------
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int np = 0; np < HD / 16; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(b0, b1, b2, b3, Vs + (kk * 16 + (lane & 15)) * LD + np * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * np], pf[kk], b0, b1);
        mma_bf16(o[2 * np + 1], pf[kk], b2, b3);
      }
    }
  }
  // ---- epilogue: normalise, gate, store ---------------------------------------------------
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int t = qt * 64 + warp * 16 + g + r * 8;
    if (t >= a.T) continue;
    const float inv = lrow[r] > 0.f ? 1.f / lrow[r] : 0.f;
    const bf16* gp = a.gate ? a.gate + (int64_t)t * a.ldg + (int64_t)h * 2 * HD + HD : nullptr;
    bf16* op = a.out + (int64_t)t * a.ldo + (int64_t)h * HD;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      const int d = n * 8 + tq * 2;
      const float g0 = gp ? sigmoid_f(__bfloat162float(gp[d])) : 1.f, g1 = gp ? sigmoid_f(__bfloat162float(gp[d + 1])) : 1.f;
      *reinterpret_cast<uint32_t*>(op + d) = pack_bf162(o[n][r * 2] * inv * g0, o[n][r * 2 + 1] * inv * g1);
    }
  }
}

// ------------------------------------------------------------------------------------------
// Decode: one query per row, split over strided key tiles.
struct DecodeArgs {
  const bf16* proj; int64_t ldp;      // [M, ldp] fused q|gate, k, v projection of this token
  const float* qg; const float* kg;   // norm gains
  const float* cos; const float* sin; // [max_pos, rot] tables
  const int* positions;               // [M] token index (KV slot index / causal bound)
  const int* rope_pos;                // [M] rotary position (token index + rope delta)
  const int* block_table; int64_t ldbt;  // [M, ldbt]
  bf16* kpool; bf16* vpool;
  float* part_o;                      // [M, nh, nsplit, hd]
  float* part_ml;                     // [M, nh, nsplit, 2]
  int nh, nkv, rot, nsplit;
  float scale_log2, eps;
  unsigned* tickets;                  // [M, nkv] arrival counters (zero between launches)
  bf16* out; int64_t ldo;             // [M, nh*hd] gated output, written by the last split to arrive
  // sparse mode (block-selected attention): queries come normed and rotated from q_in, K/V of the
  // current token are already in the pool, and row m attends to the blocks sel[m, 0..nsel[m]) of
  // `ratio` tokens plus the tokens after its last complete block (nsel[m] < 0: every visible token)
  const bf16* q_in; const int* sel; const int* nsel; int topk, ratio;
  float* kscale; float* vscale;       // int8 pools: [slots, nkv] scales (null: bf16 pools)
};

constexpr int kDecWarps = 8;          // warps per decode CTA; each takes 4 keys per iteration
constexpr int kDecKeys = 4;

// EPL bf16 channels of one lane as packed 32-bit words (kept packed while in flight: half the registers)
template <int EPL>
__device__ __forceinline__ void dec_load(const bf16* p, uint32_t* w) {
  if (EPL == 8) {
    const uint4 v = ld_stream(p);
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  } else {
#pragma unroll
    for (int e = 0; e < EPL / 2; ++e) w[e] = reinterpret_cast<const uint32_t*>(p)[e];
  }
}
// EPL int8 channels of one lane times the key's scale, as the same packed bf16 words
template <int EPL>
__device__ __forceinline__ void dec_load_q8(const int8_t* p, float sc, uint32_t* w) {
  if (EPL == 8) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const uint4 b = q8x8_to_bf16x8(v, sc);
    w[0] = b.x; w[1] = b.y; w[2] = b.z; w[3] = b.w;
  } else {
#pragma unroll
    for (int e = 0; e < EPL / 2; ++e) w[e] = pack_bf162((float)p[2 * e] * sc, (float)p[2 * e + 1] * sc);
  }
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Split-KV decode attention for one (kv head, split, batch row).  Eight warps walk the split's keys
// four at a time each, with the next four keys' K and V rows already requested while the current
// ones are scored, so that a CTA keeps ~16 KB in flight; lanes own HD/32 consecutive channels.  The
// warps merge pairwise through shared memory, the CTA writes one partial (o, m, l) per query head,
// and the last split of the (row, kv head) group to arrive merges all partials with every thread
// owning four channels of one head (independent float4 loads, scales staged in shared memory),
// applies the sigmoid gate and writes the bf16 output.
// MINB = 2 compiles the same kernel for two resident CTAs per SM (128 registers): a batch of rows
// launches far more CTAs than SMs, and throughput then wants residency more than the last register.
template <int HD, int REP, bool SPARSE, int MINB = 1>
__global__ void __launch_bounds__(kDecWarps * 32, MINB) attn_decode_kernel(const DecodeArgs a) {
  constexpr int EPL = HD / 32;
  constexpr int NT = kDecWarps * 32;
  __shared__ float q_s[REP][HD];
  __shared__ __align__(16) float mo[kDecWarps / 2][REP][HD];
  __shared__ float mml[kDecWarps / 2][REP][2];
  __shared__ float sc_s[REP][64];                 // per-split scales of the final merge (nsplit <= 64)
  __shared__ float l_s[REP][64];
  __shared__ float linv_s[REP];
  const int kvh = blockIdx.x, split = blockIdx.y, m = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  griddep_launch();
  griddep_wait();
  const int pos = a.positions[m];
  float* po = a.part_o + (((int64_t)m * a.nh + kvh * REP) * a.nsplit + split) * HD;
  float* pml = a.part_ml + (((int64_t)m * a.nh + kvh * REP) * a.nsplit + split) * 2;
  if (pos < 0) {  // padded row
    for (int i = tid; i < REP * 2; i += NT) pml[(int64_t)(i >> 1) * a.nsplit * 2 + (i & 1)] = (i & 1) ? 0.f : -INFINITY;
    return;
  }
  const bf16* prow = a.proj + (int64_t)m * a.ldp;
  const int rp = SPARSE ? 0 : a.rope_pos[m];
  const float* cs = a.cos + (int64_t)rp * a.rot;
  const float* sn = a.sin + (int64_t)rp * a.rot;
  const int* bt = a.block_table + (int64_t)m * a.ldbt;
  if (SPARSE) {
    for (int i = tid; i < REP * HD; i += NT)
      q_s[i / HD][i % HD] = __bfloat162float(a.q_in[((int64_t)m * a.nh + kvh * REP) * HD + i]) * a.scale_log2;
  } else {
    // q heads of this kv group: norm + rope -> shared (pre-scaled for base-2 softmax)
    for (int r = warp; r < REP; r += kDecWarps) {
      float x[EPL];
      const bf16* src = prow + (int64_t)(kvh * REP + r) * 2 * HD + lane * EPL;
#pragma unroll
      for (int e = 0; e < EPL; ++e) x[e] = __bfloat162float(src[e]);
      norm_rope_lane<HD>(x, a.qg, cs, sn, a.rot, a.eps, lane);
#pragma unroll
      for (int e = 0; e < EPL; ++e) q_s[r][lane * EPL + e] = x[e] * a.scale_log2;
    }
    // the split that owns the tile holding `pos` appends this token's K/V first
    if ((pos / kBlock) % a.nsplit == split) {
      const int64_t slot = (int64_t)bt[pos / kBlock] * kBlock + pos % kBlock;
      if (warp == kDecWarps - 1) {
        float x[EPL];
        const bf16* src = prow + (int64_t)a.nh * 2 * HD + (int64_t)kvh * HD + lane * EPL;
#pragma unroll
        for (int e = 0; e < EPL; ++e) x[e] = __bfloat162float(src[e]);
        norm_rope_lane<HD>(x, a.kg, cs, sn, a.rot, a.eps, lane);
        if (a.kscale) {
          const float sc = quant_row_q8<EPL>(x, reinterpret_cast<int8_t*>(a.kpool) + (slot * a.nkv + kvh) * HD, lane);
          if (lane == 0) a.kscale[slot * a.nkv + kvh] = sc;
        } else {
          bf16* dst = a.kpool + (slot * a.nkv + kvh) * HD + lane * EPL;
#pragma unroll
          for (int e = 0; e < EPL; ++e) dst[e] = __float2bfloat16(x[e]);
        }
      } else if (warp == kDecWarps - 2) {
        const bf16* src = prow + (int64_t)a.nh * 2 * HD + (int64_t)(a.nkv + kvh) * HD + lane * EPL;
        if (a.vscale) {
          float x[EPL];
#pragma unroll
          for (int e = 0; e < EPL; ++e) x[e] = __bfloat162float(src[e]);
          const float sc = quant_row_q8<EPL>(x, reinterpret_cast<int8_t*>(a.vpool) + (slot * a.nkv + kvh) * HD, lane);
          if (lane == 0) a.vscale[slot * a.nkv + kvh] = sc;
        } else {
          bf16* dst = a.vpool + (slot * a.nkv + kvh) * HD + lane * EPL;
#pragma unroll
          for (int e = 0; e < EPL; ++e) dst[e] = src[e];
        }
      }
      __threadfence_block();
    }
  }
  __syncthreads();
  float q[REP][EPL], o[REP][EPL], mx[REP], l[REP];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    mx[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) { q[r][e] = q_s[r][lane * EPL + e]; o[r][e] = 0.f; }
  }
  // keys of this split, numbered j.  Dense: j = local tile * 64 + offset, tiles strided over the
  // splits.  Sparse: the row's kept tokens (selected blocks, then the ragged tail) form one virtual
  // list that the splits cut into equal contiguous pieces.
  const int ntiles = pos / kBlock + 1;
  int nj, j_base = 0, n_sel = 0, tail0 = 0;
  if (SPARSE) {
    n_sel = a.nsel[m];
    const int nb = (pos + 1) / a.ratio;
    tail0 = nb * a.ratio;
    const int total = n_sel < 0 ? pos + 1 : n_sel * a.ratio + (pos + 1 - tail0);
    int chunk = (total + a.nsplit - 1) / a.nsplit;
    chunk = (chunk + kDecWarps * kDecKeys - 1) / (kDecWarps * kDecKeys) * (kDecWarps * kDecKeys);
    j_base = split * chunk;
    nj = max(0, min(chunk, total - j_base));
  } else {
    const int nloc = split < ntiles ? (ntiles - 1 - split) / a.nsplit + 1 : 0;
    nj = nloc * kBlock;
  }
  auto key_row = [&](int j, bool& ok) -> int64_t {
    if (SPARSE) {
      ok = j < nj;
      if (!ok) return 0;
      const int jj = j_base + j;
      int tok;
      if (n_sel < 0) tok = jj;
      else if (jj < n_sel * a.ratio) tok = a.sel[(int64_t)m * a.topk + jj / a.ratio] * a.ratio + jj % a.ratio;
      else tok = tail0 + (jj - n_sel * a.ratio);
      return ((int64_t)bt[tok / kBlock] * kBlock + tok % kBlock) * a.nkv + kvh;
    }
    const int kt = split + (j / kBlock) * a.nsplit;
    const int i = j % kBlock;
    ok = j < nj && kt * kBlock + i <= pos;
    return ok ? ((int64_t)bt[kt] * kBlock + i) * a.nkv + kvh : 0;
  };
  constexpr int WPL = EPL / 2;
  uint32_t kfa[kDecKeys][WPL], vfa[kDecKeys][WPL], kfb[kDecKeys][WPL], vfb[kDecKeys][WPL];
  bool oka[kDecKeys], okb[kDecKeys];
  auto fetch = [&](int it, uint32_t (&kf)[kDecKeys][WPL], uint32_t (&vf)[kDecKeys][WPL], bool (&okk)[kDecKeys]) {
#pragma unroll
    for (int u = 0; u < kDecKeys; ++u) {
      const int64_t row = key_row(it * (kDecWarps * kDecKeys) + warp * kDecKeys + u, okk[u]);
      if (okk[u]) {
        if (a.kscale) {
          dec_load_q8<EPL>(reinterpret_cast<const int8_t*>(a.kpool) + row * HD + lane * EPL, a.kscale[row], kf[u]);
          dec_load_q8<EPL>(reinterpret_cast<const int8_t*>(a.vpool) + row * HD + lane * EPL, a.vscale[row], vf[u]);
        } else {
          dec_load<EPL>(a.kpool + row * HD + lane * EPL, kf[u]);
          dec_load<EPL>(a.vpool + row * HD + lane * EPL, vf[u]);
        }
      }
    }
  };
  auto score = [&](const uint32_t (&kf)[kDecKeys][WPL], const uint32_t (&vf)[kDecKeys][WPL], const bool (&okk)[kDecKeys]) {
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      float d[kDecKeys];
#pragma unroll
      for (int u = 0; u < kDecKeys; ++u) {
        float sdot = 0.f;
        if (okk[u]) {
#pragma unroll
          for (int e = 0; e < WPL; ++e) {
            sdot = fmaf(q[r][2 * e], bf_lo(kf[u][e]), sdot);
            sdot = fmaf(q[r][2 * e + 1], bf_hi(kf[u][e]), sdot);
          }
        }
        d[u] = sdot;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int u = 0; u < kDecKeys; ++u) d[u] += __shfl_xor_sync(0xffffffffu, d[u], off);
      }
      float mn = mx[r];
#pragma unroll
      for (int u = 0; u < kDecKeys; ++u) {
        if (!okk[u]) d[u] = -INFINITY;
        mn = fmaxf(mn, d[u]);
      }
      if (mn == -INFINITY) continue;
      const float c = exp2f(mx[r] - mn);
      float p[kDecKeys], ps = 0.f;
#pragma unroll
      for (int u = 0; u < kDecKeys; ++u) { p[u] = exp2f(d[u] - mn); ps += p[u]; }
      l[r] = l[r] * c + ps;
      mx[r] = mn;
#pragma unroll
      for (int e = 0; e < WPL; ++e) {
        float a0 = o[r][2 * e] * c, a1 = o[r][2 * e + 1] * c;
#pragma unroll
        for (int u = 0; u < kDecKeys; ++u)
          if (okk[u]) { a0 = fmaf(p[u], bf_lo(vf[u][e]), a0); a1 = fmaf(p[u], bf_hi(vf[u][e]), a1); }
        o[r][2 * e] = a0; o[r][2 * e + 1] = a1;
      }
    }
  };
  // two register buffers, named (not indexed) so that they stay in registers
  const int niter = (nj + kDecWarps * kDecKeys - 1) / (kDecWarps * kDecKeys);
  if (niter > 0) fetch(0, kfa, vfa, oka);
  for (int it = 0; it < niter; it += 2) {
    if (it + 1 < niter) fetch(it + 1, kfb, vfb, okb);
    score(kfa, vfa, oka);
    if (it + 1 >= niter) break;
    if (it + 2 < niter) fetch(it + 2, kfa, vfa, oka);
    score(kfb, vfb, okb);
  }
  // ---- merge the warps pairwise through shared memory -------------------------------------------
#pragma unroll
  for (int step = kDecWarps / 2; step > 0; step >>= 1) {
    if (warp >= step && warp < 2 * step) {
#pragma unroll
      for (int r = 0; r < REP; ++r) {
#pragma unroll
        for (int e = 0; e < EPL; ++e) mo[warp - step][r][lane * EPL + e] = o[r][e];
        if (lane == 0) { mml[warp - step][r][0] = mx[r]; mml[warp - step][r][1] = l[r]; }
      }
    }
    __syncthreads();
    if (warp < step) {
#pragma unroll
      for (int r = 0; r < REP; ++r) {
        const float m2 = mml[warp][r][0], l2 = mml[warp][r][1];
        const float mn = fmaxf(mx[r], m2);
        const float c1 = mn == -INFINITY ? 0.f : exp2f(mx[r] - mn);
        const float c2 = mn == -INFINITY ? 0.f : exp2f(m2 - mn);
#pragma unroll
        for (int e = 0; e < EPL; ++e) o[r][e] = o[r][e] * c1 + mo[warp][r][lane * EPL + e] * c2;
        l[r] = l[r] * c1 + l2 * c2;
        mx[r] = mn;
      }
    }
    __syncthreads();
  }
  if (warp == 0) {
#pragma unroll
    for (int r = 0; r < REP; ++r) {
#pragma unroll
      for (int e = 0; e < EPL; ++e) po[(int64_t)r * a.nsplit * HD + lane * EPL + e] = o[r][e];
      if (lane == 0) {
        pml[(int64_t)r * a.nsplit * 2] = mx[r];
        pml[(int64_t)r * a.nsplit * 2 + 1] = l[r];
      }
    }
  }
  // ---- the last split of this (row, kv head) to arrive merges all splits and applies the gate ----
  __shared__ bool is_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    unsigned* tk = a.tickets + (int64_t)m * a.nkv + kvh;
    is_last = atomicAdd(tk, 1u) == (unsigned)a.nsplit - 1;
    if (is_last) *tk = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const float* bo = a.part_o + ((int64_t)m * a.nh + kvh * REP) * a.nsplit * HD;
  const float* bml = a.part_ml + ((int64_t)m * a.nh + kvh * REP) * a.nsplit * 2;
  const int ns = a.nsplit;
  for (int i = tid; i < REP * ns; i += NT) {                       // (m, l) of every (head, split): one parallel pass
    sc_s[i / ns][i % ns] = __ldcg(bml + (int64_t)i * 2);
    l_s[i / ns][i % ns] = __ldcg(bml + (int64_t)i * 2 + 1);
  }
  __syncthreads();
  if (warp < REP) {                                               // one warp per head: max, scales, 1 / l
    const int r = warp;
    float Mx = -INFINITY;
    for (int sp = lane; sp < ns; sp += 32) Mx = fmaxf(Mx, sc_s[r][sp]);
    Mx = warp_max(Mx);
    float L = 0.f;
    for (int sp = lane; sp < ns; sp += 32) {
      const float c = Mx == -INFINITY ? 0.f : exp2f(sc_s[r][sp] - Mx);
      sc_s[r][sp] = c;
      L += l_s[r][sp] * c;
    }
    L = warp_sum(L);
    if (lane == 0) linv_s[r] = L > 0.f ? 1.f / L : 0.f;
  }
  __syncthreads();
  for (int idx = tid; idx < REP * (HD / 4); idx += NT) {
    const int r = idx / (HD / 4), d = (idx % (HD / 4)) * 4;
    const float* src = bo + (int64_t)r * ns * HD + d;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int sp = 0; sp < ns; ++sp) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (int64_t)sp * HD));
      const float c = sc_s[r][sp];
      acc.x = fmaf(v.x, c, acc.x); acc.y = fmaf(v.y, c, acc.y); acc.z = fmaf(v.z, c, acc.z); acc.w = fmaf(v.w, c, acc.w);
    }
    const int h = kvh * REP + r;
    const bf16* gp = prow + (int64_t)h * 2 * HD + HD + d;
    const float li = linv_s[r];
    bf16* dst = a.out + (int64_t)m * a.ldo + (int64_t)h * HD + d;
    dst[0] = __float2bfloat16(acc.x * li * sigmoid_f(__bfloat162float(gp[0])));
    dst[1] = __float2bfloat16(acc.y * li * sigmoid_f(__bfloat162float(gp[1])));
    dst[2] = __float2bfloat16(acc.z * li * sigmoid_f(__bfloat162float(gp[2])));
    dst[3] = __float2bfloat16(acc.w * li * sigmoid_f(__bfloat162float(gp[3])));
  }
}

// ------------------------------------------------------------------------------------------
// Decode attention for a batch of rows on the tensor cores.  The kernel above is built for the
// latency of one sequence (many key splits, scalar dot products with warp shuffles) and becomes issue
// bound when every row brings its own CTAs.  Here one CTA serves one (row, kv head): the REP query
// heads of the kv head are rows 0..REP-1 of a 16-row mma tile (the rest zero), the four warps take 16
// keys each of every 64-key tile (S = Q K^T and O += P V as bf16 mma.m16n8k16 from ldmatrix
// fragments, tiles staged with cp.async), keep their own running maximum and sum, and merge once at
// the end.  Query / key normalisation, rotary embedding, the KV append of the current token and the
// sigmoid output gate are part of the kernel as in the single-sequence one.
template <int HD>
__global__ void __launch_bounds__(128, 2) attn_decode_batch_kernel(const DecodeArgs a) {
  constexpr int LD = HD + 8, EPL = HD / 32, CPR = HD / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);   // [16][LD]
  bf16* Ks = Qs + 16 * LD;                        // [64][LD]
  bf16* Vs = Ks + 64 * LD;                        // [64][LD]
  bf16* kcur = Vs + 64 * LD;                      // [HD] this token's key (normed, rotated)
  bf16* vcur = kcur + HD;                         // [HD]
  float* mo = reinterpret_cast<float*>(Ks);       // after the loop: [4 warps][8 rows][HD] partial outputs
  __shared__ float mm_s[4][8], ml_s[4][8];
  __shared__ float sc_s[8][64], l_s[8][64], linv_s[8];
  __shared__ bool is_last;
  const int kvh = blockIdx.x, m = blockIdx.y, split = blockIdx.z, nsplit = gridDim.z, rep = a.nh / a.nkv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3;
  griddep_launch();
  griddep_wait();
  const int pos = a.positions[m];
  if (pos < 0) return;                            // padded row
  const bf16* prow = a.proj + (int64_t)m * a.ldp;
  const int rp = a.rope_pos[m];
  const float* cs = a.cos + (int64_t)rp * a.rot;
  const float* sn = a.sin + (int64_t)rp * a.rot;
  const int* bt = a.block_table + (int64_t)m * a.ldbt;
  // ---- prologue: q heads -> Qs (bf16), this token's K / V -> pool and shared copies ---------------
  for (int idx = tid; idx < 16 * CPR; idx += 128)
    *reinterpret_cast<uint4*>(Qs + (idx / CPR) * LD + (idx % CPR) * 8) = make_uint4(0, 0, 0, 0);
  __syncthreads();
  for (int r = warp; r < rep + 2; r += 4) {
    float x[EPL];
    if (r < rep) {
      const bf16* src = prow + (int64_t)(kvh * rep + r) * 2 * HD + lane * EPL;
#pragma unroll
      for (int e = 0; e < EPL; ++e) x[e] = __bfloat162float(src[e]);
      norm_rope_lane<HD>(x, a.qg, cs, sn, a.rot, a.eps, lane);
#pragma unroll
      for (int e = 0; e < EPL; ++e) Qs[r * LD + lane * EPL + e] = __float2bfloat16(x[e]);
    } else if ((pos / kBlock) % nsplit == split) {   // the split that owns the last tile appends this token
      const int64_t slot = (int64_t)bt[pos / kBlock] * kBlock + pos % kBlock;
      if (r == rep) {
        const bf16* src = prow + (int64_t)a.nh * 2 * HD + (int64_t)kvh * HD + lane * EPL;
#pragma unroll
        for (int e = 0; e < EPL; ++e) x[e] = __bfloat162float(src[e]);
        norm_rope_lane<HD>(x, a.kg, cs, sn, a.rot, a.eps, lane);
        if (a.kscale) {            // the shared copy holds the dequantised row, what later steps will read
          const float sc = quant_row_q8<EPL>(x, reinterpret_cast<int8_t*>(a.kpool) + (slot * a.nkv + kvh) * HD, lane);
          if (lane == 0) a.kscale[slot * a.nkv + kvh] = sc;
#pragma unroll
          for (int e = 0; e < EPL; ++e) kcur[lane * EPL + e] = __float2bfloat16(x[e]);
        } else {
          bf16* dst = a.kpool + (slot * a.nkv + kvh) * HD + lane * EPL;
#pragma unroll
          for (int e = 0; e < EPL; ++e) { const bf16 v = __float2bfloat16(x[e]); dst[e] = v; kcur[lane * EPL + e] = v; }
        }
      } else {
        const bf16* src = prow + (int64_t)a.nh * 2 * HD + (int64_t)(a.nkv + kvh) * HD + lane * EPL;
        if (a.vscale) {
#pragma unroll
          for (int e = 0; e < EPL; ++e) x[e] = __bfloat162float(src[e]);
          const float sc = quant_row_q8<EPL>(x, reinterpret_cast<int8_t*>(a.vpool) + (slot * a.nkv + kvh) * HD, lane);
          if (lane == 0) a.vscale[slot * a.nkv + kvh] = sc;
#pragma unroll
          for (int e = 0; e < EPL; ++e) vcur[lane * EPL + e] = __float2bfloat16(x[e]);
        } else {
          bf16* dst = a.vpool + (slot * a.nkv + kvh) * HD + lane * EPL;
#pragma unroll
          for (int e = 0; e < EPL; ++e) { dst[e] = src[e]; vcur[lane * EPL + e] = src[e]; }
        }
      }
    }
  }
  float o[HD / 8][2];                             // rows g (< 8) only: rows 8..15 of the tile are padding
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = 0.f;
  float mrow = -INFINITY, lrow = 0.f;
  const int ntiles = pos / kBlock + 1;
  __syncthreads();                                // prologue stores visible (a split may have no tile at all)
  for (int kt = split; kt < ntiles; kt += nsplit) {
    __syncthreads();                              // previous tile consumed
    const int64_t slot0 = (int64_t)bt[kt] * kBlock;
    load_kv_tile<HD, 128>(Ks, Vs, LD, a.kpool, a.vpool, a.kscale, a.vscale, slot0, a.nkv, kvh, tid);
    __syncthreads();
    if (kt == ntiles - 1) {                       // the current token's row comes from this CTA, not from memory
      for (int c = tid; c < 2 * CPR; c += 128) {
        const bool isv = c >= CPR;
        const int cc = isv ? c - CPR : c;
        *reinterpret_cast<uint4*>((isv ? Vs : Ks) + (pos % kBlock) * LD + cc * 8) =
            *reinterpret_cast<const uint4*>((isv ? vcur : kcur) + cc * 8);
      }
      __syncthreads();
    }
    // ---- S = Q K^T for this warp's 16 keys ---------------------------------------------------
    float sc[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll 4
    for (int kk = 0; kk < HD / 16; ++kk) {
      uint32_t af[4], b0, b1, b2, b3;
      ldsm_x4(af[0], af[1], af[2], af[3], Qs + (lane & 15) * LD + kk * 16 + (lane >> 4) * 8);
      ldsm_x4(b0, b1, b2, b3, Ks + (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * LD + kk * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(sc[0], af, b0, b1);
      mma_bf16(sc[1], af, b2, b3);
    }
    // ---- mask + online softmax (base 2), row g of the tile --------------------------------------
    float mnew = mrow;
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = kt * kBlock + warp * 16 + n * 8 + tq * 2 + e;
        const float v = key <= pos ? sc[n][e] * a.scale_log2 : -INFINITY;
        sc[n][e] = v;
        mnew = fmaxf(mnew, v);
      }
    mnew = fmaxf(mnew, __shfl_xor_sync(0xffffffffu, mnew, 1));
    mnew = fmaxf(mnew, __shfl_xor_sync(0xffffffffu, mnew, 2));
    const float msafe = (mnew == -INFINITY) ? 0.f : mnew;
    const float corr = exp2f(mrow - msafe);
    mrow = mnew;
    const float p0 = exp2f(sc[0][0] - msafe), p1 = exp2f(sc[0][1] - msafe);
    const float p2 = exp2f(sc[1][0] - msafe), p3 = exp2f(sc[1][1] - msafe);
    lrow = lrow * corr + p0 + p1 + p2 + p3;
    uint32_t pf[4];
    pf[0] = pack_bf162(p0, p1);
    pf[1] = 0u;                                   // rows 8..15
    pf[2] = pack_bf162(p2, p3);
    pf[3] = 0u;
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) { o[n][0] *= corr; o[n][1] *= corr; }
    // ---- O += P V for the same 16 keys -------------------------------------------------------------
#pragma unroll
    for (int np = 0; np < HD / 16; ++np) {
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(b0, b1, b2, b3, Vs + (warp * 16 + (lane & 15)) * LD + np * 16 + (lane >> 4) * 8);
      float c0[4] = {o[2 * np][0], o[2 * np][1], 0.f, 0.f}, c1[4] = {o[2 * np + 1][0], o[2 * np + 1][1], 0.f, 0.f};
      mma_bf16(c0, pf, b0, b1);
      mma_bf16(c1, pf, b2, b3);
      o[2 * np][0] = c0[0]; o[2 * np][1] = c0[1];
      o[2 * np + 1][0] = c1[0]; o[2 * np + 1][1] = c1[1];
    }
  }
  // ---- merge the four warps, normalise, gate, store -----------------------------------------------------
  lrow += __shfl_xor_sync(0xffffffffu, lrow, 1);
  lrow += __shfl_xor_sync(0xffffffffu, lrow, 2);
  __syncthreads();                                // all warps are done with Ks / Vs
  if (tq == 0) { mm_s[warp][g] = mrow; ml_s[warp][g] = lrow; }
#pragma unroll
  for (int n = 0; n < HD / 8; ++n)
    *reinterpret_cast<float2*>(mo + ((warp * 8 + g) * HD) + n * 8 + tq * 2) = make_float2(o[n][0], o[n][1]);
  __syncthreads();
  for (int idx = tid; idx < rep * (HD / 4); idx += 128) {
    const int r = idx / (HD / 4), d = (idx % (HD / 4)) * 4;
    float M4 = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M4 = fmaxf(M4, mm_s[w][r]);
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float sw = mm_s[w][r] == -INFINITY ? 0.f : exp2f(mm_s[w][r] - M4);
      L += ml_s[w][r] * sw;
      const float4 x = *reinterpret_cast<const float4*>(mo + (w * 8 + r) * HD + d);
      acc.x += x.x * sw; acc.y += x.y * sw; acc.z += x.z * sw; acc.w += x.w * sw;
    }
    const int h = kvh * rep + r;
    if (nsplit > 1) {                             // unnormalised partial of this split
      *reinterpret_cast<float4*>(a.part_o + (((int64_t)m * a.nh + h) * nsplit + split) * HD + d) = acc;
      if (d == 0) {
        float* pml = a.part_ml + (((int64_t)m * a.nh + h) * nsplit + split) * 2;
        pml[0] = M4;
        pml[1] = L;
      }
      continue;
    }
    const float li = L > 0.f ? 1.f / L : 0.f;
    const bf16* gp = prow + (int64_t)h * 2 * HD + HD + d;
    bf16* dst = a.out + (int64_t)m * a.ldo + (int64_t)h * HD + d;
    dst[0] = __float2bfloat16(acc.x * li * sigmoid_f(__bfloat162float(gp[0])));
    dst[1] = __float2bfloat16(acc.y * li * sigmoid_f(__bfloat162float(gp[1])));
    dst[2] = __float2bfloat16(acc.z * li * sigmoid_f(__bfloat162float(gp[2])));
    dst[3] = __float2bfloat16(acc.w * li * sigmoid_f(__bfloat162float(gp[3])));
  }
  if (nsplit == 1) return;
  // ---- several splits per (row, kv head): the last one to arrive merges all partials and applies the gate ----
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    unsigned* tk = a.tickets + (int64_t)m * a.nkv + kvh;
    is_last = atomicAdd(tk, 1u) == (unsigned)nsplit - 1;
    if (is_last) *tk = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const float* bo = a.part_o + ((int64_t)m * a.nh + kvh * rep) * nsplit * HD;
  const float* bml = a.part_ml + ((int64_t)m * a.nh + kvh * rep) * nsplit * 2;
  for (int i = tid; i < rep * nsplit; i += 128) {
    sc_s[i / nsplit][i % nsplit] = __ldcg(bml + (int64_t)i * 2);
    l_s[i / nsplit][i % nsplit] = __ldcg(bml + (int64_t)i * 2 + 1);
  }
  __syncthreads();
  for (int r = warp; r < rep; r += 4) {           // one warp per head: max, scales, 1 / l
    float Mx = -INFINITY;
    for (int sp = lane; sp < nsplit; sp += 32) Mx = fmaxf(Mx, sc_s[r][sp]);
    Mx = warp_max(Mx);
    float L = 0.f;
    for (int sp = lane; sp < nsplit; sp += 32) {
      const float c = sc_s[r][sp] == -INFINITY ? 0.f : exp2f(sc_s[r][sp] - Mx);
      sc_s[r][sp] = c;
      L += l_s[r][sp] * c;
    }
    L = warp_sum(L);
    if (lane == 0) linv_s[r] = L > 0.f ? 1.f / L : 0.f;
  }
  __syncthreads();
  for (int idx = tid; idx < rep * (HD / 4); idx += 128) {
    const int r = idx / (HD / 4), d = (idx % (HD / 4)) * 4;
    const float* src = bo + (int64_t)r * nsplit * HD + d;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sp = 0; sp < nsplit; ++sp) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (int64_t)sp * HD));
      const float c = sc_s[r][sp];
      acc.x = fmaf(v.x, c, acc.x); acc.y = fmaf(v.y, c, acc.y); acc.z = fmaf(v.z, c, acc.z); acc.w = fmaf(v.w, c, acc.w);
    }
    const int h = kvh * rep + r;
    const bf16* gp = prow + (int64_t)h * 2 * HD + HD + d;
    const float li = linv_s[r];
    bf16* dst = a.out + (int64_t)m * a.ldo + (int64_t)h * HD + d;
    dst[0] = __float2bfloat16(acc.x * li * sigmoid_f(__bfloat162float(gp[0])));
    dst[1] = __float2bfloat16(acc.y * li * sigmoid_f(__bfloat162float(gp[1])));
    dst[2] = __float2bfloat16(acc.z * li * sigmoid_f(__bfloat162float(gp[2])));
    dst[3] = __float2bfloat16(acc.w * li * sigmoid_f(__bfloat162float(gp[3])));
  }
}

int g_attn_batch_ctas = 32;

template <int HD, int REP>
int launch_decode(const DecodeArgs& a, int M, cudaStream_t st) {
  if (a.sel)
    return (int)cb_launch(attn_decode_kernel<HD, REP, true>, dim3((unsigned)a.nkv, (unsigned)a.nsplit, (unsigned)M),
                          dim3(kDecWarps * 32), 0, st, a);
  if ((int64_t)a.nkv * a.nsplit * M > 2 * 148)
    return (int)cb_launch(attn_decode_kernel<HD, REP, false, 2>, dim3((unsigned)a.nkv, (unsigned)a.nsplit, (unsigned)M),
                          dim3(kDecWarps * 32), 0, st, a);
  return (int)cb_launch(attn_decode_kernel<HD, REP, false>, dim3((unsigned)a.nkv, (unsigned)a.nsplit, (unsigned)M),
                        dim3(kDecWarps * 32), 0, st, a);
}

int decode_dispatch(const DecodeArgs& a, int64_t M, int64_t nh, int64_t nkv, int64_t hd, int64_t rot, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const int rep = (int)(nh / nkv);
  int rc = CB_ERR_SHAPE;
  if (hd == 256 && (rot / 2) % 8 == 0) {
    switch (rep) {
      case 1: rc = launch_decode<256, 1>(a, (int)M, st); break;
      case 2: rc = launch_decode<256, 2>(a, (int)M, st); break;
      case 3: rc = launch_decode<256, 3>(a, (int)M, st); break;
      case 4: rc = launch_decode<256, 4>(a, (int)M, st); break;
      case 6: rc = launch_decode<256, 6>(a, (int)M, st); break;
      case 8: rc = launch_decode<256, 8>(a, (int)M, st); break;
      default: return CB_ERR_SHAPE;
    }
  } else if (hd == 64 && (rot / 2) % 2 == 0) {
    switch (rep) {
      case 1: rc = launch_decode<64, 1>(a, (int)M, st); break;
      case 2: rc = launch_decode<64, 2>(a, (int)M, st); break;
      case 4: rc = launch_decode<64, 4>(a, (int)M, st); break;
      default: return CB_ERR_SHAPE;
    }
  }
  return rc;
}

}  // namespace

CB_EXPORT int cb_attn_prep(const void* proj, int64_t ldp, const void* qg, const void* kg, const void* cos,
                           const void* sin, const void* rope_idx, const void* kv_slot, void* q_out,
                           void* kpool, void* vpool, int64_t T, int64_t nh, int64_t nkv, int64_t hd,
                           int64_t rot, float eps, void* kscale, void* vscale, void* stream) {
  if (T == 0) return 0;
  if ((kscale == nullptr) != (vscale == nullptr)) return CB_ERR_ARG;
  PrepArgs a{(const bf16*)proj, ldp, (const float*)qg, (const float*)kg, (const float*)cos, (const float*)sin,
             (const int*)rope_idx, (const int*)kv_slot, (bf16*)q_out, (bf16*)kpool, (bf16*)vpool,
             (int)T, (int)nh, (int)nkv, (int)rot, eps, (float*)kscale, (float*)vscale};
  const int64_t tasks = T * (nh + 2 * nkv);
  dim3 grid((unsigned)((tasks + 7) / 8));
  if (hd == 256 && (rot / 2) % 8 == 0) return (int)cb_launch(attn_prep_kernel<256>, grid, dim3(256), 0, (cudaStream_t)stream, a);
  if (hd == 64 && (rot / 2) % 2 == 0) return (int)cb_launch(attn_prep_kernel<64>, grid, dim3(256), 0, (cudaStream_t)stream, a);
  return CB_ERR_SHAPE;
}

CB_EXPORT int cb_attn_prefill(const void* q, const void* gate, int64_t ldg, const void* kpool, const void* vpool,
                              const void* block_table, void* out, int64_t ldo, int64_t T, int64_t q_pos0,
                              int64_t nh, int64_t nkv, int64_t hd, int64_t causal, int64_t kv_len,
                              const void* keep, int64_t keep_words, int64_t ratio, const void* kscale,
                              const void* vscale, void* stream) {
  if (T == 0) return 0;
  if ((kscale == nullptr) != (vscale == nullptr)) return CB_ERR_ARG;
  int rl = 0;
  if (keep) {
    while ((1 << rl) < ratio) ++rl;
    if ((1 << rl) != ratio || ratio < 2 || ratio > kBlock) return CB_ERR_SHAPE;
  }
  PrefillArgs a{(const bf16*)q, (const bf16*)gate, ldg, (const bf16*)kpool, (const bf16*)vpool,
                (const int*)block_table, (bf16*)out, ldo, (int)T, (int)q_pos0, (int)nh, (int)nkv,
                1.4426950408889634f / sqrtf((float)hd), (int)causal, (int)kv_len,
                (const unsigned*)keep, (int)keep_words, rl, (const float*)kscale, (const float*)vscale};
  dim3 grid((unsigned)((T + 63) / 64), (unsigned)nh);
  const size_t smem = (size_t)3 * 64 * (hd + 8) * sizeof(bf16);
  cudaError_t e;
  if (hd == 256) {
    e = cudaFuncSetAttribute(attn_prefill_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return (int)cb_launch(attn_prefill_kernel<256>, grid, dim3(128), smem, (cudaStream_t)stream, a);
  }
  if (hd == 64) return (int)cb_launch(attn_prefill_kernel<64>, grid, dim3(128), smem, (cudaStream_t)stream, a);
  return CB_ERR_SHAPE;
}

CB_EXPORT int cb_attn_decode(const void* proj, int64_t ldp, const void* qg, const void* kg, const void* cos,
                             const void* sin, const void* positions, const void* rope_pos,
                             const void* block_table, int64_t ldbt, void* kpool, void* vpool, void* part_o,
                             void* part_ml, void* tickets, void* out, int64_t ldo, int64_t M, int64_t nh, int64_t nkv,
                             int64_t hd, int64_t rot, int64_t nsplit, float eps, void* kscale, void* vscale,
                             void* stream) {
  if (M == 0) return 0;
  if (nh % nkv || nsplit < 1 || nsplit > 64 || !tickets) return CB_ERR_SHAPE;
  if ((kscale == nullptr) != (vscale == nullptr)) return CB_ERR_ARG;
  DecodeArgs a{(const bf16*)proj, ldp, (const float*)qg, (const float*)kg, (const float*)cos, (const float*)sin,
               (const int*)positions, (const int*)rope_pos, (const int*)block_table, ldbt, (bf16*)kpool,
               (bf16*)vpool, (float*)part_o, (float*)part_ml, (int)nh, (int)nkv, (int)rot, (int)nsplit,
               1.4426950408889634f / sqrtf((float)hd), eps, (unsigned*)tickets, (bf16*)out, ldo,
               nullptr, nullptr, nullptr, 0, 1, (float*)kscale, (float*)vscale};
  if (hd == 256 && (rot / 2) % 8 == 0 && nh / nkv <= 8 && g_attn_batch_ctas > 0 && nkv * M >= g_attn_batch_ctas) {
    // enough (row, kv head) pairs to fill the machine with one CTA each: tensor-core batch kernel
    constexpr int HD = 256;
    const size_t smem = (size_t)(16 + 64 + 64) * (HD + 8) * sizeof(bf16) + 2 * HD * sizeof(bf16);
    cudaError_t e = cudaFuncSetAttribute(attn_decode_batch_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    return (int)cb_launch(attn_decode_batch_kernel<HD>, dim3((unsigned)nkv, (unsigned)M, (unsigned)nsplit), dim3(128), smem,
                          (cudaStream_t)stream, a);
  }
  return decode_dispatch(a, M, nh, nkv, hd, rot, stream);
}

// Number of (row, kv head) pairs from which the dense decode uses the batch kernel (0: never).
CB_EXPORT int cb_set_attn_batch_ctas(int64_t n) { g_attn_batch_ctas = (int)n; return 0; }

// Block-selected ("QSA") decode attention: q [M, nh, hd] is normed and rotated, this step's K/V are in
// the pool already; row m reads blocks sel[m, :nsel[m]] of `ratio` tokens and its ragged tail.
CB_EXPORT int cb_attn_sparse(const void* q, const void* proj, int64_t ldp, const void* positions,
                             const void* block_table, int64_t ldbt, const void* kpool, const void* vpool,
                             const void* sel, const void* nsel, int64_t topk, int64_t ratio, void* part_o,
                             void* part_ml, void* tickets, void* out, int64_t ldo, int64_t M, int64_t nh,
                             int64_t nkv, int64_t hd, int64_t nsplit, void* stream) {
  if (M == 0) return 0;
  if (nh % nkv || nsplit < 1 || nsplit > 64 || !tickets || !sel || !nsel || ratio < 1) return CB_ERR_SHAPE;
  DecodeArgs a{(const bf16*)proj, ldp, nullptr, nullptr, nullptr, nullptr, (const int*)positions, nullptr,
               (const int*)block_table, ldbt, (bf16*)kpool, (bf16*)vpool, (float*)part_o, (float*)part_ml, (int)nh,
               (int)nkv, 0, (int)nsplit, 1.4426950408889634f / sqrtf((float)hd), 0.f, (unsigned*)tickets, (bf16*)out,
               ldo, (const bf16*)q, (const int*)sel, (const int*)nsel, (int)topk, (int)ratio, nullptr, nullptr};
  return decode_dispatch(a, M, nh, nkv, hd, 0, stream);
}
