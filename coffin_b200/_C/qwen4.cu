// Kernels of the Qwen4-exp family that the Qwen3.5 family does not have:
//
//  * hyper-connection read/write (hyper_norm, hyper_up): the residual stream is `hc` lanes of H
//    channels.  hyper_norm applies the pending write-back of the previous mixer (stream += out (x)
//    inject) and the grouped zero-centred RMSNorm in one pass over the stream; the low-rank
//    down-projection is a plain GEMV; hyper_up turns the low-rank vector into the per-channel read
//    gate, folds the gated lanes into the mixer input and computes the per-lane write gate.
//    Reference: grouped_rms_norm / hyper_down / hyper_up of backends/corex/kernels/hyper.cu and the
//    torch chain of models/qwen4exp/gated_residual.py:300-478.
//  * QSA indexer (qsa_index_prep, qsa_block_keys, qsa_select): index queries are normed and
//    rotated, raw index keys are stored in a paged pool next to the KV pool, the key of a block of
//    `ratio` tokens (mean -> norm -> rotary at the block start) is computed once when the block
//    completes and cached in a paged block-key pool, and selection scores all complete blocks
//    (sum over heads of relu(q.k)) and keeps the best `topk` by an exact radix select (ties to the
//    lowest block).  Reference: QSAIndexer.project/block_keys/select,
//    models/qwen4exp/qsa.py:469-723, which recomputes every block key for every query.
//
// The sparse attention itself is a mode of the decode kernel in attn.cu.
#include "common.cuh"

namespace {

constexpr int kBlock = 64;   // tokens per KV page

// ---------------------------------------------------------------------------------------------
// hyper_norm: one CTA per (row, lane).  stream [M, hc*H] bf16 (updated in place when a write-back is
// pending), normed [M, hc*H] bf16.
struct HyperNormArgs {
  bf16* stream; const float* gain;        // gain = 1 + w, [hc*H]
  const bf16* block_out;                  // [M, H] pending mixer output, or null
  const float* inject;                    // [M, hc] its per-lane write gates
  const bf16* add;                        // [M, hc*H] extra term added to the stream first (PLE), or null
  bf16* normed;
  int H, hc;
  float eps;
};

__global__ void __launch_bounds__(256) hyper_norm_kernel(const HyperNormArgs a) {
  __shared__ float red[32];
  griddep_launch();
  griddep_wait();
  const int m = blockIdx.x / a.hc, c = blockIdx.x % a.hc;
  const int64_t base = ((int64_t)m * a.hc + c) * a.H;
  const float w = a.block_out ? a.inject[(int64_t)m * a.hc + c] : 0.f;
  // H <= 8192: each thread keeps its (up to 4) 8-channel vectors in registers between the passes
  float v[4][8];
  float ss = 0.f;
  const int nvec = a.H >> 3;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = threadIdx.x + i * 256;
    if (idx < nvec) {
      bf16x8_to_float(*reinterpret_cast<const uint4*>(a.stream + base + idx * 8), v[i]);
      if (a.add) {
        float t[8];
        bf16x8_to_float(*reinterpret_cast<const uint4*>(a.add + base + idx * 8), t);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = __bfloat162float(__float2bfloat16(v[i][e] + t[e]));
      }
      if (a.block_out) {
        float t[8];
        bf16x8_to_float(*reinterpret_cast<const uint4*>(a.block_out + (int64_t)m * a.H + idx * 8), t);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[i][e] = __bfloat162float(__float2bfloat16(fmaf(t[e], w, v[i][e])));
      }
      if (a.block_out || a.add) *reinterpret_cast<uint4*>(a.stream + base + idx * 8) = float_to_bf16x8(v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / (float)a.H + a.eps);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = threadIdx.x + i * 256;
    if (idx < nvec) {
      const float* g = a.gain + (int64_t)c * a.H + idx * 8;
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = v[i][e] * rstd * g[e];
      *reinterpret_cast<uint4*>(a.normed + base + idx * 8) = float_to_bf16x8(o);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// hyper_up: mixed[m, h] = 1/hc * sum_c sigmoid(act[m, :] . Wu[c*H + h, :]) * normed[m, c*H + h]
// with act = silu(low / hc); the last hc CTAs compute inject[m, c] = 2 sigmoid(normed[m, :] . Wi[c, :] / hc).
struct HyperUpArgs {
  const bf16* normed; const float* low;   // [M, hc*H], [M, R] (raw down-projection)
  const bf16* Wu; const bf16* Wi;         // [hc*H, R], [hc, hc*H] or null
  bf16* mixed; float* inject;             // [M, H], [M, hc]
  int M, H, hc, R;
};

constexpr int kUpMaxRows = 8;

__global__ void __launch_bounds__(256) hyper_up_kernel(const HyperUpArgs a) {
  extern __shared__ float act[];          // [M][R]
  __shared__ float red[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  griddep_launch();
  griddep_wait();
  const int nmix = (a.H + 7) / 8;
  if ((int)blockIdx.x >= nmix) {
    // write gate of lane c
    const int c = blockIdx.x - nmix;
    const int64_t W = (int64_t)a.hc * a.H;
    for (int m = 0; m < a.M; ++m) {
      float s = 0.f;
      for (int64_t i = tid; i < (W >> 3); i += 256) {
        float x[8], wv[8];
        bf16x8_to_float(*reinterpret_cast<const uint4*>(a.normed + m * W + i * 8), x);
        bf16x8_to_float(ld_stream(a.Wi + c * W + i * 8), wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) s = fmaf(x[e], wv[e], s);
      }
      s = block_sum(s, red);
      if (tid == 0) a.inject[(int64_t)m * a.hc + c] = 2.f * sigmoid_f(s / (float)a.hc);
    }
    return;
  }
  for (int i = tid; i < a.M * a.R; i += 256) act[i] = silu_f(a.low[i] / (float)a.hc);
  __syncthreads();
  const int h = blockIdx.x * 8 + warp;
  if (h >= a.H) return;
  float acc[kUpMaxRows];
#pragma unroll
  for (int m = 0; m < kUpMaxRows; ++m) acc[m] = 0.f;
  const int nq = a.R >> 2;                // 4-element (8-byte) chunks of a gate row
  for (int c = 0; c < a.hc; ++c) {
    const bf16* wrow = a.Wu + ((int64_t)c * a.H + h) * a.R;
    float dot[kUpMaxRows];
#pragma unroll
    for (int m = 0; m < kUpMaxRows; ++m) dot[m] = 0.f;
    for (int q = lane; q < nq; q += 32) {
      const uint2 wv = *reinterpret_cast<const uint2*>(wrow + q * 4);
      const float w0 = __uint_as_float(wv.x << 16), w1 = __uint_as_float(wv.x & 0xffff0000u);
      const float w2 = __uint_as_float(wv.y << 16), w3 = __uint_as_float(wv.y & 0xffff0000u);
#pragma unroll
      for (int m = 0; m < kUpMaxRows; ++m)
        if (m < a.M) {
          const float4 x = *reinterpret_cast<const float4*>(act + m * a.R + q * 4);
          dot[m] = fmaf(w0, x.x, fmaf(w1, x.y, fmaf(w2, x.z, fmaf(w3, x.w, dot[m]))));
        }
    }
#pragma unroll
    for (int m = 0; m < kUpMaxRows; ++m)
      if (m < a.M) {
        const float g = sigmoid_f(warp_sum(dot[m]));
        acc[m] = fmaf(g, __bfloat162float(a.normed[((int64_t)m * a.hc + c) * a.H + h]), acc[m]);
      }
  }
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < kUpMaxRows; ++m)
      if (m < a.M) a.mixed[(int64_t)m * a.H + h] = __float2bfloat16(acc[m] / (float)a.hc);
  }
}

// ---------------------------------------------------------------------------------------------
// QSA indexer
struct IndexPrepArgs {
  const bf16* proj; int64_t ldp; int64_t col0;  // index part of a projection row starts at column col0:
                                                // [ni * di] queries then [di] raw key
  const float* qgain;                           // 1 + w of the query norm, [di]
  const float* cos; const float* sin;           // [*, rot] rotary rows
  const int* rope_idx;                          // [T] row of cos/sin per token (null: row t)
  const int* kv_slot;                           // [T] pool row per token (-1: do not store)
  float* iq;                                    // [T, ni, di] normed + rotated queries
  bf16* ipool;                                  // [slots, di] raw index keys
  int T, ni, di, rot;
  float eps;
};

// One warp per (token, query head) and one per (token, raw key).
__global__ void __launch_bounds__(256) qsa_index_prep_kernel(const IndexPrepArgs a) {
  griddep_launch();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  const int64_t task = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int per = a.ni + 1;
  if (task >= (int64_t)a.T * per) return;
  const int t = (int)(task / per), h = (int)(task % per);
  const bf16* src = a.proj + (int64_t)t * a.ldp + a.col0 + (int64_t)h * a.di;
  if (h == a.ni) {
    const int slot = a.kv_slot[t];
    if (slot < 0) return;
    for (int i = lane; i < a.di; i += 32) a.ipool[(int64_t)slot * a.di + i] = src[i];
    return;
  }
  float ss = 0.f;
  for (int i = lane; i < a.di; i += 32) { const float x = __bfloat162float(src[i]); ss += x * x; }
  const float rstd = rsqrtf(warp_sum(ss) / (float)a.di + a.eps);
  const int row = a.rope_idx ? a.rope_idx[t] : t;
  const float* cs = a.cos + (int64_t)row * a.rot;
  const float* sn = a.sin + (int64_t)row * a.rot;
  float* dst = a.iq + ((int64_t)t * a.ni + h) * a.di;
  const int half = a.rot >> 1;
  for (int i = lane; i < a.di; i += 32) {
    const float x = __bfloat162float(src[i]) * rstd * a.qgain[i];
    float y = x;
    if (i < a.rot) {
      const int j = i < half ? i + half : i - half;
      const float xo = __bfloat162float(src[j]) * rstd * a.qgain[j];
      y = x * cs[i] + (i < half ? -xo : xo) * sn[i];
    }
    dst[i] = y;
  }
}

struct BlockKeysArgs {
  const bf16* ipool; float* bkpool;             // [slots, di], [pages * (64 / ratio), di]
  const float* kgain;                           // 1 + w of the key norm
  const float* cos; const float* sin;           // 1-D rotary table [max_pos, rot]
  const int* block_table;                       // pages of the sequence
  int b0, b1, ratio, di, rot;
  float eps;
  // row mode (decode rows inside a CUDA graph): warp w looks at row w of `positions`; if that row's
  // token completes a block (position + 1 a multiple of ratio) it computes that block's key from the
  // row's own block table (row w of block_table, ldbt apart), else it does nothing.  b1 = row count.
  const int* positions; int64_t ldbt;
};

// One warp per block b in [b0, b1): tokens [b * ratio, (b + 1) * ratio) of the sequence.
__global__ void __launch_bounds__(256) qsa_block_keys_kernel(const BlockKeysArgs a) {
  griddep_launch();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  int b = a.b0 + blockIdx.x * 8 + (threadIdx.x >> 5);
  if (b >= a.b1) return;
  const int per_page = kBlock / a.ratio;
  const int* table = a.block_table;
  if (a.positions) {
    const int p = a.positions[b];
    if (p < 0 || (p + 1) % a.ratio) return;       // this row's token does not complete a block
    table += (int64_t)b * a.ldbt;
    b = p / a.ratio;
  }
  const int page = table[b / per_page];
  const int64_t tok0 = (int64_t)page * kBlock + (int64_t)(b % per_page) * a.ratio;
  // di <= 256: up to 8 channels per lane
  float m[8];
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int i = lane + 32 * u;
    m[u] = 0.f;
    if (i < a.di) {
      for (int r = 0; r < a.ratio; ++r) m[u] += __bfloat162float(a.ipool[(tok0 + r) * a.di + i]);
      m[u] = __bfloat162float(__float2bfloat16(m[u] / (float)a.ratio));   // the pooled key is a bf16 tensor
      ss += m[u] * m[u];
    }
  }
  const float rstd = rsqrtf(warp_sum(ss) / (float)a.di + a.eps);
  const float* cs = a.cos + (int64_t)b * a.ratio * a.rot;
  const float* sn = a.sin + (int64_t)b * a.ratio * a.rot;
  const int half = a.rot >> 1;
  float* dst = a.bkpool + ((int64_t)page * per_page + b % per_page) * a.di;
  // rotary partner of channel i is i +- half: both live in other lanes/registers; recompute through shared exchange
  __shared__ float ex[8][256];
  float* e = ex[threadIdx.x >> 5];
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int i = lane + 32 * u;
    if (i < a.di) e[i] = m[u] * rstd * a.kgain[i];
  }
  __syncwarp();
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int i = lane + 32 * u;
    if (i < a.di) {
      float y = e[i];
      if (i < a.rot) {
        const float xo = i < half ? -e[i + half] : e[i - half];
        y = e[i] * cs[i] + xo * sn[i];
      }
      dst[i] = y;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// qsa_select: one CTA per query row.  Writes the kept blocks (ascending) to sel[row, topk] and their
// number to nsel[row]; nsel = -1 means "attend to every visible token".  Optionally also a bit mask
// of the kept blocks (all ones for a full row) for the prefill kernel.
struct SelectArgs {
  const float* iq;                              // [rows, ni, di]
  const float* bkpool; const int* block_table; int64_t ldbt;   // block keys; pages per row's sequence
  const int* positions;                         // [rows] position of the query (visible = pos + 1 tokens)
  const int* row_seq;                           // [rows] which block-table row (null: row r uses table r; ldbt 0: shared)
  float* scores;                                // scratch [rows, max_blocks]
  int* sel; int* nsel;                          // [rows, topk], [rows]
  unsigned* mask; int mask_words;               // optional [rows, mask_words]
  int ni, di, ratio, topk, full_factor, max_blocks;
};

__global__ void __launch_bounds__(256) qsa_select_kernel(const SelectArgs a) {
  __shared__ float q_s[8][256];                 // ni <= 8, di <= 256
  __shared__ unsigned hist[256];
  __shared__ unsigned sh_prefix, sh_need;
  __shared__ unsigned wcount[8];
  griddep_launch();
  griddep_wait();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pos = a.positions[row];
  unsigned* mrow = a.mask ? a.mask + (int64_t)row * a.mask_words : nullptr;
  if (pos < 0) {
    if (tid == 0) a.nsel[row] = 0;
    if (mrow) for (int i = tid; i < a.mask_words; i += 256) mrow[i] = 0u;
    return;
  }
  const int nb = (pos + 1) / a.ratio;
  if (nb <= a.topk || nb <= a.topk * a.full_factor) {
    if (tid == 0) a.nsel[row] = -1;
    if (mrow) for (int i = tid; i < a.mask_words; i += 256) mrow[i] = 0xffffffffu;
    return;
  }
  for (int i = tid; i < a.ni * a.di; i += 256) q_s[i / a.di][i % a.di] = a.iq[(int64_t)row * a.ni * a.di + i];
  __syncthreads();
  const int* bt = a.block_table + (a.row_seq ? a.row_seq[row] : row) * a.ldbt;
  const int per_page = kBlock / a.ratio;
  float* sc = a.scores + (int64_t)row * a.max_blocks;
  const float inv = rsqrtf((float)a.di);
  // scores: one warp per block
  for (int b = warp; b < nb; b += 8) {
    const float* k = a.bkpool + ((int64_t)bt[b / per_page] * per_page + b % per_page) * a.di;
    float kv[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) { const int i = lane + 32 * u; kv[u] = i < a.di ? k[i] : 0.f; }
    float s = 0.f;
    for (int h = 0; h < a.ni; ++h) {
      float d = 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) { const int i = lane + 32 * u; if (i < a.di) d = fmaf(q_s[h][i], kv[u], d); }
      d = warp_sum(d);
      s += fmaxf(d, 0.f);
    }
    if (lane == 0) sc[b] = s * inv;
  }
  __syncthreads();
  // exact k-th largest by radix select over the float bits (scores are >= 0: bit order = value order)
  unsigned prefix = 0, need = (unsigned)a.topk;
  for (int pass = 3; pass >= 0; --pass) {
    hist[tid] = 0;
    __syncthreads();
    const unsigned hi_mask = pass == 3 ? 0u : (0xffffffffu << ((pass + 1) * 8));
    for (int b = tid; b < nb; b += 256) {
      const unsigned u = __float_as_uint(sc[b]);
      if ((u & hi_mask) == (prefix & hi_mask)) atomicAdd(&hist[(u >> (pass * 8)) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned acc = 0;
      int d = 255;
      for (; d > 0; --d) {
        if (acc + hist[d] >= need) break;
        acc += hist[d];
      }
      sh_prefix = prefix | ((unsigned)d << (pass * 8));
      sh_need = need - acc;
    }
    __syncthreads();
    prefix = sh_prefix;
    need = sh_need;
    __syncthreads();
  }
  // prefix = bits of the k-th largest score; `need` of the blocks equal to it are kept, lowest index first
  const unsigned thr = prefix;
  if (mrow) for (int i = tid; i < a.mask_words; i += 256) mrow[i] = 0u;
  __syncthreads();
  unsigned eq_seen = 0, out_base = 0;
  for (int b0 = 0; b0 < nb; b0 += 256) {
    const int b = b0 + tid;
    const unsigned u = b < nb ? __float_as_uint(sc[b]) : 0u;
    const bool gt = b < nb && u > thr, eq = b < nb && u == thr;
    // ordered ranks of the equal-to-threshold entries in this chunk
    const unsigned eq_ballot = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) wcount[warp] = __popc(eq_ballot);
    __syncthreads();
    unsigned eq_before = eq_seen;
    for (int w = 0; w < warp; ++w) eq_before += wcount[w];
    unsigned eq_total = 0;
    for (int w = 0; w < 8; ++w) eq_total += wcount[w];
    eq_before += __popc(eq_ballot & ((1u << lane) - 1u));
    const bool keep = gt || (eq && eq_before < need);
    __syncthreads();
    const unsigned kb = __ballot_sync(0xffffffffu, keep);
    if (lane == 0) wcount[warp] = __popc(kb);
    __syncthreads();
    unsigned before = out_base;
    for (int w = 0; w < warp; ++w) before += wcount[w];
    unsigned total = 0;
    for (int w = 0; w < 8; ++w) total += wcount[w];
    before += __popc(kb & ((1u << lane) - 1u));
    if (keep) {
      a.sel[(int64_t)row * a.topk + before] = b;
      if (mrow) atomicOr(&mrow[b >> 5], 1u << (b & 31));
    }
    eq_seen += eq_total;
    out_base += total;
    __syncthreads();
  }
  if (tid == 0) a.nsel[row] = (int)out_base;
}

}  // namespace

CB_EXPORT int cb_hyper_norm(void* stream_buf, const void* gain, const void* block_out, const void* inject,
                            const void* add, void* normed, int64_t M, int64_t H, int64_t hc, float eps, void* stream) {
  if (M == 0) return 0;
  if (H % 8 || H > 8192 || hc < 1) return CB_ERR_SHAPE;
  HyperNormArgs a{(bf16*)stream_buf, (const float*)gain, (const bf16*)block_out, (const float*)inject,
                  (const bf16*)add, (bf16*)normed, (int)H, (int)hc, eps};
  return (int)cb_launch(hyper_norm_kernel, dim3((unsigned)(M * hc)), dim3(256), 0, (cudaStream_t)stream, a);
}

CB_EXPORT int cb_hyper_up(const void* normed, const void* low, const void* Wu, const void* Wi, void* mixed,
                          void* inject, int64_t M, int64_t H, int64_t hc, int64_t R, void* stream) {
  if (M == 0) return 0;
  if (M > kUpMaxRows || R % 4 || (hc * H) % 8 || M * R * 4 > 48 * 1024) return CB_ERR_SHAPE;
  HyperUpArgs a{(const bf16*)normed, (const float*)low, (const bf16*)Wu, (const bf16*)Wi, (bf16*)mixed,
                (float*)inject, (int)M, (int)H, (int)hc, (int)R};
  const unsigned grid = (unsigned)((H + 7) / 8 + (Wi ? hc : 0));
  return (int)cb_launch(hyper_up_kernel, dim3(grid), dim3(256), (size_t)M * R * sizeof(float), (cudaStream_t)stream, a);
}

CB_EXPORT int cb_qsa_index_prep(const void* proj, int64_t ldp, int64_t col0, const void* qgain, const void* cos,
                                const void* sin, const void* rope_idx, const void* kv_slot, void* iq, void* ipool,
                                int64_t T, int64_t ni, int64_t di, int64_t rot, float eps, void* stream) {
  if (T == 0) return 0;
  if (rot % 2 || rot > di || !kv_slot) return CB_ERR_SHAPE;
  IndexPrepArgs a{(const bf16*)proj, ldp, col0, (const float*)qgain, (const float*)cos, (const float*)sin,
                  (const int*)rope_idx, (const int*)kv_slot, (float*)iq, (bf16*)ipool, (int)T, (int)ni, (int)di,
                  (int)rot, eps};
  const int64_t tasks = T * (ni + 1);
  return (int)cb_launch(qsa_index_prep_kernel, dim3((unsigned)((tasks + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, a);
}

CB_EXPORT int cb_qsa_block_keys(const void* ipool, void* bkpool, const void* kgain, const void* cos, const void* sin,
                                const void* block_table, int64_t b0, int64_t b1, int64_t ratio, int64_t di,
                                int64_t rot, float eps, void* stream) {
  if (b1 <= b0) return 0;
  if (ratio < 1 || kBlock % ratio || di > 256 || rot % 2 || rot > di) return CB_ERR_SHAPE;
  BlockKeysArgs a{(const bf16*)ipool, (float*)bkpool, (const float*)kgain, (const float*)cos, (const float*)sin,
                  (const int*)block_table, (int)b0, (int)b1, (int)ratio, (int)di, (int)rot, eps, nullptr, 0};
  return (int)cb_launch(qsa_block_keys_kernel, dim3((unsigned)((b1 - b0 + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, a);
}
// Row mode: for each of `rows` decode rows, the key of the block that the row's token completes (if any).
// Decided on the device from `positions`, so the call can sit in a CUDA graph.
CB_EXPORT int cb_qsa_block_keys_rows(const void* ipool, void* bkpool, const void* kgain, const void* cos, const void* sin,
                                     const void* block_tables, int64_t ldbt, const void* positions, int64_t rows,
                                     int64_t ratio, int64_t di, int64_t rot, float eps, void* stream) {
  if (rows < 1) return 0;
  if (ratio < 1 || kBlock % ratio || di > 256 || rot % 2 || rot > di || !positions) return CB_ERR_SHAPE;
  BlockKeysArgs a{(const bf16*)ipool, (float*)bkpool, (const float*)kgain, (const float*)cos, (const float*)sin,
                  (const int*)block_tables, 0, (int)rows, (int)ratio, (int)di, (int)rot, eps, (const int*)positions, ldbt};
  return (int)cb_launch(qsa_block_keys_kernel, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, (cudaStream_t)stream, a);
}

CB_EXPORT int cb_qsa_select(const void* iq, const void* bkpool, const void* block_table, int64_t ldbt,
                            const void* positions, const void* row_seq, void* scores, void* sel, void* nsel,
                            void* mask, int64_t mask_words, int64_t rows, int64_t ni, int64_t di, int64_t ratio,
                            int64_t topk, int64_t full_factor, int64_t max_blocks, void* stream) {
  if (rows == 0) return 0;
  if (ni > 8 || di > 256 || kBlock % ratio || topk < 1) return CB_ERR_SHAPE;
  SelectArgs a{(const float*)iq, (const float*)bkpool, (const int*)block_table, ldbt, (const int*)positions,
               (const int*)row_seq, (float*)scores, (int*)sel, (int*)nsel, (unsigned*)mask, (int)mask_words,
               (int)ni, (int)di, (int)ratio, (int)topk, (int)full_factor, (int)max_blocks};
  return (int)cb_launch(qsa_select_kernel, dim3((unsigned)rows), dim3(256), 0, (cudaStream_t)stream, a);
}
