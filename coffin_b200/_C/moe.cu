// Routed mixture-of-experts glue kernels: router (fp32 softmax, top-k, renormalise) and the
// weighted combine of expert outputs with the shared expert.  The expert projections themselves
// run on the grouped tensor-core GEMV (decode, gemv_mma.cu slot mode) or the tcgen05 GEMM (prefill).
// Reference: moe_router_t (backends/corex/kernels/moe_grouped.cu:725-879), the merge kernels
// (moe_grouped_i8.cu:546-640) and shared_gate_scale (moe_epilogue.cu:35-95).
#include <string.h>
#include "tp.cuh"

namespace {

constexpr int kMaxTopK = 32;

// One warp per token. logits [T, ldl] fp32 (first E columns are expert logits).
__global__ void __launch_bounds__(256) moe_router_kernel(const float* __restrict__ logits, int64_t ldl, int E, int top_k,
                                                          int normalize, int* __restrict__ out_idx,
                                                          float* __restrict__ out_w, int T, int e_lo, int e_hi) {
  griddep_launch();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  const int64_t tok = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= T) return;
  const float* row = logits + tok * ldl;
  constexpr int PER = 16;                       // up to 512 experts
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = (lane + 32 * i) < E ? __expf(v[i] - mx) : -1.f;   // probabilities (unnormalised); -1 = taken/invalid
    if (v[i] > 0.f) sum += v[i];
  }
  sum = warp_sum(sum);
  float wsum = 0.f, myw = 0.f;
  int myidx = 0;
  for (int k = 0; k < top_k; ++k) {
    float best = -1.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > best) { best = v[i]; bi = e; }          // ascending e per lane: ties keep the lowest index
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    // the owner lane removes the winner (compare-select keeps v[] in registers)
#pragma unroll
    for (int i = 0; i < PER; ++i) if ((bi & 31) == lane && i == (bi >> 5)) v[i] = -1.f;
    const float p = best / sum;
    wsum += p;
    if (lane == k) { myw = p; myidx = bi; }
  }
  // expert parallel: this rank owns experts [e_lo, e_hi); other slots get index -1 and weight 0
  if (lane < top_k) {
    const bool local = myidx >= e_lo && myidx < e_hi;
    out_idx[tok * top_k + lane] = local ? myidx - e_lo : -1;
    out_w[tok * top_k + lane] = local ? (normalize ? myw / wsum : myw) : 0.f;
  }
}

// out[t, :] = sum_j w[t, j] * y[t * top_k + j, :]  (+ sigmoid(gate_logit[t]) * shared[t, :])
__global__ void __launch_bounds__(256) moe_combine_kernel(const bf16* __restrict__ y, const float* __restrict__ w,
                                                           const bf16* __restrict__ shared, const float* __restrict__ gate_logit,
                                                           int64_t ldg, bf16* __restrict__ out, int64_t H, int top_k, int push_site, const TpComm tp,
                                                           const int* __restrict__ pos) {
  griddep_launch();
  griddep_wait();
  const int64_t t = blockIdx.x;
  const float sg = shared ? sigmoid_f(gate_logit[t * ldg]) : 0.f;
  for (int64_t c = threadIdx.x; c < (H >> 3); c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const float wj = w[t * top_k + j];
      if (wj == 0.f) continue;                    // slot of another rank's expert (its row was never written)
      const int64_t row = pos ? pos[t * top_k + j] : t * top_k + j;   // expert-sorted rows are found through pos
      if (row < 0) continue;
      float f[8];
      bf16x8_to_float(*reinterpret_cast<const uint4*>(y + row * H + c * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(wj, f[i], acc[i]);
    }
    if (shared) {
      float f[8];
      bf16x8_to_float(*reinterpret_cast<const uint4*>(shared + t * H + c * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = fmaf(sg, f[i], acc[i]);
    }
    if (push_site >= 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) tp_push_value(tp, push_site, t * H + c * 8 + i, acc[i]);
    } else {
      *reinterpret_cast<uint4*>(out + t * H + c * 8) = float_to_bf16x8(acc);
    }
  }
}

__global__ void __launch_bounds__(1024) moe_dispatch_kernel(const int* __restrict__ idx, int S, int top_k, int E,
                                                            int* __restrict__ pos, int* __restrict__ src_tok,
                                                            int* g_count, int* g_row0, int* g_rows, int* g_expert,
                                                            int max_tiles) {
  // Shared memory: per-warp histograms [32][E] (a warp's atomics only meet its own lanes), then the
  // per-expert totals, row offsets and tile offsets.  One CTA: the whole dispatch of a 2048-token chunk
  // (16384 slots) is ~10 us of shared-memory work; several CTAs would need a grid-wide prefix.
  extern __shared__ int dsm[];
  int* wh = dsm;                 // [32][E] slots of expert e seen by warp w; later the warp's running cursor
  int* cnt = dsm + 32 * E;       // [E]
  int* off = cnt + E;            // [E + 1] first sorted row of every expert
  int* toff = off + E + 1;       // [E + 1] first tile of every expert
  griddep_launch();
  griddep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < 32 * E; i += 1024) wh[i] = 0;
  __syncthreads();
  // every warp owns a contiguous range of slots (so that the second pass sees the same slots)
  const int per = (S + 31) / 32, s0 = warp * per, s1 = min(S, s0 + per);
  for (int s = s0 + lane; s < s1; s += 32) {
    const int e = idx[s];
    if (e >= 0 && e < E) atomicAdd(&wh[warp * E + e], 1);
  }
  __syncthreads();
  // totals per expert and, in place, the exclusive prefix over warps (the warp's first row inside the expert)
  for (int e = tid; e < E; e += 1024) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int n = wh[w * E + e];
      wh[w * E + e] = run;
      run += n;
    }
    cnt[e] = run;
  }
  __syncthreads();
  // exclusive prefixes over experts: rows and 128-row tiles (one warp, E <= 1024)
  if (warp == 0) {
    int carry_r = 0, carry_t = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int n = e < E ? cnt[e] : 0, nt = (n + 127) >> 7;
      int pr = n, pt = nt;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int ur = __shfl_up_sync(0xffffffffu, pr, d), ut = __shfl_up_sync(0xffffffffu, pt, d);
        if (lane >= d) { pr += ur; pt += ut; }
      }
      if (e < E) { off[e] = carry_r + pr - n; toff[e] = carry_t + pt - nt; }
      carry_r += __shfl_sync(0xffffffffu, pr, 31);
      carry_t += __shfl_sync(0xffffffffu, pt, 31);
    }
    if (lane == 0) {
      off[E] = carry_r;
      toff[E] = carry_t;
      *g_count = min(carry_t, max_tiles);
    }
  }
  __syncthreads();
  // tile list: expert e emits its tiles at toff[e]
  for (int e = tid; e < E; e += 1024) {
    const int n = cnt[e], r0 = off[e];
    int nt = toff[e];
    for (int i = 0; i < n; i += 128, ++nt) {
      if (nt < max_tiles) {
        g_row0[nt] = r0 + i;
        g_rows[nt] = min(128, n - i);
        g_expert[nt] = e;
      }
    }
  }
  for (int r = off[E] + tid; r < S; r += 1024) src_tok[r] = 0;
  // scatter: slot -> sorted row = first row of the expert + rows of earlier warps + this warp's cursor
  for (int s = s0 + lane; s < s1; s += 32) {
    const int e = idx[s];
    if (e >= 0 && e < E) {
      const int r = off[e] + atomicAdd(&wh[warp * E + e], 1);
      pos[s] = r;
      src_tok[r] = s / top_k;
    } else {
      pos[s] = -1;
    }
  }
}

}  // namespace

CB_EXPORT int cb_moe_router(const void* logits, int64_t ldl, int64_t T, int64_t E, int64_t top_k, int64_t normalize,
                            void* out_idx, void* out_w, int64_t e_lo, int64_t e_hi, void* stream) {
  if (T == 0) return 0;
  if (E > 512 || top_k > kMaxTopK || top_k < 1 || top_k > E) return CB_ERR_SHAPE;
  return (int)cb_launch(moe_router_kernel, dim3((unsigned)((T + 7) / 8)), dim3(256), 0, (cudaStream_t)stream,
                        (const float*)logits, ldl, (int)E, (int)top_k, (int)normalize, (int*)out_idx, (float*)out_w, (int)T, (int)e_lo, (int)e_hi);
}

CB_EXPORT int cb_moe_combine(const void* y, const void* w, const void* shared, const void* gate_logit, int64_t ldg,
                             void* out, int64_t T, int64_t H, int64_t top_k, const void* tp, int64_t push_site,
                             void* stream) {
  if (T == 0) return 0;
  if (H % 8 || (push_site >= 0 && !tp)) return CB_ERR_SHAPE;
  TpComm c;
  if (tp) c = *(const TpComm*)tp; else memset(&c, 0, sizeof(c));
  return (int)cb_launch(moe_combine_kernel, dim3((unsigned)T), dim3(256), 0, (cudaStream_t)stream, (const bf16*)y,
                        (const float*)w, (const bf16*)shared, (const float*)gate_logit, ldg, (bf16*)out, H, (int)top_k,
                        (int)push_site, c, (const int*)nullptr);
}

// The same merge for expert-sorted rows: slot (t, j)'s row of y is pos[t * top_k + j] (< 0: none).
CB_EXPORT int cb_moe_combine_pos(const void* y, const void* w, const void* pos, const void* shared, const void* gate_logit,
                                 int64_t ldg, void* out, int64_t T, int64_t H, int64_t top_k, void* stream) {
  if (T == 0) return 0;
  if (H % 8 || !pos) return CB_ERR_SHAPE;
  TpComm c;
  memset(&c, 0, sizeof(c));
  return (int)cb_launch(moe_combine_kernel, dim3((unsigned)T), dim3(256), 0, (cudaStream_t)stream, (const bf16*)y,
                        (const float*)w, (const bf16*)shared, (const float*)gate_logit, ldg, (bf16*)out, H, (int)top_k,
                        -1, c, (const int*)pos);
}

// Expert-major dispatch of S = T * top_k routed slots, one CTA: per-warp histograms, prefixes over warps and
// experts, scatter (53 us -> with one shared histogram and a serial prefix the CTA spent its time in barriers).
//   pos[s]      row of slot s in the expert-sorted order, -1 for a slot whose expert is not local
//   src_tok[r]  token whose activation row goes to sorted row r (0 for the unused rows at the end)
//   tile list   m-tiles of at most 128 rows that never cross an expert boundary (g_count of them)
// Rows of one expert are adjacent but in no fixed order among themselves: every output row depends
// on its own input row only, so the result does not depend on that order.
// Replaces the reference's moe_dispatch (kernels/moe_dispatch.cu:101, count -> prefix -> scatter).
CB_EXPORT int cb_moe_dispatch(const void* idx, int64_t S, int64_t top_k, int64_t E, void* pos, void* src_tok,
                              void* g_count, void* g_row0, void* g_rows, void* g_expert, int64_t max_tiles,
                              void* stream) {
  if (S < 1 || E < 1 || E > 1024 || top_k < 1 || max_tiles < 1) return CB_ERR_SHAPE;
  const size_t smem = (size_t)(32 * E + 3 * E + 2) * sizeof(int);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(moe_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cb_launch(moe_dispatch_kernel, dim3(1), dim3(1024), smem, (cudaStream_t)stream,
                        (const int*)idx, (int)S, (int)top_k, (int)E, (int*)pos, (int*)src_tok, (int*)g_count,
                        (int*)g_row0, (int*)g_rows, (int*)g_expert, (int)max_tiles);
}
