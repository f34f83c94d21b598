// Bandwidth-bound bf16 GEMV for decode (M <= 8 rows share one weight read).
//
// y[m, n] = sum_k W[n, k] * x[m, k], W row-major [N, K] (the checkpoint layout, K contiguous).
// The kernel is built around three facts of the decode step on B200:
//   * the weights are read exactly once (8 GB per token on the 4B model), so every lane
//     issues 16-byte streaming loads with U*PHYS of them in flight before any use;
//   * small-N projections (o_proj / out_proj / down_proj, N = hidden) do not fill 148 SMs by
//     rows alone, so the warps of a CTA can split K (KSPLIT) and reduce through shared memory;
//   * the op before a projection is always "residual add + RMSNorm" and the op after the
//     gate/up projection is always SwiGLU, so both are folded in: every CTA recomputes the
//     (tiny) normalised activation row into shared memory while its first weight lines are in
//     flight, and the SwiGLU variant computes gate row i and up row i in the same warp.
// Replaces the reference's gemv family (backends/corex/kernels/gemv.cu:76-947, one launch
// each for add, norm, GEMV, silu_mul) with a single launch per projection.
#include <string.h>
#include "tp.cuh"

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kU = 4;  // 16-byte loads in flight per lane per physical row

struct GemvArgs {
  const bf16* W;      // [N(or 2N for swiglu), K]
  const bf16* x;      // [M, K] when no norm prologue
  void* y;            // [M, N] bf16 or fp32
  int64_t N, K, ldy;  // logical output rows, reduction length, output row pitch (elements)
  int64_t up_off;     // swiglu: row offset of the "up" half inside W
  // norm prologue: x = rmsnorm(res_in + add) * gain ; block 0 also writes res_out = res_in + add
  const bf16* res_in;
  const bf16* add;    // may be null
  const float* gain;  // [K] fp32, already 1 + w
  bf16* res_out;      // may be null (no residual write-back); must not alias res_in/add
  float eps;
  int nrg;            // row groups per round; KSPLIT = kWarps / nrg
  int rounds;         // rounds of the grid-wide sweep (nrg * R rows per CTA per round)
  int pf_rounds;      // rounds of weights kept in flight towards L2 ahead of the compute
  int pull_site, push_site;   // tensor parallel: -1 = off
  TpComm tp;
};

// L2 prefetch of the weight rows [ra, rb) (contiguous bytes), one 128-byte line per thread-step.
__device__ __forceinline__ void prefetch_rows(const bf16* W, int64_t K, int64_t ra, int64_t rb) {
  if (rb <= ra) return;
  const char* base = reinterpret_cast<const char*>(W + ra * K);
  const int64_t bytes = (rb - ra) * K * (int64_t)sizeof(bf16);
  for (int64_t off = (int64_t)threadIdx.x * 128; off < bytes; off += (int64_t)kThreads * 128)
    asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
}

// One CTA per SM owns a contiguous band of output rows and walks it in rounds of nrg * R rows.
// The band's weights are pulled into L2 a few rounds ahead of the arithmetic, starting before the
// wait on the previous kernel, so that under programmatic dependent launch the HBM stream never
// stops at a kernel boundary; the compute phase then reads L2-resident lines.
template <int M, int R, bool SWIGLU, bool NORM, bool OUT_F32>
__global__ void __launch_bounds__(kThreads, 2) gemv_kernel(const GemvArgs a) {
  constexpr int PHYS = R * (SWIGLU ? 2 : 1);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);                       // [M][K]
  float* part = reinterpret_cast<float*>(smem_raw + (size_t)M * a.K * sizeof(bf16));  // [kWarps][PHYS][M]
  __shared__ float red[32];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nrg = a.nrg, ksplit = kWarps / nrg;
  const int rg = warp % nrg, ks = warp / nrg;
  const int64_t K = a.K;
  const int round_rows = nrg * R;
  // Sweep order: in round r the grid covers one contiguous window of rows (CTA c takes the
  // round_rows rows at (r * grid + c) * round_rows), so concurrently streamed rows are neighbours
  // in memory and DRAM pages stay open.
  const int nrounds = a.rounds;
  const int64_t row_end = a.N;
  auto round_start = [&](int r) { return ((int64_t)r * gridDim.x + blockIdx.x) * round_rows; };
  const int64_t nchunk = K >> 3;                 // 16-byte chunks per row
  const int64_t cper = ((nchunk + ksplit - 1) / ksplit + 31) & ~(int64_t)31;
  const int64_t c0 = ks * cper, c1 = min(nchunk, c0 + cper);

  griddep_launch();
  for (int r = 0; r < a.pf_rounds && r < nrounds; ++r) {
    const int64_t pa = round_start(r), pb = min(row_end, pa + round_rows);
    prefetch_rows(a.W, K, pa, pb);
    if (SWIGLU) prefetch_rows(a.W, K, a.up_off + pa, a.up_off + pb);
  }
  griddep_wait();

  // ---- prologue: activation rows into shared memory --------------------------------------
  if (NORM) {
    for (int m = 0; m < M; ++m) {
      float ss = 0.f;
      for (int64_t c = tid; c < nchunk; c += kThreads) {
        float f[8], g[8];
        bf16x8_to_float(*reinterpret_cast<const uint4*>(a.res_in + m * K + c * 8), f);
        if (a.pull_site >= 0) {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            f[i] = __bfloat162float(__float2bfloat16(f[i] + tp_pull_value(a.tp, a.pull_site, m * K + c * 8 + i)));
        } else if (a.add) {
          bf16x8_to_float(*reinterpret_cast<const uint4*>(a.add + m * K + c * 8), g);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i] + g[i]));
        }
        uint4 packed = float_to_bf16x8(f);
        *reinterpret_cast<uint4*>(xs + m * K + c * 8) = packed;
        if (a.res_out && blockIdx.x == 0) *reinterpret_cast<uint4*>(a.res_out + m * K + c * 8) = packed;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
      }
      const float rstd = rsqrtf(block_sum(ss, red) / (float)K + a.eps);
      for (int64_t c = tid; c < nchunk; c += kThreads) {
        float f[8];
        bf16x8_to_float(*reinterpret_cast<const uint4*>(xs + m * K + c * 8), f);
        const float4 g0 = *reinterpret_cast<const float4*>(a.gain + c * 8);
        const float4 g1 = *reinterpret_cast<const float4*>(a.gain + c * 8 + 4);
        f[0] *= rstd * g0.x; f[1] *= rstd * g0.y; f[2] *= rstd * g0.z; f[3] *= rstd * g0.w;
        f[4] *= rstd * g1.x; f[5] *= rstd * g1.y; f[6] *= rstd * g1.z; f[7] *= rstd * g1.w;
        *reinterpret_cast<uint4*>(xs + m * K + c * 8) = float_to_bf16x8(f);
      }
    }
  } else {
    for (int64_t c = tid; c < (int64_t)M * nchunk; c += kThreads)
      *reinterpret_cast<uint4*>(xs + c * 8) = *reinterpret_cast<const uint4*>(a.x + c * 8);
  }
  __syncthreads();

  for (int round = 0; round < nrounds; ++round) {
    const int64_t round0 = round_start(round);
    if (a.pf_rounds > 0 && round + a.pf_rounds < nrounds) {  // keep the L2 stream pf_rounds ahead
      const int64_t pa = round_start(round + a.pf_rounds);
      const int64_t pb = min(row_end, pa + round_rows);
      prefetch_rows(a.W, K, pa, pb);
      if (SWIGLU) prefetch_rows(a.W, K, a.up_off + pa, a.up_off + pb);
    }
    const int64_t row0 = round0 + rg * R;  // first logical row of this warp in this round
    // physical row pointers (clamped so out-of-range warps read valid memory and skip the store)
    const bf16* wrow[PHYS];
#pragma unroll
    for (int p = 0; p < PHYS; ++p) {
      int64_t r = row0 + (p % R);
      if (r >= a.N) r = a.N - 1;
      if (SWIGLU && p >= R) r += a.up_off;
      wrow[p] = a.W + r * K;
    }
    float acc[PHYS][M];
#pragma unroll
    for (int p = 0; p < PHYS; ++p)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[p][m] = 0.f;

    if (row0 < row_end) {
      for (int64_t c = c0 + lane; c < c1; c += 32 * kU) {
        uint4 wv[kU][PHYS];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int64_t cc = c + 32 * u;
#pragma unroll
          for (int p = 0; p < PHYS; ++p)
            wv[u][p] = (cc < c1) ? ld_stream(wrow[p] + cc * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
          const int64_t cc = c + 32 * u;
          if (cc < c1) {
            float wf[PHYS][8];
#pragma unroll
            for (int p = 0; p < PHYS; ++p) bf16x8_to_float(wv[u][p], wf[p]);
#pragma unroll
            for (int m = 0; m < M; ++m) {
              float xf[8];
              bf16x8_to_float(*reinterpret_cast<const uint4*>(xs + m * K + cc * 8), xf);
#pragma unroll
              for (int p = 0; p < PHYS; ++p)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[p][m] = fmaf(wf[p][i], xf[i], acc[p][m]);
            }
          }
        }
      }
    }
    // ---- reduce: lanes, then (if K is split) the warps ------------------------------------
#pragma unroll
    for (int p = 0; p < PHYS; ++p)
#pragma unroll
      for (int m = 0; m < M; ++m) acc[p][m] = warp_sum(acc[p][m]);
    if (ksplit == 1) {
      // every lane holds the sums; lane (r * M + m) stores logical row r of row m
      if (lane < R * M) {
        const int m = lane % M, r = lane / M;
        const int64_t row = row0 + r;
        float v = 0.f, v2 = 0.f;
#pragma unroll
        for (int p = 0; p < R; ++p)
#pragma unroll
          for (int mm = 0; mm < M; ++mm)
            if (p == r && mm == m) { v = acc[p][mm]; if (SWIGLU) v2 = acc[R + p][mm]; }
        if (row < row_end) {
          if (SWIGLU) v = silu_f(v) * v2;
          if (a.push_site >= 0) tp_push_value(a.tp, a.push_site, m * a.N + row, v);
          else if (OUT_F32) reinterpret_cast<float*>(a.y)[m * a.ldy + row] = v;
          else reinterpret_cast<bf16*>(a.y)[m * a.ldy + row] = __float2bfloat16(v);
        }
      }
    } else {
      __syncthreads();  // previous round's partials consumed
      if (lane == 0) {
#pragma unroll
        for (int p = 0; p < PHYS; ++p)
#pragma unroll
          for (int m = 0; m < M; ++m) part[(warp * PHYS + p) * M + m] = acc[p][m];
      }
      __syncthreads();
      for (int o = tid; o < nrg * R * M; o += kThreads) {
        const int m = o % M, r = (o / M) % R, g = o / (M * R);
        const int64_t row = round0 + g * R + r;
        if (row >= row_end) continue;
        float v = 0.f, v2 = 0.f;
        for (int s = 0; s < ksplit; ++s) {
          const int w = s * nrg + g;
          v += part[(w * PHYS + r) * M + m];
          if (SWIGLU) v2 += part[(w * PHYS + R + r) * M + m];
        }
        if (SWIGLU) v = silu_f(v) * v2;
        if (a.push_site >= 0) tp_push_value(a.tp, a.push_site, m * a.N + row, v);
        else if (OUT_F32) reinterpret_cast<float*>(a.y)[m * a.ldy + row] = v;
        else reinterpret_cast<bf16*>(a.y)[m * a.ldy + row] = __float2bfloat16(v);
      }
    }
  }
}

int g_gemv_sms = 0;
int g_gemv_ctas_per_sm = 2;   // CTAs per SM the band partition targets
int g_gemv_prefetch = 1;      // L2 prefetch-ahead on/off

template <int M, int R, bool SWIGLU, bool NORM, bool OUT_F32>
int launch(const GemvArgs& a0, cudaStream_t st) {
  GemvArgs a = a0;
  constexpr int PHYS = R * (SWIGLU ? 2 : 1);
  if (!g_gemv_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_gemv_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_gemv_sms <= 0) g_gemv_sms = 148;
  }
  // Row groups per round: all eight warps on distinct rows when there are enough rows to fill the
  // grid that way, else split K across warps so that narrow outputs still occupy every SM.
  const int64_t slots = (int64_t)g_gemv_sms * g_gemv_ctas_per_sm;
  int nrg = kWarps;
  while (nrg > 1 && (a.N + (int64_t)nrg * R - 1) / ((int64_t)nrg * R) < slots && (a.K >> 3) / (kWarps / (nrg / 2)) >= 64)
    nrg >>= 1;
  a.nrg = nrg;
  const int64_t rr = (int64_t)nrg * R;
  const int64_t grid = min(slots, (a.N + rr - 1) / rr);
  a.rounds = (int)((a.N + grid * rr - 1) / (grid * rr));
  const int64_t round_bytes = rr * (SWIGLU ? 2 : 1) * a.K * 2;
  a.pf_rounds = g_gemv_prefetch ? (int)max((int64_t)1, min((int64_t)8, (64 * 1024) / max((int64_t)1, round_bytes))) : 0;
  const size_t smem = (size_t)M * a.K * sizeof(bf16) + (size_t)kWarps * PHYS * M * sizeof(float);
  if (smem > 100 * 1024) return CB_ERR_SHAPE;
  auto kern = gemv_kernel<M, R, SWIGLU, NORM, OUT_F32>;
  if (smem + 2048 > 48 * 1024) {   // the 48 KB default also has to hold the static shared memory
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  cudaError_t e = cb_launch(kern, dim3((unsigned)grid), dim3(kThreads), smem, st, a);
  return (int)e;
}

template <int M>
int dispatch(const GemvArgs& a, bool swiglu, bool norm, bool f32, cudaStream_t st) {
  if (swiglu) {
    if (f32) return CB_ERR_ARG;
    return norm ? launch<M, 2, true, true, false>(a, st) : launch<M, 2, true, false, false>(a, st);
  }
  // narrow outputs (N = hidden) balance better with two rows per warp
  const bool narrow = a.N <= 8192;
  if (f32) return norm ? launch<M, 4, false, true, true>(a, st) : launch<M, 4, false, false, true>(a, st);
  if (narrow) return norm ? launch<M, 2, false, true, false>(a, st) : launch<M, 2, false, false, false>(a, st);
  return norm ? launch<M, 4, false, true, false>(a, st) : launch<M, 4, false, false, false>(a, st);
}

}  // namespace

CB_EXPORT int cb_set_gemv_opts(int64_t ctas_per_sm, int64_t prefetch) {
  g_gemv_ctas_per_sm = ctas_per_sm < 1 ? 1 : (int)ctas_per_sm;
  g_gemv_prefetch = prefetch ? 1 : 0;
  return 0;
}

// mode bits: 1 = swiglu epilogue (W holds gate rows then up rows at `up_off`), 2 = fp32 output.
// Norm prologue is enabled when res_in != null (then x is ignored).
CB_EXPORT int cb_gemv_bf16(const void* W, const void* x, void* y, int64_t M, int64_t N, int64_t K,
                           int64_t ldy, int64_t mode, int64_t up_off, const void* res_in,
                           const void* add, const void* gain, void* res_out, float eps, const void* tp,
                           int64_t pull_site, int64_t push_site, void* stream) {
  if (!W || (!y && push_site < 0) || (!x && !res_in) || (res_in && !gain)) return CB_ERR_ARG;
  if ((pull_site >= 0 || push_site >= 0) && !tp) return CB_ERR_ARG;
  if (pull_site >= 0 && !res_in) return CB_ERR_ARG;
  if (K % 8 || M < 1 || M > 8 || N < 1) return CB_ERR_SHAPE;
  if (res_in && res_out && (res_out == res_in || res_out == add)) return CB_ERR_ARG;
  GemvArgs a;
  a.W = (const bf16*)W; a.x = (const bf16*)x; a.y = y; a.N = N; a.K = K; a.ldy = ldy;
  a.up_off = up_off; a.res_in = (const bf16*)res_in; a.add = (const bf16*)add;
  a.gain = (const float*)gain; a.res_out = (bf16*)res_out; a.eps = eps; a.nrg = 1; a.rounds = 0; a.pf_rounds = 1;
  a.pull_site = (int)pull_site; a.push_site = (int)push_site;
  if (tp) a.tp = *(const TpComm*)tp; else memset(&a.tp, 0, sizeof(a.tp));
  const bool sw = mode & 1, f32 = mode & 2, norm = res_in != nullptr;
  cudaStream_t st = (cudaStream_t)stream;
  switch (M) {
    case 1: return dispatch<1>(a, sw, norm, f32, st);
    case 2: return dispatch<2>(a, sw, norm, f32, st);
    case 3: case 4: {
      if (M == 3) return CB_ERR_SHAPE;
      return dispatch<4>(a, sw, norm, f32, st);
    }
    case 8: return dispatch<8>(a, sw, norm, f32, st);
    default: return CB_ERR_SHAPE;
  }
}
