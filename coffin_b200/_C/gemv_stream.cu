// Single-row decode GEMV that streams the weights through per-warp cp.async rings.
//
// y[n] = sum_k W[n, k] x[k] for one activation row (the batch-1 decode step, where every
// projection is a pure HBM stream).  A register-staged loop keeps only ~16 loads per lane in
// flight and loses a full memory latency per batch; here each warp owns a small shared-memory
// ring and keeps NST row slices (~10 KB per warp, ~160 KB per SM with two CTAs) in flight with
// cp.async, independent of register pressure.  Work is cut into units of one row slice
// (K / ksplit elements); a CTA owns a contiguous band of rows, its warps take units round-robin,
// every unit's partial sum goes to shared memory and one barrier at the end reduces them in a fixed
// order (deterministic).  The first slices are requested before the wait on the previous kernel,
// so under programmatic dependent launch the weight stream crosses kernel boundaries.
// Same fused prologue (residual add + RMSNorm) and epilogue (SwiGLU, fp32 logits) as gemv.cu.
#include <string.h>
#include "tp.cuh"

namespace {

constexpr int kW = 8, kT = kW * 32;
constexpr int kRingBytes = 10 * 1024;   // per warp

struct StreamArgs {
  const bf16* W; const bf16* x; void* y;
  int64_t N, K, up_off;
  const bf16* res_in; const bf16* add; const float* gain; bf16* res_out;
  float eps;
  int rounds;         // rounds of the grid-wide sweep (one unit per warp per round)
  int ksplit;         // slices per row
  int slc;            // chunks (16 B) per slice, a multiple of 32
  int nst;            // ring stages per warp
  int pull_site, push_site;   // tensor parallel: -1 = off
  TpComm tp;
};

__device__ __forceinline__ void cp16(uint32_t saddr, const void* g) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(saddr), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void cp_wait_dyn(int n) {  // wait until at most n groups are pending
  switch (n) {
    case 0: cp_wait<0>(); break;
    case 1: cp_wait<1>(); break;
    case 2: cp_wait<2>(); break;
    case 3: cp_wait<3>(); break;
    case 4: cp_wait<4>(); break;
    case 5: cp_wait<5>(); break;
    case 6: cp_wait<6>(); break;
    default: cp_wait<7>(); break;
  }
}

template <bool SWIGLU, bool NORM, bool OUT_F32>
__global__ void __launch_bounds__(kT, 2) gemv_stream_kernel(const StreamArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int64_t K = a.K, nchunk = K >> 3;
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);                                   // [K]
  unsigned char* rings = smem_raw + ((K * 2 + 15) & ~(int64_t)15);                // [kW][kRingBytes]
  float* part = reinterpret_cast<float*>(rings + kW * kRingBytes);                // [units]
  __shared__ float red[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // Sweep order: in round r the whole grid covers a contiguous window of rows (CTA c takes the
  // kW / upr rows starting at (r * grid + c) * rpr), so the rows in flight across the GPU at any
  // time are neighbours in memory and DRAM pages stay open; per-CTA bands would scatter ~300
  // independent streams over the matrix instead.
  const int upr = a.ksplit * (SWIGLU ? 2 : 1), rpr = kW / upr;   // units per logical row, rows per round
  const int my_units = a.rounds;
  const int slc = a.slc, per_lane = slc >> 5, nst = a.nst;
  const uint32_t ring0 = (uint32_t)__cvta_generic_to_shared(rings + warp * kRingBytes);
  const unsigned char* ringp = rings + warp * kRingBytes;
  const int q = warp % upr, my_ks = q % a.ksplit, my_half = q / a.ksplit;

  auto unit_src = [&](int j, int& ks) -> const bf16* {   // this warp's unit in round j (null if past the end)
    ks = my_ks;
    const int64_t lrow = ((int64_t)j * gridDim.x + blockIdx.x) * rpr + warp / upr;
    if (lrow >= a.N) return nullptr;
    return a.W + (my_half ? a.up_off + lrow : lrow) * K;
  };
  auto issue = [&](int j) {
    int ks;
    const bf16* src = j < my_units ? unit_src(j, ks) : nullptr;
    if (src) {
      const uint32_t dst = ring0 + (uint32_t)(j % nst) * (uint32_t)slc * 16u;
#pragma unroll 4
      for (int i = 0; i < per_lane; ++i) {
        const int64_t c = (int64_t)ks * slc + lane + 32 * i;
        if (c < nchunk) cp16(dst + (uint32_t)(lane + 32 * i) * 16u, src + c * 8);
      }
    }
    cp_commit();
  };

  griddep_launch();
  for (int j = 0; j < nst - 1; ++j) issue(j);     // weights do not depend on the previous kernel
  griddep_wait();

  // ---- prologue: the activation row into shared memory ------------------------------------
  if (NORM) {
    float ss = 0.f;
    for (int64_t c = tid; c < nchunk; c += kT) {
      float f[8], g[8];
      bf16x8_to_float(*reinterpret_cast<const uint4*>(a.res_in + c * 8), f);
      if (a.pull_site >= 0) {   // add = sum over ranks of the previous projection's partial outputs
#pragma unroll
        for (int i = 0; i < 8; ++i)
          f[i] = __bfloat162float(__float2bfloat16(f[i] + tp_pull_value(a.tp, a.pull_site, c * 8 + i)));
      } else if (a.add) {
        bf16x8_to_float(*reinterpret_cast<const uint4*>(a.add + c * 8), g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i] + g[i]));
      }
      const uint4 packed = float_to_bf16x8(f);
      *reinterpret_cast<uint4*>(xs + c * 8) = packed;
      if (a.res_out && blockIdx.x == 0) *reinterpret_cast<uint4*>(a.res_out + c * 8) = packed;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    const float rstd = rsqrtf(block_sum(ss, red) / (float)K + a.eps);
    for (int64_t c = tid; c < nchunk; c += kT) {
      float f[8];
      bf16x8_to_float(*reinterpret_cast<const uint4*>(xs + c * 8), f);
      const float4 g0 = *reinterpret_cast<const float4*>(a.gain + c * 8);
      const float4 g1 = *reinterpret_cast<const float4*>(a.gain + c * 8 + 4);
      f[0] *= rstd * g0.x; f[1] *= rstd * g0.y; f[2] *= rstd * g0.z; f[3] *= rstd * g0.w;
      f[4] *= rstd * g1.x; f[5] *= rstd * g1.y; f[6] *= rstd * g1.z; f[7] *= rstd * g1.w;
      *reinterpret_cast<uint4*>(xs + c * 8) = float_to_bf16x8(f);
    }
  } else {
    for (int64_t c = tid; c < nchunk; c += kT)
      *reinterpret_cast<uint4*>(xs + c * 8) = *reinterpret_cast<const uint4*>(a.x + c * 8);
  }
  __syncthreads();

  // ---- stream the units -----------------------------------------------------------------------
  for (int j = 0; j < my_units; ++j) {
    issue(j + nst - 1);
    cp_wait_dyn(nst - 1);             // this lane's copies of unit j have landed
    int ks;
    const bool valid = unit_src(j, ks) != nullptr;
    const unsigned char* st = ringp + (size_t)(j % nst) * slc * 16;
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll 2
    for (int i = 0; i < per_lane; ++i) {
      const int64_t c = (int64_t)ks * slc + lane + 32 * i;
      if (valid && c < nchunk) {
        float wf[8], xf[8];
        bf16x8_to_float(*reinterpret_cast<const uint4*>(st + (size_t)(lane + 32 * i) * 16), wf);
        bf16x8_to_float(*reinterpret_cast<const uint4*>(xs + c * 8), xf);
#pragma unroll
        for (int e = 0; e < 8; e += 2) { acc0 = fmaf(wf[e], xf[e], acc0); acc1 = fmaf(wf[e + 1], xf[e + 1], acc1); }
      }
    }
    const float s = warp_sum(acc0 + acc1);
    if (lane == 0) part[j * kW + warp] = s;
  }
  cp_wait<0>();
  __syncthreads();

  // ---- fixed-order reduction of the slices, epilogue ------------------------------------------
  for (int idx = tid; idx < a.rounds * rpr; idx += kT) {
    const int r = idx / rpr, i = idx % rpr;
    const int64_t lrow = ((int64_t)r * gridDim.x + blockIdx.x) * rpr + i;
    if (lrow >= a.N) continue;
    float v = 0.f, v2 = 0.f;
    for (int s = 0; s < a.ksplit; ++s) {
      v += part[r * kW + i * upr + s];
      if (SWIGLU) v2 += part[r * kW + i * upr + a.ksplit + s];
    }
    if (SWIGLU) v = silu_f(v) * v2;
    if (a.push_site >= 0) tp_push_value(a.tp, a.push_site, lrow, v);
    else if (OUT_F32) reinterpret_cast<float*>(a.y)[lrow] = v;
    else reinterpret_cast<bf16*>(a.y)[lrow] = __float2bfloat16(v);
  }
}

int g_stream_sms = 0;
int g_stream_ctas = 2;

template <bool SWIGLU, bool NORM, bool OUT_F32>
int launch_stream(StreamArgs a, cudaStream_t st) {
  if (!g_stream_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_stream_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_stream_sms <= 0) g_stream_sms = 148;
  }
  const int64_t nchunk = a.K >> 3;
  // slice of about 2.5 KB (four ring stages per warp), at most 8 / (swiglu ? 2 : 1) slices per row
  const int max_ks = SWIGLU ? 4 : 8;
  int ks = 1;
  while (ks < max_ks && (((nchunk + ks - 1) / ks + 31) & ~(int64_t)31) * 16 > 2560) ks <<= 1;
  a.ksplit = ks;
  a.slc = (int)(((nchunk + ks - 1) / ks + 31) & ~(int64_t)31);
  if ((int64_t)a.slc * 16 * 2 > kRingBytes) return CB_ERR_SHAPE;
  a.nst = (int)min((int64_t)8, (int64_t)kRingBytes / ((int64_t)a.slc * 16));
  const int rpr = kW / (ks * (SWIGLU ? 2 : 1));
  const int64_t slots = (int64_t)g_stream_sms * g_stream_ctas;
  const int64_t grid = min(slots, (a.N + rpr - 1) / rpr);
  a.rounds = (int)((a.N + grid * rpr - 1) / (grid * rpr));
  const size_t smem = (size_t)((a.K * 2 + 15) & ~(int64_t)15) + (size_t)kW * kRingBytes +
                      (size_t)a.rounds * kW * sizeof(float) + 16;
  if (smem > 110 * 1024) return CB_ERR_SHAPE;
  auto kern = gemv_stream_kernel<SWIGLU, NORM, OUT_F32>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  return (int)cb_launch(kern, dim3((unsigned)grid), dim3(kT), smem, st, a);
}

}  // namespace

CB_EXPORT int cb_set_stream_opts(int64_t ctas_per_sm) { g_stream_ctas = ctas_per_sm < 1 ? 1 : (int)ctas_per_sm; return 0; }

// Single-row projection; same arguments as cb_gemv_bf16 with M fixed to 1.
CB_EXPORT int cb_gemv_stream_bf16(const void* W, const void* x, void* y, int64_t N, int64_t K, int64_t mode,
                                  int64_t up_off, const void* res_in, const void* add, const void* gain,
                                  void* res_out, float eps, const void* tp, int64_t pull_site, int64_t push_site,
                                  void* stream) {
  if (!W || (!y && push_site < 0) || (!x && !res_in) || (res_in && !gain)) return CB_ERR_ARG;
  if ((pull_site >= 0 || push_site >= 0) && !tp) return CB_ERR_ARG;
  if (pull_site >= 0 && !res_in) return CB_ERR_ARG;
  if (K % 8 || N < 1) return CB_ERR_SHAPE;
  if (res_in && res_out && (res_out == res_in || res_out == add)) return CB_ERR_ARG;
  StreamArgs a;
  a.W = (const bf16*)W; a.x = (const bf16*)x; a.y = y; a.N = N; a.K = K; a.up_off = up_off;
  a.res_in = (const bf16*)res_in; a.add = (const bf16*)add; a.gain = (const float*)gain;
  a.res_out = (bf16*)res_out; a.eps = eps; a.rounds = 0; a.ksplit = 1; a.slc = 32; a.nst = 2;
  a.pull_site = (int)pull_site; a.push_site = (int)push_site;
  if (tp) a.tp = *(const TpComm*)tp; else memset(&a.tp, 0, sizeof(a.tp));
  const bool sw = mode & 1, f32 = mode & 2, norm = res_in != nullptr;
  cudaStream_t st = (cudaStream_t)stream;
  if (sw) {
    if (f32) return CB_ERR_ARG;
    return norm ? launch_stream<true, true, false>(a, st) : launch_stream<true, false, false>(a, st);
  }
  if (f32) return norm ? launch_stream<false, true, true>(a, st) : launch_stream<false, false, true>(a, st);
  return norm ? launch_stream<false, true, false>(a, st) : launch_stream<false, false, false>(a, st);
}
