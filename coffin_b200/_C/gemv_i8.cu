// W8A8 decode projection (1..8 activation rows): int8 weights [N, K] with a per-row scale, the
// activation rows quantised per token to int8 inside the prologue, dot products on the int8 tensor
// core path (mma.m16n8k32.s8, exact int32 accumulation), result * x_scale[m] * w_scale[n].
// Same structure as gemv_mma.cu: a warp owns 16 weight rows, lane (g, t) loads 16-byte chunks
// (16 int8) of rows g and g+8 which are its A fragments for two MMAs under a k permutation that
// the activation (B operand, from shared memory) follows; fused residual add + RMSNorm prologue,
// SwiGLU / fp32 epilogues, K-split for narrow outputs, grid-wide sweep order.  Halves the bytes
// streamed per token relative to bf16.  Replaces the reference's int8 GEMV family
// (backends/corex/kernels/gemv.cu:839-947 nk int8, w8a8.cu:76-242 activation quant).
#include <string.h>
#include <algorithm>
#include "tp.cuh"

namespace {

constexpr int kW = 8, kT = kW * 32;

struct I8Args {
  const int8_t* W; const float* wscale; const bf16* x; void* y;
  int64_t N, K, ldy, up_off;
  const bf16* res_in; const bf16* add; const float* gain; bf16* res_out;
  float eps;
  int M, ksplit, rounds;
  int pull_site, push_site;   // tensor parallel: -1 = off
  TpComm tp;
  // routed experts (slot mode): blockIdx.y selects (expert, activation row); W is a stack [E, expert_rows, K]
  // with wscale [E, expert_rows]
  const int* slot_expert; const int* slot_xrow; int64_t expert_rows;
};

__device__ __forceinline__ void mma_s8(int* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool SWIGLU, bool NORM, bool OUT_F32>
__global__ void __launch_bounds__(kT, 3) gemv_i8_kernel(const I8Args a_in) {
  constexpr int PB = SWIGLU ? 2 : 1;
  constexpr int U = SWIGLU ? 2 : 4;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  I8Args a = a_in;
  if (a.slot_expert) {
    asm volatile("griddepcontrol.wait;" ::: "memory");      // the routing tables come from the kernel just before
    const int slot = blockIdx.y, e = a.slot_expert[slot];
    if (e < 0) { cbtrace::stamp(0); cbtrace::stamp(1); return; }      // a slot routed to another rank's expert
    a.W += (int64_t)e * a.expert_rows * a.K;
    a.wscale += (int64_t)e * a.expert_rows;
    a.x += (int64_t)(a.slot_xrow ? a.slot_xrow[slot] : slot) * a.K;
    a.y = OUT_F32 ? (void*)(reinterpret_cast<float*>(a.y) + (int64_t)slot * a.ldy)
                  : (void*)(reinterpret_cast<bf16*>(a.y) + (int64_t)slot * a.ldy);
  }
  const int64_t K = a.K, nchunk = K >> 4;          // 16 int8 per chunk
  const int M = a.M;
  bf16* stage = reinterpret_cast<bf16*>(smem_raw);                         // [K] staging row (values are bf16-exact)
  int8_t* xq = reinterpret_cast<int8_t*>(smem_raw + (size_t)K * 2);         // [M][K]
  float* xscale = reinterpret_cast<float*>(smem_raw + (size_t)K * 2 + (((size_t)M * K + 15) & ~(size_t)15));  // [8]
  float* part = xscale + 8;                                                 // [rounds][kW][PB][16][8]
  __shared__ float red[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int ksplit = a.ksplit, rbr = kW / ksplit;
  const int ks = warp % ksplit, rb_in = warp / ksplit;
  const int64_t npair = (nchunk + 3) >> 2;
  const int64_t pper = (npair + ksplit - 1) / ksplit;
  const int64_t p0 = ks * pper, p1 = min(npair, p0 + pper);

  auto row_ptrs = [&](int round, const int8_t** wlo, const int8_t** whi) -> bool {
    const int64_t blk = ((int64_t)round * gridDim.x + blockIdx.x) * rbr + rb_in;
    const int64_t r_lo = blk * 16 + g, r_hi = r_lo + 8;
#pragma unroll
    for (int b = 0; b < PB; ++b) {
      const int64_t off = b ? a.up_off : 0;
      wlo[b] = a.W + (off + min(r_lo, a.N - 1)) * K;
      whi[b] = a.W + (off + min(r_hi, a.N - 1)) * K;
    }
    return blk * 16 < a.N;
  };
  auto load_batch = [&](int64_t p, const int8_t* const* wlo, const int8_t* const* whi, uint4 (*lo)[PB], uint4 (*hi)[PB]) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t c = (p + u) * 4 + t;
      const bool ok = (p + u) < p1 && c < nchunk;
#pragma unroll
      for (int b = 0; b < PB; ++b) {
        lo[u][b] = ok ? ld_stream(wlo[b] + c * 16) : make_uint4(0, 0, 0, 0);
        hi[u][b] = ok ? ld_stream(whi[b] + c * 16) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  griddep_launch();
  uint4 lo[U][PB], hi[U][PB];
  {
    const int8_t* wlo[PB];
    const int8_t* whi[PB];
    if (row_ptrs(0, wlo, whi) && p0 < p1) load_batch(p0, wlo, whi, lo, hi);
  }
  griddep_wait();

  // ---- prologue: (residual add + norm,) per-row absmax, int8 quantisation into shared memory ----
  for (int m = 0; m < M; ++m) {
    float ss = 0.f;
    for (int64_t c = tid; c < (K >> 3); c += kT) {
      float f[8], q[8];
      if (NORM) {
        bf16x8_to_float(*reinterpret_cast<const uint4*>(a.res_in + m * K + c * 8), f);
        if (a.pull_site >= 0) {
          float pulled[8];
          tp_pull8(a.tp, a.pull_site, m * K + c * 8, pulled);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i] + pulled[i]));
        } else if (a.add) {
          bf16x8_to_float(*reinterpret_cast<const uint4*>(a.add + m * K + c * 8), q);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i] + q[i]));
        }
        if (a.res_out && blockIdx.x == 0) *reinterpret_cast<uint4*>(a.res_out + m * K + c * 8) = float_to_bf16x8(f);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
      } else {
        bf16x8_to_float(*reinterpret_cast<const uint4*>(a.x + m * K + c * 8), f);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) stage[c * 8 + i] = __float2bfloat16(f[i]);
    }
    float rstd = 1.f;
    if (NORM) rstd = rsqrtf(block_sum(ss, red) / (float)K + a.eps);
    else __syncthreads();
    float amax = 0.f;
    for (int64_t i = tid; i < K; i += kT) {
      float v = __bfloat162float(stage[i]);
      if (NORM) v = __bfloat162float(__float2bfloat16(v * rstd * a.gain[i]));   // the bf16 activation the dense path sees
      stage[i] = __float2bfloat16(v);
      amax = fmaxf(amax, fabsf(v));
    }
    amax = block_max(amax, red);
    const float sc = fmaxf(amax, 1e-8f) / 127.f, inv = 1.f / sc;
    if (tid == 0) xscale[m] = sc;
    for (int64_t i = tid; i < K; i += kT)
      xq[m * K + i] = (int8_t)max(-127, min(127, __float2int_rn(__bfloat162float(stage[i]) * inv)));
    __syncthreads();
  }

  const int8_t* xrow = xq + (int64_t)g * K;
  const bool has_x = g < M;
  for (int round = 0; round < a.rounds; ++round) {
    const int64_t blk = ((int64_t)round * gridDim.x + blockIdx.x) * rbr + rb_in;
    const int64_t r_lo = blk * 16 + g, r_hi = r_lo + 8;
    int acc[PB][4];
#pragma unroll
    for (int b = 0; b < PB; ++b) acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0;
    const int8_t* wlo[PB];
    const int8_t* whi[PB];
    const bool blk_ok = row_ptrs(round, wlo, whi);
    if (blk_ok) {
      for (int64_t p = p0; p < p1; p += U) {
        if (round > 0 || p > p0) load_batch(p, wlo, whi, lo, hi);
        uint4 xv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t c = (p + u) * 4 + t;
          const bool ok = (p + u) < p1 && c < nchunk;
          xv[u] = (ok && has_x) ? *reinterpret_cast<const uint4*>(xrow + c * 16) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int b = 0; b < PB; ++b) {
            mma_s8(acc[b], lo[u][b].x, hi[u][b].x, lo[u][b].y, hi[u][b].y, xv[u].x, xv[u].y);
            mma_s8(acc[b], lo[u][b].z, hi[u][b].z, lo[u][b].w, hi[u][b].w, xv[u].z, xv[u].w);
          }
      }
    }
    if (ksplit == 1) {
      if (blk_ok) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int m = 2 * t + (e & 1);
          const int64_t row = (e & 2) ? r_hi : r_lo;
          if (m < M && row < a.N) {
            float v = (float)acc[0][e] * xscale[m] * a.wscale[row];
            if (SWIGLU) v = silu_f(v) * ((float)acc[PB - 1][e] * xscale[m] * a.wscale[a.up_off + row]);
            if (a.push_site >= 0) tp_push_value(a.tp, a.push_site, (int64_t)m * a.N + row, v);
            else if (OUT_F32) reinterpret_cast<float*>(a.y)[(int64_t)m * a.ldy + row] = v;
            else reinterpret_cast<bf16*>(a.y)[(int64_t)m * a.ldy + row] = __float2bfloat16(v);
          }
        }
      }
    } else {
      float* pw = part + (((size_t)round * kW + warp) * PB) * 128;
#pragma unroll
      for (int b = 0; b < PB; ++b)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          pw[b * 128 + (g + ((e & 2) ? 8 : 0)) * 8 + 2 * t + (e & 1)] = (float)acc[b][e];
    }
  }
  if (ksplit > 1) {
    __syncthreads();
    const int per_round = rbr * 16 * 8;
    for (int idx = tid; idx < a.rounds * per_round; idx += kT) {
      const int round = idx / per_round, rem = idx % per_round;
      const int rb = rem / 128, r = (rem % 128) / 8, m = rem % 8;
      const int64_t row = (((int64_t)round * gridDim.x + blockIdx.x) * rbr + rb) * 16 + r;
      if (m >= M || row >= a.N) continue;
      float v = 0.f, v2 = 0.f;
      for (int s = 0; s < ksplit; ++s) {
        const float* pw = part + (((size_t)round * kW + rb * ksplit + s) * PB) * 128;
        v += pw[r * 8 + m];
        if (SWIGLU) v2 += pw[128 + r * 8 + m];
      }
      v *= xscale[m] * a.wscale[row];
      if (SWIGLU) v = silu_f(v) * (v2 * xscale[m] * a.wscale[a.up_off + row]);
      if (a.push_site >= 0) tp_push_value(a.tp, a.push_site, (int64_t)m * a.N + row, v);
      else if (OUT_F32) reinterpret_cast<float*>(a.y)[(int64_t)m * a.ldy + row] = v;
      else reinterpret_cast<bf16*>(a.y)[(int64_t)m * a.ldy + row] = __float2bfloat16(v);
    }
  }
}

int g_i8_sms = 0;

template <bool SWIGLU, bool NORM, bool OUT_F32>
int launch_i8(I8Args a, cudaStream_t st, int n_slots = 1) {
  if (!g_i8_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_i8_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_i8_sms <= 0) g_i8_sms = 148;
  }
  constexpr int PB = SWIGLU ? 2 : 1;
  const int64_t nblk = (a.N + 15) / 16;
  const int64_t npair = ((a.K >> 4) + 3) >> 2;
  // three CTAs per SM while their activations fit; several rows of a long K get fewer, larger shares
  size_t smem = 0;
  int64_t grid = 0;
  for (int per_sm = 3; per_sm >= 1; --per_sm) {
    const int64_t slots = std::max<int64_t>(1, (int64_t)g_i8_sms * per_sm / n_slots);
    int ks = 1;
    while (ks < kW && (nblk * ks + kW - 1) / kW < slots && npair / (ks * 2) >= 4) ks <<= 1;
    a.ksplit = ks;
    const int rbr = kW / ks;
    const int64_t units = (nblk + rbr - 1) / rbr;
    grid = units < slots ? units : slots;
    a.rounds = (int)((units + grid - 1) / grid);
    smem = (size_t)a.K * 2 + (((size_t)a.M * a.K + 15) & ~(size_t)15) + 32;
    if (ks > 1) smem += (size_t)a.rounds * kW * PB * 128 * sizeof(float);
    if ((smem + 2048) * per_sm <= (size_t)227 * 1024) break;
  }
  if (smem > 200 * 1024) return CB_ERR_SHAPE;
  auto kern = gemv_i8_kernel<SWIGLU, NORM, OUT_F32>;
  if (smem + 2048 > 48 * 1024) {   // the 48 KB default also has to hold the static shared memory
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cb_launch(kern, dim3((unsigned)grid, (unsigned)n_slots), dim3(kT), smem, st, a);
}

// Per-row dynamic int8 quantisation of bf16 activations (prefill side of W8A8):
// s = max(absmax, 1e-8) / 127; optional SwiGLU of a [M, 2I] input first.
__global__ void __launch_bounds__(256) quant_rows_kernel(const bf16* __restrict__ x, int64_t ldx, int8_t* __restrict__ q,
                                                          float* __restrict__ scale, int64_t K, int swiglu) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* row = reinterpret_cast<float*>(smem_raw);
  __shared__ float red[32];
  griddep_launch();
  griddep_wait();
  const int64_t r = blockIdx.x;
  float amax = 0.f;
  for (int64_t i = threadIdx.x; i < K; i += blockDim.x) {
    float v = __bfloat162float(x[r * ldx + i]);
    if (swiglu) v = __bfloat162float(__float2bfloat16(silu_f(v) * __bfloat162float(x[r * ldx + K + i])));
    row[i] = v;
    amax = fmaxf(amax, fabsf(v));
  }
  amax = block_max(amax, red);
  const float sc = fmaxf(amax, 1e-8f) / 127.f, inv = 1.f / sc;
  if (threadIdx.x == 0) scale[r] = sc;
  for (int64_t i = threadIdx.x; i < K; i += blockDim.x)
    q[r * K + i] = (int8_t)max(-127, min(127, __float2int_rn(row[i] * inv)));
}

// The same for rows whose length is a multiple of 8 and whose rows start on 16 bytes: 16-byte loads, 8-byte
// stores, two passes over the (cache-resident) row instead of a shared-memory copy.
__device__ __forceinline__ void quant_chunk(const bf16* xr, int64_t K, int64_t c, int swiglu, float* f) {
  bf16x8_to_float(*reinterpret_cast<const uint4*>(xr + c * 8), f);
  if (swiglu) {
    float u[8];
    bf16x8_to_float(*reinterpret_cast<const uint4*>(xr + K + c * 8), u);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = __bfloat162float(__float2bfloat16(silu_f(f[e]) * u[e]));
  }
}
__global__ void __launch_bounds__(256) quant_rows_vec_kernel(const bf16* __restrict__ x, int64_t ldx, int8_t* __restrict__ q,
                                                              float* __restrict__ scale, int64_t K, int swiglu) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  uint4* rowv = reinterpret_cast<uint4*>(smem_raw);        // the (SwiGLU'd) row as bf16, read once from memory
  __shared__ float red[32];
  griddep_launch();
  griddep_wait();
  const int64_t r = blockIdx.x, nchunk = K >> 3;
  const bf16* xr = x + r * ldx;
  float amax = 0.f;
  for (int64_t c = threadIdx.x; c < nchunk; c += blockDim.x) {
    float f[8];
    quant_chunk(xr, K, c, swiglu, f);
    rowv[c] = float_to_bf16x8(f);                          // exact: the values are bf16 already
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
  }
  amax = block_max(amax, red);
  const float sc = fmaxf(amax, 1e-8f) / 127.f, inv = 1.f / sc;
  if (threadIdx.x == 0) scale[r] = sc;
  for (int64_t c = threadIdx.x; c < nchunk; c += blockDim.x) {   // a thread reads back the chunks it wrote
    float f[8];
    bf16x8_to_float(rowv[c], f);
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int qi = max(-127, min(127, __float2int_rn(f[e] * inv)));
      w[e >> 2] |= (uint32_t)(qi & 0xff) << (8 * (e & 3));
    }
    *reinterpret_cast<uint2*>(q + r * K + c * 8) = make_uint2(w[0], w[1]);
  }
}

}  // namespace

// Same contract as cb_gemv_bf16 with int8 weights + per-row scales; K % 16 == 0.
CB_EXPORT int cb_gemv_i8(const void* W, const void* wscale, const void* x, void* y, int64_t M, int64_t N, int64_t K,
                         int64_t ldy, int64_t mode, int64_t up_off, const void* res_in, const void* add,
                         const void* gain, void* res_out, float eps, const void* tp, int64_t pull_site,
                         int64_t push_site, void* stream) {
  if (!W || !wscale || (!y && push_site < 0) || (!x && !res_in) || (res_in && !gain)) return CB_ERR_ARG;
  if ((pull_site >= 0 || push_site >= 0) && !tp) return CB_ERR_ARG;
  if (pull_site >= 0 && !res_in) return CB_ERR_ARG;
  if (K % 16 || M < 1 || M > 8 || N < 1) return CB_ERR_SHAPE;
  if (res_in && res_out && (res_out == res_in || res_out == add)) return CB_ERR_ARG;
  I8Args a{(const int8_t*)W, (const float*)wscale, (const bf16*)x, y, N, K, ldy, up_off, (const bf16*)res_in,
           (const bf16*)add, (const float*)gain, (bf16*)res_out, eps, (int)M, 1, 1, (int)pull_site, (int)push_site};
  if (tp) a.tp = *(const TpComm*)tp; else memset(&a.tp, 0, sizeof(a.tp));
  a.slot_expert = nullptr; a.slot_xrow = nullptr; a.expert_rows = 0;
  const bool sw = mode & 1, f32 = mode & 2, norm = res_in != nullptr;
  cudaStream_t st = (cudaStream_t)stream;
  if (sw) {
    if (f32) return CB_ERR_ARG;
    return norm ? launch_i8<true, true, false>(a, st) : launch_i8<true, false, false>(a, st);
  }
  if (f32) return norm ? launch_i8<false, true, true>(a, st) : launch_i8<false, false, true>(a, st);
  return norm ? launch_i8<false, true, false>(a, st) : launch_i8<false, false, false>(a, st);
}

// Routed experts from int8 stacks: slot s computes y[s, :] = (W[slot_expert[s]] x[slot_xrow[s], :]) with the
// activation row quantised in the prologue; W [E, rows, K] and wscale [E, rows] with rows = N (plain) or 2N
// (mode bit 0, SwiGLU: gate rows then up rows).  A negative expert index leaves the slot's output untouched.
CB_EXPORT int cb_moe_gemv_i8(const void* W, const void* wscale, const void* x, void* y, int64_t n_slots, int64_t N,
                             int64_t K, int64_t ldy, int64_t mode, const void* slot_expert, const void* slot_xrow,
                             void* stream) {
  if (!W || !wscale || !x || !y || !slot_expert) return CB_ERR_ARG;
  if (K % 16 || N < 1 || n_slots < 1 || n_slots > 65535) return CB_ERR_SHAPE;
  I8Args a{(const int8_t*)W, (const float*)wscale, (const bf16*)x, y, N, K, ldy, N, nullptr, nullptr, nullptr, nullptr,
           0.f, 1, 1, 1, -1, -1};
  memset(&a.tp, 0, sizeof(a.tp));
  a.slot_expert = (const int*)slot_expert; a.slot_xrow = (const int*)slot_xrow;
  a.expert_rows = (mode & 1) ? 2 * N : N;
  cudaStream_t st = (cudaStream_t)stream;
  if (mode & 1) return (mode & 2) ? CB_ERR_ARG : launch_i8<true, false, false>(a, st, (int)n_slots);
  return (mode & 2) ? launch_i8<false, false, true>(a, st, (int)n_slots) : launch_i8<false, false, false>(a, st, (int)n_slots);
}

CB_EXPORT int cb_quant_rows(const void* x, int64_t ldx, void* q, void* scale, int64_t M, int64_t K, int64_t swiglu,
                            void* stream) {
  if (M == 0) return 0;
  if (K % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)q & 7) == 0 && K * 2 <= 200 * 1024) {
    const size_t sv = (size_t)K * 2;
    if (sv + 2048 > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(quant_rows_vec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sv);
      if (e != cudaSuccess) return (int)e;
    }
    return (int)cb_launch(quant_rows_vec_kernel, dim3((unsigned)M), dim3(256), sv, (cudaStream_t)stream, (const bf16*)x, ldx,
                          (int8_t*)q, (float*)scale, K, (int)swiglu);
  }
  if (K * 4 > 200 * 1024) return CB_ERR_SHAPE;
  const size_t smem = (size_t)K * 4;
  if (smem + 2048 > 48 * 1024) {   // the 48 KB default also has to hold the static shared memory
    cudaError_t e = cudaFuncSetAttribute(quant_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cb_launch(quant_rows_kernel, dim3((unsigned)M), dim3(256), smem, (cudaStream_t)stream, (const bf16*)x, ldx,
                        (int8_t*)q, (float*)scale, K, (int)swiglu);
}
