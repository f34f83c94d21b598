// W4A8 decode projection (1..8 activation rows): 4-bit weights with one fp32 scale per group of
// 128 input channels, activations quantised per token to int8 in the prologue, products on the
// integer tensor cores.
//
// Storage read by the kernel (repacked once at load from the checkpoint's [K/2, N] layout):
//   Wq    [N, K/2] bytes, byte j of a row = code(k = 2j) | code(k = 2j + 1) << 4, code = q + 8 in 0..15
//   scale [N, K/128] fp32
// A warp owns 16 output rows and walks K one scale group at a time: the four lanes t = 0..3 of a row
// each load 16 bytes (32 codes), i.e. exactly the 128 channels of one group.  A 32-bit word splits
// into its even and odd nibbles with two masks - those two registers are used *as they are* as the
// A fragments of mma.m16n8k32.u8.s8: the k order inside the MMA is free as long as the activation
// (B operand) follows the same order, so the prologue stores the int8 activation in the order
// [k0 k2 k4 k6 k1 k3 k5 k7] per 8 channels and nothing is shuffled in the loop.  Codes stay unsigned;
// the "- 8" is applied per group as  sum(code * a) - 8 * sum(a)  with the group sums of the
// activation computed once in the prologue.  Each group's int32 result is scaled by its fp32 scale
// and accumulated in fp32; the token scale is applied at the end.
// One kernel serves the dense projections (fused residual add + RMSNorm prologue, SwiGLU epilogue)
// and the routed experts (slot mode: blockIdx.y selects (expert, activation row) as in gemv_mma.cu).
// A quarter of the bf16 bytes per token.  Replaces the reference's w4a8_dot / w4a8_finish pair and
// the grouped w4 expert kernels (backends/corex/kernels/w4a8.cu, moe_grouped_w4*.cu); format:
// tools/quant_disk_w4a8.py:45-89.
#include <string.h>
#include "common.cuh"

namespace {

constexpr int kW = 8, kT = kW * 32, kGroup = 128;

struct W4Args {
  const uint8_t* W; const float* wscale; const bf16* x; void* y;
  int64_t N, K, ldy, up_off;
  const bf16* res_in; const bf16* add; const float* gain; bf16* res_out;
  float eps;
  int M, ksplit, rounds;
  const int* slot_expert; const int* slot_xrow; int64_t expert_rows;   // slot mode: rows per expert (N or 2N)
};

__device__ __forceinline__ void mma_u8s8(int* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool SWIGLU, bool NORM, bool OUT_F32>
__global__ void __launch_bounds__(kT, 2) gemv_w4_kernel(const W4Args a_in) {
  constexpr int PB = SWIGLU ? 2 : 1;
  constexpr int U = SWIGLU ? 2 : 4;               // groups in flight per warp
  extern __shared__ __align__(16) unsigned char smem_raw[];
  W4Args a = a_in;
  if (a.slot_expert) {
    asm volatile("griddepcontrol.wait;" ::: "memory");      // routing tables come from the kernel just before
    const int slot = blockIdx.y, e = a.slot_expert[slot];
    if (e < 0) { cbtrace::stamp(0); cbtrace::stamp(1); return; }
    a.W += (int64_t)e * a.expert_rows * (a.K >> 1);
    a.wscale += (int64_t)e * a.expert_rows * (a.K / kGroup);
    a.x += (int64_t)(a.slot_xrow ? a.slot_xrow[slot] : slot) * a.K;
    a.y = OUT_F32 ? (void*)(reinterpret_cast<float*>(a.y) + (int64_t)slot * a.ldy)
                  : (void*)(reinterpret_cast<bf16*>(a.y) + (int64_t)slot * a.ldy);
  }
  const int64_t K = a.K;
  const int G = (int)(K / kGroup), M = a.M;
  const int64_t row_bytes = K >> 1;
  bf16* stage = reinterpret_cast<bf16*>(smem_raw);                                   // [K]
  int8_t* xq = reinterpret_cast<int8_t*>(smem_raw + (size_t)K * 2);                   // [M][K], permuted per 8
  int* asum = reinterpret_cast<int*>(smem_raw + (size_t)K * 2 + (size_t)M * K);       // [M][G]
  float* xscale = reinterpret_cast<float*>(asum + (size_t)M * G);                     // [8]
  float* part = xscale + 8;                                                           // [rounds][kW][PB][16][8]
  __shared__ float red[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int ksplit = a.ksplit, rbr = kW / ksplit;
  const int ks = warp % ksplit, rb_in = warp / ksplit;
  const int gper = (G + ksplit - 1) / ksplit;
  const int g0 = ks * gper, g1 = min(G, g0 + gper);       // this warp's scale groups

  auto row_ptrs = [&](int round, const uint8_t** wlo, const uint8_t** whi, int64_t* rlo, int64_t* rhi) -> bool {
    const int64_t blk = ((int64_t)round * gridDim.x + blockIdx.x) * rbr + rb_in;
    const int64_t r_lo = blk * 16 + g, r_hi = r_lo + 8;
#pragma unroll
    for (int b = 0; b < PB; ++b) {
      const int64_t off = b ? a.up_off : 0;
      rlo[b] = off + min(r_lo, a.N - 1);
      rhi[b] = off + min(r_hi, a.N - 1);
      wlo[b] = a.W + rlo[b] * row_bytes;
      whi[b] = a.W + rhi[b] * row_bytes;
    }
    return blk * 16 < a.N;
  };
  auto load_batch = [&](int gi, const uint8_t* const* wlo, const uint8_t* const* whi, uint4 (*lo)[PB], uint4 (*hi)[PB]) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool ok = gi + u < g1;
      const int64_t off = ((int64_t)(gi + u) * 4 + t) * 16;
#pragma unroll
      for (int b = 0; b < PB; ++b) {
        lo[u][b] = ok ? ld_stream(wlo[b] + off) : make_uint4(0, 0, 0, 0);
        hi[u][b] = ok ? ld_stream(whi[b] + off) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  griddep_launch();
  uint4 lo[U][PB], hi[U][PB];
  {
    const uint8_t* wlo[PB];
    const uint8_t* whi[PB];
    int64_t rlo[PB], rhi[PB];
    if (row_ptrs(0, wlo, whi, rlo, rhi) && g0 < g1) load_batch(g0, wlo, whi, lo, hi);
  }
  griddep_wait();

  // ---- prologue: (residual add + norm,) per-token int8 quantisation, permuted store, group sums ----
  for (int m = 0; m < M; ++m) {
    float ss = 0.f;
    for (int64_t c = tid; c < (K >> 3); c += kT) {
      float f[8], q[8];
      if (NORM) {
        bf16x8_to_float(*reinterpret_cast<const uint4*>(a.res_in + m * K + c * 8), f);
        if (a.add) {
          bf16x8_to_float(*reinterpret_cast<const uint4*>(a.add + m * K + c * 8), q);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i] + q[i]));
        }
        if (a.res_out && blockIdx.x == 0 && blockIdx.y == 0)
          *reinterpret_cast<uint4*>(a.res_out + m * K + c * 8) = float_to_bf16x8(f);
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
      if (NORM) v = __bfloat162float(__float2bfloat16(v * rstd * a.gain[i]));
      stage[i] = __float2bfloat16(v);
      amax = fmaxf(amax, fabsf(v));
    }
    amax = block_max(amax, red);
    const float sc = fmaxf(amax, 1e-8f) / 127.f, inv = 1.f / sc;
    if (tid == 0) xscale[m] = sc;
    for (int64_t i = tid; i < K; i += kT) {
      const int j = (int)(i & 7);
      const int64_t dst = (i & ~(int64_t)7) + ((j & 1) ? 4 + (j >> 1) : (j >> 1));     // evens first, then odds
      xq[m * K + dst] = (int8_t)max(-127, min(127, __float2int_rn(__bfloat162float(stage[i]) * inv)));
    }
    __syncthreads();
    for (int gi = tid; gi < G; gi += kT) {
      const int* w = reinterpret_cast<const int*>(xq + m * K + (int64_t)gi * kGroup);
      int s = 0;
#pragma unroll 8
      for (int i = 0; i < kGroup / 4; ++i) s = __dp4a(w[i], 0x01010101, s);
      asum[m * G + gi] = s;
    }
    __syncthreads();
  }

  const int8_t* xrow = xq + (int64_t)g * K;
  const bool has_x = g < M;
  const int m0 = 2 * t, m1 = 2 * t + 1;
  for (int round = 0; round < a.rounds; ++round) {
    const int64_t blk = ((int64_t)round * gridDim.x + blockIdx.x) * rbr + rb_in;
    const int64_t r_lo = blk * 16 + g, r_hi = r_lo + 8;
    float facc[PB][4];
#pragma unroll
    for (int b = 0; b < PB; ++b) facc[b][0] = facc[b][1] = facc[b][2] = facc[b][3] = 0.f;
    const uint8_t* wlo[PB];
    const uint8_t* whi[PB];
    int64_t rlo[PB], rhi[PB];
    const bool blk_ok = row_ptrs(round, wlo, whi, rlo, rhi);
    if (blk_ok) {
      for (int gi = g0; gi < g1; gi += U) {
        if (round > 0 || gi > g0) load_batch(gi, wlo, whi, lo, hi);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (gi + u >= g1) break;
          uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
          if (has_x) {
            const uint4* xp = reinterpret_cast<const uint4*>(xrow + (int64_t)(gi + u) * kGroup + t * 32);
            x0 = xp[0];
            x1 = xp[1];
          }
          const int s0 = m0 < M ? asum[m0 * G + gi + u] : 0, s1 = m1 < M ? asum[m1 * G + gi + u] : 0;
#pragma unroll
          for (int b = 0; b < PB; ++b) {
            int acc[4] = {0, 0, 0, 0};
            const uint32_t wl[4] = {lo[u][b].x, lo[u][b].y, lo[u][b].z, lo[u][b].w};
            const uint32_t wh[4] = {hi[u][b].x, hi[u][b].y, hi[u][b].z, hi[u][b].w};
            const uint32_t xb[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
              mma_u8s8(acc, wl[i] & 0x0F0F0F0Fu, wh[i] & 0x0F0F0F0Fu, (wl[i] >> 4) & 0x0F0F0F0Fu,
                       (wh[i] >> 4) & 0x0F0F0F0Fu, xb[2 * i], xb[2 * i + 1]);
            const float sl = a.wscale[rlo[b] * G + gi + u], sh = a.wscale[rhi[b] * G + gi + u];
            facc[b][0] = fmaf((float)(acc[0] - 8 * s0), sl, facc[b][0]);
            facc[b][1] = fmaf((float)(acc[1] - 8 * s1), sl, facc[b][1]);
            facc[b][2] = fmaf((float)(acc[2] - 8 * s0), sh, facc[b][2]);
            facc[b][3] = fmaf((float)(acc[3] - 8 * s1), sh, facc[b][3]);
          }
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
            float v = facc[0][e] * xscale[m];
            if (SWIGLU) v = silu_f(v) * (facc[PB - 1][e] * xscale[m]);
            if (OUT_F32) reinterpret_cast<float*>(a.y)[(int64_t)m * a.ldy + row] = v;
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
          pw[b * 128 + (g + ((e & 2) ? 8 : 0)) * 8 + 2 * t + (e & 1)] = facc[b][e];
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
      v *= xscale[m];
      if (SWIGLU) v = silu_f(v) * (v2 * xscale[m]);
      if (OUT_F32) reinterpret_cast<float*>(a.y)[(int64_t)m * a.ldy + row] = v;
      else reinterpret_cast<bf16*>(a.y)[(int64_t)m * a.ldy + row] = __float2bfloat16(v);
    }
  }
}

int g_w4_sms = 0;

template <bool SWIGLU, bool NORM, bool OUT_F32>
int launch_w4(W4Args a, cudaStream_t st, int n_slots) {
  if (!g_w4_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_w4_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_w4_sms <= 0) g_w4_sms = 148;
  }
  constexpr int PB = SWIGLU ? 2 : 1;
  const int G = (int)(a.K / kGroup);
  const int64_t nblk = (a.N + 15) / 16;
  // two CTAs per SM while their activations fit; several rows of a long K get one
  size_t smem = 0;
  int64_t grid = 0;
  for (int per_sm = 2; per_sm >= 1; --per_sm) {
    const int64_t slots = std::max<int64_t>(1, (int64_t)g_w4_sms * per_sm / n_slots);
    int ks = 1;
    while (ks < kW && (nblk * ks + kW - 1) / kW < slots && G / (ks * 2) >= 1) ks <<= 1;
    a.ksplit = ks;
    const int rbr = kW / ks;
    const int64_t units = (nblk + rbr - 1) / rbr;
    grid = units < slots ? units : slots;
    a.rounds = (int)((units + grid - 1) / grid);
    smem = (size_t)a.K * 2 + (size_t)a.M * a.K + (size_t)a.M * G * 4 + 32;
    if (ks > 1) smem += (size_t)a.rounds * kW * PB * 128 * sizeof(float);
    if ((smem + 2048) * per_sm <= (size_t)227 * 1024) break;
  }
  if (smem > 200 * 1024) return CB_ERR_SHAPE;
  auto kern = gemv_w4_kernel<SWIGLU, NORM, OUT_F32>;
  if (smem + 2048 > 48 * 1024) {   // the 48 KB default also has to hold the static shared memory
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cb_launch(kern, dim3((unsigned)grid, (unsigned)n_slots), dim3(kT), smem, st, a);
}

template <bool NORM>
int dispatch_w4(const W4Args& a, int64_t mode, cudaStream_t st, int n_slots) {
  const bool sw = mode & 1, f32 = mode & 2;
  if (sw) return f32 ? CB_ERR_ARG : launch_w4<true, NORM, false>(a, st, n_slots);
  return f32 ? launch_w4<false, NORM, true>(a, st, n_slots) : launch_w4<false, NORM, false>(a, st, n_slots);
}

}  // namespace

// y[M, N] = dequant(Wq)[N, K] x[M, K]  (mode bit 0: SwiGLU over gate rows [0, N) / up rows [up_off, up_off + N);
// bit 1: fp32 output).  K % 128 == 0.
CB_EXPORT int cb_gemv_w4(const void* Wq, const void* wscale, const void* x, void* y, int64_t M, int64_t N, int64_t K,
                         int64_t ldy, int64_t mode, int64_t up_off, const void* res_in, const void* add,
                         const void* gain, void* res_out, float eps, void* stream) {
  if (!Wq || !wscale || !y || (!x && !res_in) || (res_in && !gain)) return CB_ERR_ARG;
  if (K % kGroup || M < 1 || M > 8 || N < 1) return CB_ERR_SHAPE;
  W4Args a;
  a.W = (const uint8_t*)Wq; a.wscale = (const float*)wscale; a.x = (const bf16*)x; a.y = y;
  a.N = N; a.K = K; a.ldy = ldy; a.up_off = up_off;
  a.res_in = (const bf16*)res_in; a.add = (const bf16*)add; a.gain = (const float*)gain; a.res_out = (bf16*)res_out;
  a.eps = eps; a.M = (int)M; a.ksplit = 1; a.rounds = 1;
  a.slot_expert = nullptr; a.slot_xrow = nullptr; a.expert_rows = 0;
  cudaStream_t st = (cudaStream_t)stream;
  return res_in ? dispatch_w4<true>(a, mode, st, 1) : dispatch_w4<false>(a, mode, st, 1);
}

// Routed experts: slot s computes y[s, :] = dequant(Wq[slot_expert[s]]) x[slot_xrow[s], :];
// Wq [E, rows, K/2] and wscale [E, rows, K/128] with rows = N (plain) or 2N (SwiGLU: gate rows then up rows).
CB_EXPORT int cb_moe_gemv_w4(const void* Wq, const void* wscale, const void* x, void* y, int64_t n_slots, int64_t N,
                             int64_t K, int64_t ldy, int64_t mode, const void* slot_expert, const void* slot_xrow,
                             void* stream) {
  if (!Wq || !wscale || !x || !y || !slot_expert) return CB_ERR_ARG;
  if (K % kGroup || N < 1 || n_slots < 1 || n_slots > 65535) return CB_ERR_SHAPE;
  W4Args a;
  a.W = (const uint8_t*)Wq; a.wscale = (const float*)wscale; a.x = (const bf16*)x; a.y = y;
  a.N = N; a.K = K; a.ldy = ldy; a.up_off = N;
  a.res_in = nullptr; a.add = nullptr; a.gain = nullptr; a.res_out = nullptr; a.eps = 0.f; a.M = 1;
  a.ksplit = 1; a.rounds = 1;
  a.slot_expert = (const int*)slot_expert; a.slot_xrow = (const int*)slot_xrow;
  a.expert_rows = (mode & 1) ? 2 * N : N;
  return dispatch_w4<false>(a, mode, (cudaStream_t)stream, (int)n_slots);
}

// ---- dequantisation to bf16 (prefill runs the bf16 tcgen05 GEMM on the expanded tile) ------------
namespace {
__global__ void __launch_bounds__(256) w4_dequant_kernel(const uint8_t* __restrict__ Wq, const float* __restrict__ scale,
                                                         bf16* __restrict__ out, int64_t N, int64_t K) {
  griddep_launch();
  griddep_wait();
  const int64_t half = K >> 1, G = K / kGroup;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < N * (half >> 2); i += (int64_t)gridDim.x * 256) {
    const int64_t row = i / (half >> 2), w = i % (half >> 2);       // word w of the row = 8 codes
    const uint32_t v = reinterpret_cast<const uint32_t*>(Wq + row * half)[w];
    const float s = scale[row * G + (w * 8) / kGroup];
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t byte = (v >> (8 * j)) & 0xffu;
      f[2 * j] = (float)((int)(byte & 15u) - 8) * s;
      f[2 * j + 1] = (float)((int)(byte >> 4) - 8) * s;
    }
    *reinterpret_cast<uint4*>(out + row * K + w * 8) = float_to_bf16x8(f);
  }
}
}  // namespace

CB_EXPORT int cb_w4_dequant(const void* Wq, const void* wscale, void* out, int64_t N, int64_t K, void* stream) {
  if (K % kGroup || N < 1) return CB_ERR_SHAPE;
  const int64_t work = N * (K >> 3);
  const unsigned grid = (unsigned)std::min<int64_t>((work + 255) / 256, 148 * 8);
  return (int)cb_launch(w4_dequant_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (const uint8_t*)Wq,
                        (const float*)wscale, (bf16*)out, N, K);
}
