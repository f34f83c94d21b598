// Decode projection (1..8 activation rows) with the dot products on the tensor cores.
//
// Profiling the scalar GEMVs showed them instruction-bound, not memory-bound: unpacking bf16 and
// issuing one FMA per element costs ~4 instructions per weight element, and at 6.5 TB/s the SMs
// cannot issue that many.  Here a warp owns 16 weight rows and feeds them to mma.m16n8k16 as the
// A operand straight from its 16-byte global loads: lane (g, t) loads chunk 4j+t of rows g and g+8,
// which are exactly its A fragments for two MMAs if the k index is permuted the same way for the
// B operand - and B is the activation, read from shared memory with the same permutation.  The 8
// columns of B are the (up to) 8 batch rows, so one kernel serves M = 1..8 at the same cost:
// ~0.5 instructions per weight element.  The kernel keeps the fused prologue (residual add +
// RMSNorm, or the tensor-parallel pull-sum) and epilogues (SwiGLU, fp32 logits, tensor-parallel
// push) of gemv.cu, the K-split for narrow outputs and the grid-wide sweep order.
#include <string.h>
#include "tp.cuh"

namespace {

constexpr int kW = 8, kT = kW * 32;
constexpr int kU = 4;   // k-step pairs (32 elements each) in flight per lane

struct MmaArgs {
  const bf16* W; const bf16* x; void* y;
  int64_t N, K, ldy, up_off;
  const bf16* res_in; const bf16* add; const float* gain; bf16* res_out;
  float eps;
  int M;              // activation rows (1..8)
  int ksplit;         // k-slices per 16-row block (a power of two <= 8)
  int rounds;         // rounds of the grid-wide sweep
  int pull_site, push_site;
  int pf_rounds;      // sweep rounds whose weights are requested into L2 before the dependency wait
  int64_t xs_ld;      // activation elements staged per row (K, or this CTA's K slice)
  int stage_batches;  // weight batches per warp copied into shared memory ahead of the dependency wait
  int kcta;           // CTAs that share one 16-row block, each with its own k range (1: none; then ksplit == 8)
  float* ws; unsigned* tickets;   // cross-CTA partial sums [unit][kcta][2][128] and arrival counters [unit]
  // grouped (mixture-of-experts) mode: blockIdx.y is a slot; slot s multiplies activation row
  // slot_xrow[s] by the weights of expert slot_expert[s] and writes output row s.  M must be 1.
  const int* slot_expert; const int* slot_xrow; int64_t expert_stride;
  // fused consumer of a pushing projection (tensor parallel): the last CTA of the grid to finish pulls the
  // ranks' sums of push_site for every row, adds tail_res_in, stores the new residual in tail_res_out and
  // its RMSNorm (gain tail_gain) in tail_out - what a separate pull kernel would do one launch later
  const bf16* tail_res_in; const float* tail_gain; bf16* tail_res_out; bf16* tail_out; float tail_eps;
  TpComm tp;
};

__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Scratch of the cross-CTA K split: a projection with few output rows (2560 x 9216, say) has too few
// 16-row blocks to fill the SMs with one CTA per block, and a CTA alone keeps only ~32 KB in flight,
// so its time is set by memory latency, not bandwidth.  Up to kMaxKcta CTAs then share a block, each
// streaming a slice of K; they leave fp32 partial sums here and the last one to arrive (ticket)
// adds them in slice order and runs the epilogue, so the result does not depend on arrival order.
// One decode stream per process uses this scratch at a time (kernels of one stream are ordered).
constexpr int kMaxKcta = 4, kMaxSplitUnits = 2048;
__device__ float g_split_ws[(size_t)kMaxSplitUnits * kMaxKcta * 2 * 128];
__device__ unsigned g_split_tickets[kMaxSplitUnits];

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all_() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <bool SWIGLU, bool NORM, bool OUT_F32>
__global__ void __launch_bounds__(kT, 3) gemv_mma_kernel(const MmaArgs a_in) {
  constexpr int PB = SWIGLU ? 2 : 1;   // physical 16-row blocks per unit (gate, up)
  constexpr int U = SWIGLU ? 2 : kU;   // same number of loads in flight either way
  extern __shared__ __align__(16) unsigned char smem_raw[];
  MmaArgs a = a_in;
  if (a.slot_expert) {
    // the routing tables come from the kernels just before this one: wait before reading them
    // (the second wait below is then a no-op)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int slot = blockIdx.y;
    if (a.slot_expert[slot] < 0) {                // expert owned by another rank
      cbtrace::stamp(0);
      cbtrace::stamp(1);
      return;
    }
    a.W += (int64_t)a.slot_expert[slot] * a.expert_stride;
    a.x += (int64_t)(a.slot_xrow ? a.slot_xrow[slot] : slot) * a.K;
    a.y = OUT_F32 ? (void*)(reinterpret_cast<float*>(a.y) + (int64_t)slot * a.ldy)
                  : (void*)(reinterpret_cast<bf16*>(a.y) + (int64_t)slot * a.ldy);
  }
  const int64_t K = a.K, nchunk = K >> 3;
  const int M = a.M;
  // A CTA that shares its row block with other CTAs (cross-CTA K split) only ever multiplies its own
  // K slice: without a norm prologue (which needs whole rows) it stages just that slice, xs_ld
  // elements per row starting at chunk xs_c0.  Fewer bytes per CTA keep more CTAs resident when
  // several activation rows times a long K would otherwise fill the shared memory.
  const int64_t xs_ld = a.xs_ld, xs_c0 = a.xs_ld == K ? 0 : (int64_t)(blockIdx.x % a.kcta) * (a.xs_ld >> 3);
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);                                  // [M][xs_ld]
  float* part = reinterpret_cast<float*>(smem_raw + (((size_t)M * xs_ld * 2 + 15) & ~(size_t)15));  // [rounds][warps][PB][16][8]
  const int nT = blockDim.x, nW = nT >> 5;                  // the CTA has ksplit * (row blocks per round) warps
  // per-warp staging area behind the partial sums: [batch][u][b][lo|hi][lane] 16-byte vectors
  constexpr int kBatchVecs = U * PB * 2;                     // vectors per lane per batch
  uint4* stage = reinterpret_cast<uint4*>(
      smem_raw + (((size_t)M * xs_ld * 2 + 15) & ~(size_t)15) +
      (a_in.ksplit > 1 ? (size_t)a_in.rounds * nW * PB * 128 * sizeof(float) : 0)) +
      (size_t)(threadIdx.x >> 5) * a_in.stage_batches * kBatchVecs * 32;
  __shared__ float red[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int ksplit = a.ksplit, rbr = nW / ksplit;          // row blocks per CTA round
  const int ks = warp % ksplit, rb_in = warp / ksplit;
  const int kcta = a.kcta;
  const int unit_id = kcta > 1 ? blockIdx.x / kcta : blockIdx.x;   // which row-block unit this CTA works on
  const int kc = kcta > 1 ? blockIdx.x % kcta : 0;
  const unsigned unit_stride = kcta > 1 ? gridDim.x / kcta : gridDim.x;
  // k range of this warp in units of 4 chunks (one MMA pair)
  const int64_t npair = (nchunk + 3) >> 2;
  const int64_t pper = (npair + (int64_t)ksplit * kcta - 1) / ((int64_t)ksplit * kcta);
  const int64_t p0 = ((int64_t)kc * ksplit + ks) * pper, p1 = min(npair, p0 + pper);

  // Weights do not depend on the previous kernel: request this warp's first batch of round 0 into
  // registers before waiting on the producer of the activations, so that (under programmatic
  // dependent launch) the HBM stream of this projection starts during the previous kernel's tail and
  // runs through the norm prologue below.
  auto row_ptrs = [&](int round, const bf16** wlo, const bf16** whi) -> bool {
    const int64_t blk = ((int64_t)round * unit_stride + unit_id) * rbr + rb_in;
    const int64_t r_lo = blk * 16 + g, r_hi = r_lo + 8;
#pragma unroll
    for (int b = 0; b < PB; ++b) {
      const int64_t off = b ? a.up_off : 0;
      wlo[b] = a.W + (off + min(r_lo, a.N - 1)) * K;
      whi[b] = a.W + (off + min(r_hi, a.N - 1)) * K;
    }
    return blk * 16 < a.N;
  };
  auto load_batch = [&](int64_t p, const bf16* const* wlo, const bf16* const* whi, uint4 (*lo)[PB], uint4 (*hi)[PB]) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t c = (p + u) * 4 + t;
      const bool ok = (p + u) < p1 && c < nchunk;
#pragma unroll
      for (int b = 0; b < PB; ++b) {
        lo[u][b] = ok ? ld_stream(wlo[b] + c * 8) : make_uint4(0, 0, 0, 0);
        hi[u][b] = ok ? ld_stream(whi[b] + c * 8) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  // The batches after the first go to this warp's staging area with cp.async (no registers held),
  // each lane copying exactly the vectors it will read back, so no cross-lane synchronisation is
  // needed - only the lane's own cp.async completion.
  auto stage_batch = [&](int sb, int64_t p, const bf16* const* wlo, const bf16* const* whi) {
    uint4* dst = stage + (size_t)sb * kBatchVecs * 32 + lane;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t c = (p + u) * 4 + t;
      const bool ok = (p + u) < p1 && c < nchunk;
#pragma unroll
      for (int b = 0; b < PB; ++b) {
        if (ok) {
          cp_async16(dst + ((u * PB + b) * 2 + 0) * 32, wlo[b] + c * 8);
          cp_async16(dst + ((u * PB + b) * 2 + 1) * 32, whi[b] + c * 8);
        }
      }
    }
  };
  auto unstage_batch = [&](int sb, int64_t p, uint4 (*lo)[PB], uint4 (*hi)[PB]) {
    const uint4* src = stage + (size_t)sb * kBatchVecs * 32 + lane;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t c = (p + u) * 4 + t;
      const bool ok = (p + u) < p1 && c < nchunk;
#pragma unroll
      for (int b = 0; b < PB; ++b) {
        lo[u][b] = ok ? src[((u * PB + b) * 2 + 0) * 32] : make_uint4(0, 0, 0, 0);
        hi[u][b] = ok ? src[((u * PB + b) * 2 + 1) * 32] : make_uint4(0, 0, 0, 0);
      }
    }
  };
  griddep_launch();
  uint4 lo[U][PB], hi[U][PB];
  {
    const bf16* wlo[PB];
    const bf16* whi[PB];
    if (row_ptrs(0, wlo, whi) && p0 < p1) {
      load_batch(p0, wlo, whi, lo, hi);
      for (int sb = 0; sb < a.stage_batches; ++sb) {
        const int64_t p = p0 + (int64_t)(sb + 1) * U;
        if (p < p1) stage_batch(sb, p, wlo, whi);
      }
    }
    cp_async_commit();
  }
  // The rows a CTA sweeps in one round are contiguous in memory: ask the L2 for them with one bulk
  // prefetch per (round, gate/up half), still before the wait.  Under programmatic dependent launch
  // this CTA is resident long before its activations exist, so the HBM stream of this projection
  // fills the bubbles (prologue, tail, launch gap) of the projection running ahead of it.
  if (tid < a.pf_rounds * PB) {
    const int round = tid / PB, b = tid % PB;
    const int64_t row0 = ((int64_t)round * unit_stride + unit_id) * rbr * 16;
    if (row0 < a.N) {
      const int64_t rows = min((int64_t)rbr * 16, a.N - row0);
      const bf16* src = a.W + ((b ? a.up_off : 0) + row0) * K;
      const uint32_t bytes = (uint32_t)(rows * K * 2);
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
    }
  }
  griddep_wait();

  // ---- prologue: activation rows into shared memory ------------------------------------------
  if (NORM) {
    for (int m = 0; m < M; ++m) {
      float ss = 0.f;
      for (int64_t c = tid; c < nchunk; c += nT) {
        float f[8], q[8];
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
        const uint4 packed = float_to_bf16x8(f);
        *reinterpret_cast<uint4*>(xs + m * K + c * 8) = packed;
        if (a.res_out && blockIdx.x == 0) *reinterpret_cast<uint4*>(a.res_out + m * K + c * 8) = packed;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
      }
      const float rstd = rsqrtf(block_sum(ss, red) / (float)K + a.eps);
      for (int64_t c = tid; c < nchunk; c += nT) {
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
    const int64_t lc = xs_ld >> 3;                     // chunks staged per row
    // asynchronous 16-byte copies: a thread's share (tens of chunks when several rows are staged) is
    // in flight at once instead of one L2 round trip per chunk
    if ((int64_t)M * lc > 4 * nT) {
      for (int64_t i = tid; i < (int64_t)M * lc; i += nT) {
        const int64_t m = i / lc, c = xs_c0 + i % lc;
        if (c < nchunk) cp_async16(xs + i * 8, a.x + (m * nchunk + c) * 8);
      }
      cp_async_commit();
      cp_async_wait_all_();
    } else {
      for (int64_t i = tid; i < (int64_t)M * lc; i += nT) {
        const int64_t m = i / lc, c = xs_c0 + i % lc;
        if (c < nchunk) *reinterpret_cast<uint4*>(xs + i * 8) = *reinterpret_cast<const uint4*>(a.x + (m * nchunk + c) * 8);
      }
    }
  }
  __syncthreads();

  const bf16* xrow = xs + (int64_t)g * xs_ld - xs_c0 * 8;   // batch row g supplies column g of the B operand; indexed by global chunk
  const bool has_x = g < M;

  for (int round = 0; round < a.rounds; ++round) {
    const int64_t blk = ((int64_t)round * unit_stride + unit_id) * rbr + rb_in;   // 16-row block index
    const int64_t r_lo = blk * 16 + g, r_hi = r_lo + 8;
    float acc[PB][4];
#pragma unroll
    for (int b = 0; b < PB; ++b) acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.f;
    const bf16* wlo[PB];
    const bf16* whi[PB];
    const bool blk_ok = row_ptrs(round, wlo, whi);
    if (blk_ok) {
      for (int64_t p = p0; p < p1; p += U) {
        const int64_t bi = (p - p0) / U;                            // batch number within this warp's slice
        if (round == 0 && bi >= 1 && bi <= a.stage_batches) {
          if (bi == 1) cp_async_wait_all_();
          unstage_batch((int)bi - 1, p, lo, hi);
        } else if (round > 0 || bi > 0) {
          load_batch(p, wlo, whi, lo, hi);                          // batch 0 of round 0 is already in registers
        }
        uint4 xv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int64_t c = (p + u) * 4 + t;
          const bool ok = (p + u) < p1 && c < nchunk;
          xv[u] = (ok && has_x) ? *reinterpret_cast<const uint4*>(xrow + c * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int b = 0; b < PB; ++b) {
            mma16816(acc[b], lo[u][b].x, hi[u][b].x, lo[u][b].y, hi[u][b].y, xv[u].x, xv[u].y);
            mma16816(acc[b], lo[u][b].z, hi[u][b].z, lo[u][b].w, hi[u][b].w, xv[u].z, xv[u].w);
          }
      }
    }
    // acc[b][0..1]: (row g, batch rows 2t, 2t+1); acc[b][2..3]: (row g+8, same batch rows)
    if (ksplit == 1) {
      if (blk_ok) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int m = 2 * t + (e & 1);
          const int64_t row = (e & 2) ? r_hi : r_lo;
          if (m < M && row < a.N) {
            float v = acc[0][e];
            if (SWIGLU) v = silu_f(v) * acc[PB - 1][e];
            if (a.push_site >= 0) tp_push_value(a.tp, a.push_site, (int64_t)m * a.N + row, v);
            else if (OUT_F32) reinterpret_cast<float*>(a.y)[(int64_t)m * a.ldy + row] = v;
            else reinterpret_cast<bf16*>(a.y)[(int64_t)m * a.ldy + row] = __float2bfloat16(v);
          }
        }
      }
    } else {
      float* pw = part + (((size_t)round * nW + warp) * PB) * 128;
#pragma unroll
      for (int b = 0; b < PB; ++b)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          pw[b * 128 + (g + ((e & 2) ? 8 : 0)) * 8 + 2 * t + (e & 1)] = acc[b][e];
    }
  }
  if (ksplit > 1) {
    __syncthreads();
    if (kcta > 1) {
      // cross-CTA split (one round, one row block per CTA): publish this CTA's slice sums, take a
      // ticket; the last CTA of the block re-reads all slices in order
      float* mine = a.ws + ((size_t)unit_id * kMaxKcta + kc) * 256;
      for (int idx = tid; idx < PB * 128; idx += nT) {
        float v = 0.f;
        for (int s = 0; s < ksplit; ++s) v += part[((size_t)s * PB + idx / 128) * 128 + idx % 128];
        __stcg(mine + idx, v);
      }
      __shared__ bool last;
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        last = atomicAdd(a.tickets + unit_id, 1u) == (unsigned)kcta - 1;
        if (last) a.tickets[unit_id] = 0;
      }
      __syncthreads();
      if (last) {
        __threadfence();
        const float* all = a.ws + (size_t)unit_id * kMaxKcta * 256;
        for (int idx = tid; idx < 128; idx += nT) {
          const int r = idx / 8, m = idx % 8;
          const int64_t row = (int64_t)unit_id * 16 + r;
          if (m >= M || row >= a.N) continue;
          float v = 0.f, v2 = 0.f;
          for (int c = 0; c < kcta; ++c) {
            v += __ldcg(all + c * 256 + idx);
            if (SWIGLU) v2 += __ldcg(all + c * 256 + 128 + idx);
          }
          if (SWIGLU) v = silu_f(v) * v2;
          if (a.push_site >= 0) tp_push_value(a.tp, a.push_site, (int64_t)m * a.N + row, v);
          else if (OUT_F32) reinterpret_cast<float*>(a.y)[(int64_t)m * a.ldy + row] = v;
          else reinterpret_cast<bf16*>(a.y)[(int64_t)m * a.ldy + row] = __float2bfloat16(v);
        }
      }
    } else {
    // one thread per (round, row block of the round, row in block, batch row): fixed-order sum over k-slices
    const int per_round = rbr * 16 * 8;
    for (int idx = tid; idx < a.rounds * per_round; idx += nT) {
      const int round = idx / per_round, rem = idx % per_round;
      const int rb = rem / 128, r = (rem % 128) / 8, m = rem % 8;
      const int64_t row = (((int64_t)round * gridDim.x + blockIdx.x) * rbr + rb) * 16 + r;
      if (m >= M || row >= a.N) continue;
      float v = 0.f, v2 = 0.f;
      for (int s = 0; s < ksplit; ++s) {
        const float* pw = part + (((size_t)round * nW + rb * ksplit + s) * PB) * 128;
        v += pw[r * 8 + m];
        if (SWIGLU) v2 += pw[128 + r * 8 + m];
      }
      if (SWIGLU) v = silu_f(v) * v2;
      if (a.push_site >= 0) tp_push_value(a.tp, a.push_site, (int64_t)m * a.N + row, v);
      else if (OUT_F32) reinterpret_cast<float*>(a.y)[(int64_t)m * a.ldy + row] = v;
      else reinterpret_cast<bf16*>(a.y)[(int64_t)m * a.ldy + row] = __float2bfloat16(v);
    }
    }
  }
  // ---- fused consumer: the last CTA to finish does the pull + residual add + RMSNorm of the rows --------
  // Every rank's partial sums travel as {value, epoch} pairs, this rank's own included, so the CTA needs
  // no fence: it polls (bounded) until every pair of the site carries this step's epoch.  The arithmetic
  // is the one of tp_pull_norm_kernel (comm.cu); two passes over the row instead of a row buffer.
  if (a.tail_out != nullptr) {
    __shared__ bool grid_last;
    __syncthreads();
    if (tid == 0) {
      unsigned* ticket = a.tp.arrive + a.push_site;
      grid_last = atomicAdd(ticket, 1u) == gridDim.x * gridDim.y - 1;
      if (grid_last) *ticket = 0;
    }
    __syncthreads();
    if (grid_last) {
      const int64_t W = a.N, wch = W >> 3;
      for (int m = 0; m < M; ++m) {
        float ss = 0.f;
        for (int64_t c = tid; c < wch; c += nT) {
          float f[8], pulled[8];
          bf16x8_to_float(*reinterpret_cast<const uint4*>(a.tail_res_in + m * W + c * 8), f);
          tp_pull8(a.tp, a.push_site, m * W + c * 8, pulled);
#pragma unroll
          for (int i = 0; i < 8; ++i) { f[i] = __bfloat162float(__float2bfloat16(f[i] + pulled[i])); ss += f[i] * f[i]; }
          *reinterpret_cast<uint4*>(a.tail_res_out + m * W + c * 8) = float_to_bf16x8(f);
        }
        const float rstd = rsqrtf(block_sum(ss, red) / (float)W + a.tail_eps);
        for (int64_t c = tid; c < wch; c += nT) {          // each thread re-reads the chunks it wrote
          float f[8];
          bf16x8_to_float(*reinterpret_cast<const uint4*>(a.tail_res_out + m * W + c * 8), f);
          const float4 g0 = *reinterpret_cast<const float4*>(a.tail_gain + c * 8);
          const float4 g1 = *reinterpret_cast<const float4*>(a.tail_gain + c * 8 + 4);
          f[0] *= rstd * g0.x; f[1] *= rstd * g0.y; f[2] *= rstd * g0.z; f[3] *= rstd * g0.w;
          f[4] *= rstd * g1.x; f[5] *= rstd * g1.y; f[6] *= rstd * g1.z; f[7] *= rstd * g1.w;
          *reinterpret_cast<uint4*>(a.tail_out + m * W + c * 8) = float_to_bf16x8(f);
        }
      }
    }
  }
}

int g_mma_sms = 0;
int g_mma_ctas = 3;
int g_mma_pf_rounds = 0;
int g_mma_kcta_max = 4;
int g_mma_stage = 0;   // measured: staging through shared memory is slower than the register batches alone

template <bool SWIGLU, bool NORM, bool OUT_F32>
int launch_mma(MmaArgs a, cudaStream_t st, int n_slots = 1) {
  if (!g_mma_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_mma_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_mma_sms <= 0) g_mma_sms = 148;
  }
  constexpr int PB = SWIGLU ? 2 : 1;
  const int64_t nblk = (a.N + 15) / 16;
  const int64_t npair = ((a.K >> 3) + 3) >> 2;
  // Work is cut so that every resident warp gets the same amount and everything is resident at
  // once (one wave): a warp task is one 16-row block times one K slice.
  //  * few blocks: S = ks * kcta slices per block, ks warps of one CTA times kcta CTAs (cross-CTA sum);
  //  * more blocks than that but fewer than warp slots: one CTA of ks warps per block;
  //  * more blocks than warp slots (vocabulary head): 8-warp CTAs sweep whole blocks in rounds,
  //    the grid sized so that every CTA runs the same number of rounds.
  const int warps_sm = 25;                                      // 80 registers per thread
  // elements of a row that a CTA stages when kc CTAs share a block and each has w K-slice warps
  auto slice_ld = [&](int w, int kc) -> int64_t {
    if (NORM || kc <= 1) return a.K;
    const int64_t pper = (npair + (int64_t)w * kc - 1) / ((int64_t)w * kc);
    const int64_t ld = pper * w * 32;
    return ld < a.K ? ld : a.K;
  };
  int stage_b = g_mma_stage;                                     // staged batches per warp (4 KB each)
  auto cta_slots = [&](int w, int kc = 1) -> int64_t {           // CTAs of w warps resident on the machine
    int64_t per = warps_sm / w;
    const size_t xs_bytes = (((size_t)a.M * slice_ld(w, kc) * 2 + 15) & ~(size_t)15);
    const size_t sm = xs_bytes + (w > 1 ? (size_t)w * PB * 512 : 0) + (size_t)w * stage_b * 4096 + 1024;
    const int64_t by_smem = (int64_t)((size_t)227 * 1024 / sm);
    if (per > by_smem) per = by_smem;
    if (per > 32) per = 32;
    return per * g_mma_sms / n_slots;
  };
  int ks = 1, kcta = 1, warps = kW;
  int64_t grid_x = 0;
  a.rounds = 1;
  if (nblk <= cta_slots(1)) {
    const int64_t smax = npair / 4 > 0 ? npair / 4 : 1;         // at least 4 k-step pairs per warp
    const int kc_cap = (a.slot_expert || nblk > kMaxSplitUnits) ? 1 : g_mma_kcta_max;
    // prefer deep staging; give it up (2 -> 1 -> 0 batches) when shared memory would cost residency
    int64_t best = -1;
    int best_ks = 1, best_kcta = 1, best_stage = 0;
    for (int sb = g_mma_stage; sb >= 0; --sb) {
      stage_b = sb;
      int64_t S = (int64_t)kW * kc_cap;
      if (S > smax) S = smax;
      int k1 = 1, c1 = 1;
      for (; S > 1; --S) {                                       // most slices per block that still fit one wave
        c1 = (int)((S + kW - 1) / kW);
        k1 = (int)(S / c1);
        if (nblk * c1 <= cta_slots(k1, c1)) break;
      }
      if (S <= 1) { k1 = 1; c1 = 1; }
      const int64_t warps_total = nblk * c1 * k1;
      if (warps_total > best) { best = warps_total; best_ks = k1; best_kcta = c1; best_stage = sb; }
    }
    ks = best_ks; kcta = best_kcta; stage_b = best_stage;
    warps = ks;
    grid_x = nblk * kcta;
  } else {
    // more 16-row blocks than one wave holds: 8-warp CTAs sweep in rounds.  The K split inside a CTA
    // (ks warps per block, 8 / ks blocks per round) grows until there are enough units to occupy
    // the CTAs that fit (few fit when many activation rows x a long K fill the shared memory).
    stage_b = 0;
    const int64_t cap = cta_slots(kW) > 0 ? cta_slots(kW) : 1;
    ks = 1;
    while (ks < kW && (nblk * ks + kW - 1) / kW < cap && npair / (ks * 2) >= 4) ks <<= 1;
    const int64_t units = (nblk * ks + kW - 1) / kW;
    a.rounds = (int)((units + cap - 1) / cap);
    grid_x = (units + a.rounds - 1) / a.rounds;             // every CTA the same number of rounds ...
    if (grid_x * 5 < cap * 4) grid_x = units < cap ? units : cap;   // ... unless that idles a fifth of the machine
  }
  a.stage_batches = stage_b;
  a.ksplit = ks;
  a.kcta = kcta;
  a.ws = nullptr; a.tickets = nullptr;
  if (kcta > 1) {
    cudaGetSymbolAddress((void**)&a.ws, g_split_ws);
    cudaGetSymbolAddress((void**)&a.tickets, g_split_tickets);
  }
  a.pf_rounds = a.slot_expert ? 0 : (a.rounds < g_mma_pf_rounds ? a.rounds : g_mma_pf_rounds);
  a.xs_ld = slice_ld(ks, kcta);
  size_t smem = (((size_t)a.M * a.xs_ld * 2 + 15) & ~(size_t)15);
  if (ks > 1) smem += (size_t)a.rounds * warps * PB * 128 * sizeof(float);
  if (smem > 200 * 1024) return CB_ERR_SHAPE;
  smem += (size_t)warps * stage_b * 4096;
  auto kern = gemv_mma_kernel<SWIGLU, NORM, OUT_F32>;
  if (smem + 2048 > 48 * 1024) {   // the 48 KB default also has to hold the static shared memory
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cb_launch(kern, dim3((unsigned)grid_x, (unsigned)n_slots), dim3((unsigned)warps * 32), smem, st, a);
}

}  // namespace

CB_EXPORT int cb_set_mma_gemv_opts(int64_t ctas_per_sm) { g_mma_ctas = ctas_per_sm < 1 ? 1 : (int)ctas_per_sm; return 0; }
// Largest number of CTAs that may share one 16-row block (1 switches the cross-CTA K split off).
CB_EXPORT int cb_set_mma_gemv_kcta(int64_t n) { g_mma_kcta_max = n < 1 ? 1 : (n > 4 ? 4 : (int)n); return 0; }
// Weight batches (4 KB per warp each) staged in shared memory ahead of the dependency wait.
CB_EXPORT int cb_set_mma_gemv_stage(int64_t n) { g_mma_stage = n < 0 ? 0 : (n > 4 ? 4 : (int)n); return 0; }
// Sweep rounds prefetched into L2 ahead of the dependency wait (0 = none).
CB_EXPORT int cb_set_mma_gemv_prefetch(int64_t rounds) { g_mma_pf_rounds = rounds < 0 ? 0 : (int)rounds; return 0; }

// Same contract as cb_gemv_bf16 (M = 1..8, any M in that range).  The `_tail` form adds the fused consumer
// of a pushing projection: tail_out = rmsnorm(tail_res_in + sum over ranks of push_site) * tail_gain and the
// sum itself in tail_res_out, done by the last CTA of the grid (the epoch of the step must not change
// between the push and the next kernel, which holds inside one decode step).
static int gemv_mma_impl(const void* W, const void* x, void* y, int64_t M, int64_t N, int64_t K,
                         int64_t ldy, int64_t mode, int64_t up_off, const void* res_in, const void* add,
                         const void* gain, void* res_out, float eps, const void* tp, int64_t pull_site,
                         int64_t push_site, const void* tail_res_in, const void* tail_gain, void* tail_res_out,
                         void* tail_out, float tail_eps, void* stream);
CB_EXPORT int cb_gemv_mma_bf16(const void* W, const void* x, void* y, int64_t M, int64_t N, int64_t K,
                               int64_t ldy, int64_t mode, int64_t up_off, const void* res_in, const void* add,
                               const void* gain, void* res_out, float eps, const void* tp, int64_t pull_site,
                               int64_t push_site, void* stream) {
  return gemv_mma_impl(W, x, y, M, N, K, ldy, mode, up_off, res_in, add, gain, res_out, eps, tp, pull_site, push_site,
                       nullptr, nullptr, nullptr, nullptr, 0.f, stream);
}
CB_EXPORT int cb_gemv_mma_bf16_tail(const void* W, const void* x, int64_t M, int64_t N, int64_t K, const void* tp,
                                    int64_t push_site, const void* tail_res_in, const void* tail_gain,
                                    void* tail_res_out, void* tail_out, float tail_eps, void* stream) {
  if (!tp || push_site < 0 || !tail_res_in || !tail_gain || !tail_res_out || !tail_out || N % 8) return CB_ERR_ARG;
  if (tail_res_out == tail_res_in) return CB_ERR_ARG;
  return gemv_mma_impl(W, x, nullptr, M, N, K, N, 0, N, nullptr, nullptr, nullptr, nullptr, 0.f, tp, -1, push_site,
                       tail_res_in, tail_gain, tail_res_out, tail_out, tail_eps, stream);
}
static int gemv_mma_impl(const void* W, const void* x, void* y, int64_t M, int64_t N, int64_t K,
                         int64_t ldy, int64_t mode, int64_t up_off, const void* res_in, const void* add,
                         const void* gain, void* res_out, float eps, const void* tp, int64_t pull_site,
                         int64_t push_site, const void* tail_res_in, const void* tail_gain, void* tail_res_out,
                         void* tail_out, float tail_eps, void* stream) {
  if (!W || (!y && push_site < 0) || (!x && !res_in) || (res_in && !gain)) return CB_ERR_ARG;
  if ((pull_site >= 0 || push_site >= 0) && !tp) return CB_ERR_ARG;
  if (pull_site >= 0 && !res_in) return CB_ERR_ARG;
  if (K % 8 || M < 1 || M > 8 || N < 1) return CB_ERR_SHAPE;
  if (res_in && res_out && (res_out == res_in || res_out == add)) return CB_ERR_ARG;
  MmaArgs a;
  a.W = (const bf16*)W; a.x = (const bf16*)x; a.y = y; a.N = N; a.K = K; a.ldy = ldy; a.up_off = up_off;
  a.res_in = (const bf16*)res_in; a.add = (const bf16*)add; a.gain = (const float*)gain;
  a.res_out = (bf16*)res_out; a.eps = eps; a.M = (int)M; a.ksplit = 1; a.rounds = 1;
  a.pull_site = (int)pull_site; a.push_site = (int)push_site;
  a.slot_expert = nullptr; a.slot_xrow = nullptr; a.expert_stride = 0;
  a.tail_res_in = (const bf16*)tail_res_in; a.tail_gain = (const float*)tail_gain; a.tail_res_out = (bf16*)tail_res_out;
  a.tail_out = (bf16*)tail_out; a.tail_eps = tail_eps;
  if (tp) a.tp = *(const TpComm*)tp; else memset(&a.tp, 0, sizeof(a.tp));
  const bool sw = mode & 1, f32 = mode & 2, norm = res_in != nullptr;
  cudaStream_t st = (cudaStream_t)stream;
  if (sw) {
    if (f32) return CB_ERR_ARG;
    return norm ? launch_mma<true, true, false>(a, st) : launch_mma<true, false, false>(a, st);
  }
  if (f32) return norm ? launch_mma<false, true, true>(a, st) : launch_mma<false, false, true>(a, st);
  return norm ? launch_mma<false, true, false>(a, st) : launch_mma<false, false, false>(a, st);
}

// Grouped expert projection for decode: for every slot s (a routed (token, expert) pair),
// y[s, :] = W[slot_expert[s]] x[slot_xrow[s], :]   (W: [E, N(or 2N), K] stacked experts).
// mode bit 1 = SwiGLU epilogue (gate rows then up rows inside each expert).
CB_EXPORT int cb_moe_gemv(const void* W, const void* x, void* y, int64_t n_slots, int64_t N, int64_t K, int64_t ldy,
                          int64_t mode, const void* slot_expert, const void* slot_xrow, int64_t expert_stride,
                          void* stream) {
  if (!W || !x || !y || !slot_expert) return CB_ERR_ARG;
  if (K % 8 || N < 1 || n_slots < 1 || n_slots > 65535) return CB_ERR_SHAPE;
  MmaArgs a;
  a.W = (const bf16*)W; a.x = (const bf16*)x; a.y = y; a.N = N; a.K = K; a.ldy = ldy; a.up_off = N;
  a.res_in = nullptr; a.add = nullptr; a.gain = nullptr; a.res_out = nullptr; a.eps = 0.f; a.M = 1; a.ksplit = 1;
  a.rounds = 1; a.pull_site = -1; a.push_site = -1;
  a.tail_res_in = nullptr; a.tail_gain = nullptr; a.tail_res_out = nullptr; a.tail_out = nullptr; a.tail_eps = 0.f;
  a.slot_expert = (const int*)slot_expert; a.slot_xrow = (const int*)slot_xrow; a.expert_stride = expert_stride;
  memset(&a.tp, 0, sizeof(a.tp));
  cudaStream_t st = (cudaStream_t)stream;
  if (mode & 1) return launch_mma<true, false, false>(a, st, (int)n_slots);
  return launch_mma<false, false, false>(a, st, (int)n_slots);
}
