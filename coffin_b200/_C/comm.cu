// Host helpers for peer memory: device buffers that can be opened by the other ranks of the node
// (CUDA IPC), and the step-epoch kernel.  The handles travel over the CPU control plane; the data
// path afterwards is plain loads/stores on NVLink from inside the compute kernels (tp.cuh).
// Reference role: P2pReduce.__init__ exchanging cudaIpc handles (models/qwen35/ep.py:546-736,
// backends/corex/kernels/p2p_reduce.cu:177-203).
#include <string.h>
#include "tp.cuh"

namespace {
__global__ void epoch_bump_kernel(unsigned* epoch) {
  griddep_launch();
  griddep_wait();
  if (threadIdx.x == 0) *epoch += 1;
}

// Copy an existing [T, width] bf16 tensor into this rank's peer-visible buffer and publish it (producers
// that are not a GEMM, e.g. the MoE combine under expert parallelism); the owners of the rows pull them.
__global__ void __launch_bounds__(256) tp_pf_scatter_kernel(const TpPfDev* d, const bf16* src, int64_t lds, int T,
                                                            unsigned seq) {
  griddep_launch();
  griddep_wait();
  const int W = d->width, vec = W >> 3;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < (int64_t)T * vec; i += (int64_t)gridDim.x * 256) {
    const int row = (int)(i / vec), c = (int)(i % vec) * 8;
    bf16* dst = d->inbox[d->rank] + (int64_t)row * W + c;          // local copy: the owner of the row pulls it
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src + (int64_t)row * lds + c);
  }
  // one system-scope fence per CTA: the barrier orders every thread's stores before thread 0's fence,
  // which is cumulative, so the flag it publishes afterwards covers them all
  __syncthreads();
  if (threadIdx.x == 0) __threadfence_system();
  if (threadIdx.x == 0) tp_pf_publish(d, 1, seq, gridDim.x);
}

// Pull the partial rows this rank owns from every rank's buffer (coalesced 16-byte peer loads, rank order),
// add the residual rows, store the reduced rows into every rank's result buffer.
// WORLD_MAX bounds the rank loop at compile time and U is the number of 16-byte columns a thread handles per
// pass: with few ranks more columns fit in the registers, and every column's loads (one per rank, most of
// them over NVLink) are in flight before the first add - the kernel is latency bound.
template <int WORLD_MAX, int U>
__global__ void __launch_bounds__(256) tp_pf_reduce_gather_kernel(const TpPfDev* d, const bf16* residual, int64_t ldr,
                                                                  int T, unsigned seq) {
  griddep_launch();
  griddep_wait();
  seq = tp_pf_seq(d, seq);
  tp_pf_wait(d->flags1[d->rank], d->world, seq, d->status, d->wait_ns);
  const int rpr = d->rows_per_rank, W = d->width, vec = W >> 3, world = d->world;
  const int row0 = d->rank * rpr;
  const int nrows = max(0, min(rpr, T - row0));
  const int64_t total = (int64_t)nrows * vec, stride = (int64_t)gridDim.x * 256;
  for (int64_t i0 = (int64_t)blockIdx.x * 256 + threadIdx.x; i0 < total; i0 += stride * U) {
    uint4 part[U][WORLD_MAX], res[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + u * stride;
      if (i >= total) break;
      const int lr = (int)(i / vec), c = (int)(i % vec) * 8;
#pragma unroll
      for (int r = 0; r < WORLD_MAX; ++r)
        if (r < world) part[u][r] = __ldcg(reinterpret_cast<const uint4*>(d->inbox[r] + (int64_t)(row0 + lr) * W + c));
      if (residual) res[u] = *reinterpret_cast<const uint4*>(residual + (int64_t)(row0 + lr) * ldr + c);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + u * stride;
      if (i >= total) break;
      const int lr = (int)(i / vec), c = (int)(i % vec) * 8;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < WORLD_MAX; ++r) {
        if (r < world) {
          float f[8];
          bf16x8_to_float(part[u][r], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += f[e];
        }
      }
      if (residual) {
        float f[8];
        bf16x8_to_float(res[u], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += f[e];
      }
      const uint4 v = float_to_bf16x8(acc);
      for (int p = 0; p < world; ++p)
        *reinterpret_cast<uint4*>(d->out[p] + (int64_t)(row0 + lr) * W + c) = v;
    }
  }
  // one system-scope fence per CTA: the barrier orders every thread's stores before thread 0's fence,
  // which is cumulative, so the flag it publishes afterwards covers them all
  __syncthreads();
  if (threadIdx.x == 0) __threadfence_system();
  if (threadIdx.x == 0) tp_pf_publish(d, 2, seq, gridDim.x);
}

__global__ void tp_pf_wait_kernel(const TpPfDev* d, unsigned seq) {
  griddep_launch();
  griddep_wait();
  const bool counted = seq == 0;
  seq = tp_pf_seq(d, seq);
  tp_pf_wait(d->flags2[d->rank], d->world, seq, d->status, d->wait_ns);
  if (counted && threadIdx.x == 0) *d->seq_dev = seq;      // this all-reduce is complete on this rank
}
}  // namespace

// ---------------------------------------------------------------------------------------------
// One-shot all-reduce for the few rows of a decode bucket ([M <= 64, hidden]) in ONE kernel.  The
// reduce-scatter / all-gather above crosses NVLink twice and takes three launches, which at ~160 KB is
// all latency.  Here CTA m of every rank stores row m of its partial sums into a slot of every PEER's
// inbox as {two bf16, sequence number} 8-byte pairs (data and flag travel together, so no fence, no
// arrival counter and no flag round trip), then polls (bounded) the pairs the peers stored into its own
// inbox, adds the world's rows in rank order plus the residual, and can finish with the RMSNorm the next
// projection needs: all-reduce, residual add and norm are one launch, and the wait is one NVLink
// crossing.  Slots alternate between two halves of the inbox with the sequence number: a rank can only
// be one all-reduce ahead of a peer (it needs the peer's rows of the one in between), so the half it
// writes is never one a peer is still reading.  Every rank adds the same values in the same order, so
// the ranks' results are bit-identical.
namespace {
constexpr int kOsRows = 64;          // rows per slot

// 16 bytes = two pairs = four bf16 + the sequence number twice
__device__ __forceinline__ void os_st2(uint2* dst, unsigned d0, unsigned d1, unsigned s) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(d0), "r"(s), "r"(d1), "r"(s) : "memory");
}
__device__ __forceinline__ uint4 os_ld2(const uint2* src) {
  uint4 q;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "l"(src) : "memory");
  return q;
}

__global__ void __launch_bounds__(512) tp_os_allreduce_kernel(const TpPfDev* d, const bf16* src, int64_t lds,
                                                              const bf16* residual, int64_t ldr, const float* gain,
                                                              bf16* res_out, int64_t ldo, bf16* normed, int64_t ldn,
                                                              float eps, unsigned seq, int8_t* q, float* qscale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* row = reinterpret_cast<float*>(smem_raw);   // [width]
  __shared__ float red[32];
  griddep_launch();
  griddep_wait();
  const bool counted = seq == 0;
  const unsigned s = tp_pf_seq(d, seq);
  const int W = d->width, world = d->world, me = d->rank, m = blockIdx.x;
  const int64_t pairs_row = W >> 1;
  // pair index of (half, source rank, row m)
  auto slot = [&](int r) { return (((int64_t)(s & 1u) * world + r) * kOsRows + m) * pairs_row; };
  // ---- push this rank's row to every peer
  for (int c = threadIdx.x; c < (W >> 3); c += blockDim.x) {
    const uint4 v = *reinterpret_cast<const uint4*>(src + (int64_t)m * lds + c * 8);
    for (int p = 0; p < world; ++p) {
      if (p == me) continue;
      uint2* dst = reinterpret_cast<uint2*>(d->os_inbox[p]) + slot(me) + c * 4;
      os_st2(dst, v.x, v.y, s);
      os_st2(dst + 2, v.z, v.w, s);
    }
  }
  // ---- gather the peers' rows from the own inbox, add in rank order
  const uint2* in = reinterpret_cast<const uint2*>(d->os_inbox[me]);
  const unsigned long long limit = d->wait_ns ? d->wait_ns : kTpWaitNs;
  float ss = 0.f;
  for (int c = threadIdx.x; c < (W >> 3); c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      uint4 v;
      if (r == me) {
        v = *reinterpret_cast<const uint4*>(src + (int64_t)m * lds + c * 8);
      } else {
        const uint2* p = in + slot(r) + c * 4;
        uint4 a = os_ld2(p), b = os_ld2(p + 2);
        if (a.y != s || a.w != s || b.y != s || b.w != s) {
          const unsigned long long t0 = tp_now_ns();
          unsigned spins = 0;
          bool ok = tp_status_set(d->status) != 0;      // an earlier wait already ran out: do not spin again
          while (!ok) {
            if ((++spins & 63u) == 0) {
              if (tp_status_set(d->status)) break;
              if (tp_now_ns() - t0 > limit) {
                atomicCAS(d->status, 0, 32 + r);
                break;
              }
            }
            if (a.y != s || a.w != s) a = os_ld2(p);
            if (b.y != s || b.w != s) b = os_ld2(p + 2);
            ok = a.y == s && a.w == s && b.y == s && b.w == s;
          }
        }
        v = make_uint4(a.x, a.z, b.x, b.z);
      }
      float f[8];
      bf16x8_to_float(v, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += f[e];
    }
    if (residual) {
      float f[8];
      bf16x8_to_float(*reinterpret_cast<const uint4*>(residual + (int64_t)m * ldr + c * 8), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = __bfloat162float(__float2bfloat16(acc[e])) + f[e];   // the partial sum is a bf16 tensor in the unfused path
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = __bfloat162float(__float2bfloat16(acc[e]));
    if (res_out) *reinterpret_cast<uint4*>(res_out + (int64_t)m * ldo + c * 8) = float_to_bf16x8(acc);
#pragma unroll
    for (int e = 0; e < 8; ++e) { row[c * 8 + e] = acc[e]; ss += acc[e] * acc[e]; }
  }
  if (gain) {
    const float rstd = rsqrtf(block_sum(ss, red) / (float)W + eps);
    float amax = 0.f;
    for (int c = threadIdx.x; c < (W >> 3); c += blockDim.x) {
      float f[8];
      const float4 g0 = *reinterpret_cast<const float4*>(gain + c * 8);
      const float4 g1 = *reinterpret_cast<const float4*>(gain + c * 8 + 4);
      f[0] = row[c * 8 + 0] * (rstd * g0.x); f[1] = row[c * 8 + 1] * (rstd * g0.y);
      f[2] = row[c * 8 + 2] * (rstd * g0.z); f[3] = row[c * 8 + 3] * (rstd * g0.w);
      f[4] = row[c * 8 + 4] * (rstd * g1.x); f[5] = row[c * 8 + 5] * (rstd * g1.y);
      f[6] = row[c * 8 + 6] * (rstd * g1.z); f[7] = row[c * 8 + 7] * (rstd * g1.w);
      if (normed) *reinterpret_cast<uint4*>(normed + (int64_t)m * ldn + c * 8) = float_to_bf16x8(f);
      if (q) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float v = __bfloat162float(__float2bfloat16(f[e]));
          row[c * 8 + e] = v;
          amax = fmaxf(amax, fabsf(v));
        }
      }
    }
    if (q) {   // int8 rows + scales for an int8 projection that follows (the arithmetic of quant_rows)
      amax = block_max(amax, red);
      const float sc = fmaxf(amax, 1e-8f) / 127.f, inv = 1.f / sc;
      if (threadIdx.x == 0) qscale[m] = sc;
      for (int i = threadIdx.x; i < W; i += blockDim.x)
        q[(int64_t)m * W + i] = (int8_t)max(-127, min(127, __float2int_rn(row[i] * inv)));
    }
  }
  // the last CTA to finish marks the all-reduce complete (the next one takes "last completed + 1")
  __syncthreads();
  if (counted && threadIdx.x == 0) {
    const unsigned prev = atomicAdd(d->arrive + 1, 1u);
    if (prev == gridDim.x - 1) {
      d->arrive[1] = 0;
      *d->seq_dev = s;
    }
  }
}
}  // namespace

CB_EXPORT int cb_tp_os_rows() { return kOsRows; }
CB_EXPORT int cb_tp_os_allreduce(const void* desc, const void* src, int64_t lds, const void* residual, int64_t ldr,
                                 const void* gain, void* res_out, int64_t ldo, void* normed, int64_t ldn, int64_t M,
                                 int64_t width, float eps, int64_t seq, void* q, void* qscale, void* stream) {
  if (!desc || !src || M < 1 || M > kOsRows || lds % 8 || width % 8 || width * 4 > 200 * 1024) return CB_ERR_ARG;
  if ((q == nullptr) != (qscale == nullptr) || ((normed || q) && !gain) || (gain && !normed && !q) || (!res_out && !normed && !q))
    return CB_ERR_ARG;
  const size_t smem = (size_t)width * 4;
  if (smem + 1024 > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(tp_os_allreduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int threads = (int)((width / 8 + 31) / 32 * 32);
  threads = threads > 512 ? 512 : threads;
  return (int)cb_launch(tp_os_allreduce_kernel, dim3((unsigned)M), dim3(threads), smem, (cudaStream_t)stream,
                        (const TpPfDev*)desc, (const bf16*)src, lds, (const bf16*)residual, ldr, (const float*)gain,
                        (bf16*)res_out, ldo, (bf16*)normed, ldn, eps, (unsigned)seq, (int8_t*)q, (float*)qscale);
}

CB_EXPORT int cb_tp_pf_scatter(const void* desc, const void* src, int64_t lds, int64_t T, int64_t seq, void* stream) {
  if (!desc || !src || T < 1 || lds % 8) return CB_ERR_ARG;
  return (int)cb_launch(tp_pf_scatter_kernel, dim3(148), dim3(256), 0, (cudaStream_t)stream, (const TpPfDev*)desc,
                        (const bf16*)src, lds, (int)T, (unsigned)seq);
}
// Second half of the prefill all-reduce; the result is in this rank's result buffer once
// cb_tp_pf_wait (launched right after) has returned.
CB_EXPORT int cb_tp_pf_reduce_gather(const void* desc, const void* residual, int64_t ldr, int64_t T, int64_t seq,
                                     int64_t world, void* stream) {
  if (!desc || T < 1 || (residual && ldr % 8)) return CB_ERR_ARG;
  if (world < 1 || world > kTpMaxWorld) return CB_ERR_ARG;      // the descriptor itself lives in device memory
  if (world <= 2)
    return (int)cb_launch(tp_pf_reduce_gather_kernel<2, 8>, dim3(148), dim3(256), 0, (cudaStream_t)stream,
                          (const TpPfDev*)desc, (const bf16*)residual, ldr, (int)T, (unsigned)seq);
  if (world <= 4)
    return (int)cb_launch(tp_pf_reduce_gather_kernel<4, 6>, dim3(148), dim3(256), 0, (cudaStream_t)stream,
                          (const TpPfDev*)desc, (const bf16*)residual, ldr, (int)T, (unsigned)seq);
  return (int)cb_launch(tp_pf_reduce_gather_kernel<kTpMaxWorld, 4>, dim3(148), dim3(256), 0, (cudaStream_t)stream,
                        (const TpPfDev*)desc, (const bf16*)residual, ldr, (int)T, (unsigned)seq);
}
CB_EXPORT int cb_tp_pf_wait(const void* desc, int64_t seq, void* stream) {
  if (!desc) return CB_ERR_ARG;
  return (int)cb_launch(tp_pf_wait_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, (const TpPfDev*)desc,
                        (unsigned)seq);
}
CB_EXPORT int cb_tp_pf_desc_size() { return (int)sizeof(TpPfDev); }
CB_EXPORT int cb_peer_write(void* dev, const void* host, int64_t bytes) {
  return (int)cudaMemcpy(dev, host, (size_t)bytes, cudaMemcpyHostToDevice);
}

CB_EXPORT int cb_peer_alloc(int64_t bytes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}
CB_EXPORT int cb_peer_free(void* p) { return (int)cudaFree(p); }
CB_EXPORT int cb_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
CB_EXPORT int cb_ipc_open_handle(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}
CB_EXPORT int cb_ipc_close_handle(void* p) { return (int)cudaIpcCloseMemHandle(p); }

// Device-to-device copy between two mappings of this process (a local buffer and, say, an IPC mapping of
// another process's buffer on this or a peer GPU: the copy then crosses NVLink once, no host staging).
CB_EXPORT int cb_copy_d2d(void* dst, const void* src, int64_t bytes, void* stream) {
  if (!dst || !src || bytes < 0) return CB_ERR_ARG;
  if (bytes == 0) return 0;
  return (int)cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)stream);
}

CB_EXPORT int cb_peer_read_i32(const void* dev, int* out) {
  return (int)cudaMemcpy(out, dev, sizeof(int), cudaMemcpyDeviceToHost);
}

// Advance the step epoch (first kernel of every decode step on every rank).
CB_EXPORT int cb_tp_epoch_bump(void* epoch, void* stream) {
  return (int)cb_launch(epoch_bump_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, (unsigned*)epoch);
}

// ---------------------------------------------------------------------------------------------
// Decode all-reduce, consumer side, done once per row instead of once per CTA of the next
// projection: pull the ranks' partial sums of `site` (bounded wait on the data-carried epochs), add
// them to the residual in rank order, write the new residual and its RMSNorm.  One CTA per row.
// A projection of several hundred CTAs that each pulled world x K pairs spent ~10 us per site in L2
// traffic (world x 20 KB x CTAs); here a single CTA reads them and the projection copies 5 KB.
// Arithmetic and rounding are those of the fused GEMV prologue (gemv_mma.cu), so every rank still
// holds bit-identical activations.
namespace {
__global__ void __launch_bounds__(1024) tp_pull_norm_kernel(const TpComm tp, int site, const bf16* __restrict__ res_in,
                                                            const float* __restrict__ gain, bf16* __restrict__ res_out,
                                                            bf16* __restrict__ out, int64_t K, float eps) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* row = reinterpret_cast<float*>(smem_raw);  // [K]
  __shared__ float red[32];
  griddep_launch();
  griddep_wait();
  const int64_t m = blockIdx.x;
  float ss = 0.f;
  for (int64_t c = threadIdx.x; c < (K >> 3); c += blockDim.x) {
    float f[8], pulled[8];
    bf16x8_to_float(*reinterpret_cast<const uint4*>(res_in + m * K + c * 8), f);
    tp_pull8(tp, site, m * K + c * 8, pulled);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i] + pulled[i]));
    if (res_out) *reinterpret_cast<uint4*>(res_out + m * K + c * 8) = float_to_bf16x8(f);
#pragma unroll
    for (int i = 0; i < 8; ++i) { row[c * 8 + i] = f[i]; ss += f[i] * f[i]; }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / (float)K + eps);
  for (int64_t c = threadIdx.x; c < (K >> 3); c += blockDim.x) {
    float f[8];
    const float4 g0 = *reinterpret_cast<const float4*>(gain + c * 8);
    const float4 g1 = *reinterpret_cast<const float4*>(gain + c * 8 + 4);
    f[0] = row[c * 8 + 0] * (rstd * g0.x); f[1] = row[c * 8 + 1] * (rstd * g0.y);
    f[2] = row[c * 8 + 2] * (rstd * g0.z); f[3] = row[c * 8 + 3] * (rstd * g0.w);
    f[4] = row[c * 8 + 4] * (rstd * g1.x); f[5] = row[c * 8 + 5] * (rstd * g1.y);
    f[6] = row[c * 8 + 6] * (rstd * g1.z); f[7] = row[c * 8 + 7] * (rstd * g1.w);
    *reinterpret_cast<uint4*>(out + m * K + c * 8) = float_to_bf16x8(f);
  }
}
}  // namespace

// Vocabulary-parallel arg-max without gathering the logits: every rank holds the arg-max of its own
// vocabulary slice (local index per row), sends {value, global index} of every row to every rank as two
// {word, epoch} pairs of `site`, polls the peers' pairs (bounded) and keeps the best - ties go to the
// lowest index, so all ranks agree.  One warp per row, one CTA.  Replaces an all-gather of
// [rows, vocabulary] fp32 logits plus a full-width arg-max.
namespace {
__device__ __forceinline__ unsigned long long tp_wait_pair(const TpComm& c, int64_t elem, unsigned e, int r) {
  unsigned long long v = tp_ld_pair(c.my_inbox, elem);
  if ((unsigned)(v >> 32) != e && !tp_status_set(c.status)) {
    const unsigned long long t0 = tp_now_ns(), limit = c.wait_ns ? c.wait_ns : kTpWaitNs;
    unsigned spins = 0;
    while ((unsigned)(v >> 32) != e) {
      if ((++spins & 63u) == 0) {
        if (tp_status_set(c.status)) break;
        if (tp_now_ns() - t0 > limit) {
          atomicCAS(c.status, 0, 16 + r);
          break;
        }
      }
      v = tp_ld_pair(c.my_inbox, elem);
    }
  }
  return v;
}

__global__ void __launch_bounds__(256) tp_argmax_kernel(const TpComm tp, int site, const float* __restrict__ logits,
                                                         int64_t ld, const int64_t* __restrict__ local_idx,
                                                         int vocab_off, int64_t* __restrict__ next, int M) {
  griddep_launch();
  griddep_wait();
  if ((threadIdx.x & 31) != 0) return;
  const unsigned e = *tp.epoch;
  for (int m = threadIdx.x >> 5; m < M; m += 8) {
    const int64_t li = local_idx[m];
    tp_push_value(tp, site, m * 2, logits[(int64_t)m * ld + li]);
    tp_push_value(tp, site, m * 2 + 1, __int_as_float((int)li + vocab_off));
  }
  for (int m = threadIdx.x >> 5; m < M; m += 8) {
    float v = -INFINITY;
    int ix = 0x7fffffff;
    for (int r = 0; r < tp.world; ++r) {
      const int64_t elem = ((int64_t)site * tp.world + r) * tp.slot_floats + m * 2;
      const float ov = __uint_as_float((unsigned)tp_wait_pair(tp, elem, e, r));
      const int oi = (int)(unsigned)tp_wait_pair(tp, elem + 1, e, r);
      if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
    }
    next[m] = ix == 0x7fffffff ? 0 : ix;
  }
}
}  // namespace
CB_EXPORT int cb_tp_argmax(const void* tp, int64_t site, const void* logits, int64_t ld, const void* local_idx,
                           int64_t vocab_off, void* next, int64_t M, void* stream) {
  if (!tp || !logits || !local_idx || !next || site < 0 || M < 1 || M > 64) return CB_ERR_ARG;
  return (int)cb_launch(tp_argmax_kernel, dim3(1), dim3(256), 0, (cudaStream_t)stream, *(const TpComm*)tp, (int)site,
                        (const float*)logits, ld, (const int64_t*)local_idx, (int)vocab_off, (int64_t*)next, (int)M);
}

// Producer side for projections whose kernel has no push epilogue (the int4 decode projection): store
// fp32 partial rows [M, N] into this rank's slot of `site` on every rank, paired with the step's epoch.
namespace {
__global__ void __launch_bounds__(256) tp_push_rows_kernel(const TpComm tp, int site, const float* __restrict__ src,
                                                           int64_t lds, int M, int64_t N) {
  griddep_launch();
  griddep_wait();
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < (int64_t)M * N; i += (int64_t)gridDim.x * 256) {
    const int64_t m = i / N, n = i % N;
    tp_push_value(tp, site, m * N + n, src[m * lds + n]);
  }
}
}  // namespace
CB_EXPORT int cb_tp_push_rows(const void* tp, int64_t site, const void* src, int64_t lds, int64_t M, int64_t N, void* stream) {
  if (!tp || !src || site < 0 || M < 1 || N < 1) return CB_ERR_ARG;
  const unsigned blocks = (unsigned)((M * N + 255) / 256);
  return (int)cb_launch(tp_push_rows_kernel, dim3(blocks < 148u ? blocks : 148u), dim3(256), 0, (cudaStream_t)stream,
                        *(const TpComm*)tp, (int)site, (const float*)src, lds, (int)M, N);
}

CB_EXPORT int cb_tp_pull_norm(const void* tp, int64_t site, const void* res_in, const void* gain, void* res_out,
                              void* out, int64_t M, int64_t K, float eps, void* stream) {
  if (!tp || !res_in || !gain || !out || site < 0) return CB_ERR_ARG;
  if (M < 1 || K % 8 || K * 4 > 200 * 1024) return CB_ERR_SHAPE;
  const size_t smem = (size_t)K * 4;
  if (smem + 2048 > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(tp_pull_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = K >= 8192 ? 1024 : (K >= 2048 ? 512 : 256);
  return (int)cb_launch(tp_pull_norm_kernel, dim3((unsigned)M), dim3(threads), smem, (cudaStream_t)stream,
                        *(const TpComm*)tp, (int)site, (const bf16*)res_in, (const float*)gain, (bf16*)res_out,
                        (bf16*)out, K, eps);
}
