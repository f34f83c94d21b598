// Row-wise memory-bound kernels: embedding gather, (residual add +) RMSNorm, SwiGLU, argmax,
// temperature sampling, block copies.  One CTA per row, 16-byte vector accesses, fp32 math.
// Roles in the reference: TiedEmbedding.lookup (ops/embed.py:70-145), rms_norm / add_rms_norm
// (backends/corex/kernels/norm.cu:132-206), silu_mul (attn.cu:201), the torch argmax /
// multinomial of ModelRunner.sample (engine/model_runner.py:900-924), PagedKVCache.copy_block.
#include "common.cuh"

int g_cb_use_pdl = 0;
CB_EXPORT int cb_set_pdl(int64_t on) { g_cb_use_pdl = on ? 1 : 0; return 0; }

// ---- step trace (see common.cuh) -------------------------------------------------------------
#include <string>
#include <vector>
int g_cb_trace_names = 0;
namespace {
std::vector<void (*)(unsigned long long*)>& trace_setters() {
  static std::vector<void (*)(unsigned long long*)> v;
  return v;
}
std::vector<std::string>& trace_names() {
  static std::vector<std::string> v;
  return v;
}
}  // namespace
extern "C" void cb_trace_register(void (*setter)(unsigned long long*)) { trace_setters().push_back(setter); }
extern "C" void cb_trace_name(const void* kernel) {
  const char* n = nullptr;
  if (cudaFuncGetName(&n, kernel) == cudaSuccess && n) trace_names().push_back(n);
  else trace_names().push_back("?");
}
// Install (or with a null pointer remove) the trace buffer in every translation unit.  The buffer
// holds 2 + 2 * 8192 unsigned 64-bit words and must be zeroed by the caller.
CB_EXPORT int cb_trace_set(void* buf) {
  for (auto f : trace_setters()) f((unsigned long long*)buf);
  return (int)cudaDeviceSynchronize();
}
// Record the kernel name of every launch made through cb_launch (1) or stop and keep the list (0).
CB_EXPORT int cb_trace_record_names(int64_t on) {
  if (on) trace_names().clear();
  g_cb_trace_names = on ? 1 : 0;
  return 0;
}
CB_EXPORT int64_t cb_trace_name_count() { return (int64_t)trace_names().size(); }
CB_EXPORT int cb_trace_get_name(int64_t i, char* out, int64_t cap) {
  if (i < 0 || i >= (int64_t)trace_names().size() || cap < 1) return CB_ERR_ARG;
  const std::string& s = trace_names()[(size_t)i];
  const size_t n = s.size() < (size_t)cap - 1 ? s.size() : (size_t)cap - 1;
  memcpy(out, s.data(), n);
  out[n] = 0;
  return 0;
}
CB_EXPORT int cb_version() { return 1; }

namespace {

__global__ void embed_gather_kernel(const bf16* __restrict__ table, const int64_t* __restrict__ tokens,
                                    bf16* __restrict__ out, int64_t H, int64_t V) {
  griddep_launch();
  griddep_wait();
  int64_t tok = tokens[blockIdx.x];
  if (tok < 0 || tok >= V) tok = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + tok * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (int64_t)blockIdx.x * H);
  for (int64_t c = threadIdx.x; c < (H >> 3); c += blockDim.x) dst[c] = src[c];
}

// out = rmsnorm(x [+ add]) * gain ; optionally writes the sum back (res_out may alias x here:
// one CTA owns the whole row).
// q / qscale (optional): the normalised row is also quantised to int8 with one fp32 scale per row
// (absmax / 127 of the bf16-rounded values, exactly what quant_rows would compute from `out`), so an
// int8 projection that follows needs no quantisation launch of its own.  `out` may then be null.
__global__ void rmsnorm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ add,
                               const float* __restrict__ gain, bf16* __restrict__ res_out,
                               bf16* __restrict__ out, int64_t N, int64_t ldx, int64_t ldo, float eps,
                               int8_t* __restrict__ q, float* __restrict__ qscale) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* row = reinterpret_cast<float*>(smem_raw);  // [N]
  __shared__ float red[32];
  griddep_launch();
  griddep_wait();
  const int64_t r = blockIdx.x;
  float ss = 0.f;
  for (int64_t c = threadIdx.x; c < (N >> 3); c += blockDim.x) {
    float f[8], g[8];
    bf16x8_to_float(*reinterpret_cast<const uint4*>(x + r * ldx + c * 8), f);
    if (add) {
      bf16x8_to_float(*reinterpret_cast<const uint4*>(add + r * ldx + c * 8), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(__float2bfloat16(f[i] + g[i]));
      if (res_out) *reinterpret_cast<uint4*>(res_out + r * ldx + c * 8) = float_to_bf16x8(f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) { row[c * 8 + i] = f[i]; ss += f[i] * f[i]; }
  }
  const float rstd = rsqrtf(block_sum(ss, red) / (float)N + eps);
  float amax = 0.f;
  for (int64_t c = threadIdx.x; c < (N >> 3); c += blockDim.x) {
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = row[c * 8 + i] * rstd * gain[c * 8 + i];
    if (out) *reinterpret_cast<uint4*>(out + r * ldo + c * 8) = float_to_bf16x8(f);
    if (q) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float v = __bfloat162float(__float2bfloat16(f[i]));
        row[c * 8 + i] = v;
        amax = fmaxf(amax, fabsf(v));
      }
    }
  }
  if (q) {
    amax = block_max(amax, red);
    const float sc = fmaxf(amax, 1e-8f) / 127.f, inv = 1.f / sc;
    if (threadIdx.x == 0) qscale[r] = sc;
    for (int64_t i = threadIdx.x; i < N; i += blockDim.x)
      q[r * N + i] = (int8_t)max(-127, min(127, __float2int_rn(row[i] * inv)));
  }
}

// The same normalisation for many rows (a prefill chunk): one warp per row, the row held in registers
// as packed bf16 (CPL 16-byte chunks per lane), no shared memory and no block barrier.  Reads x (+ add),
// writes res_out (optional) and out.  Values and rounding as in rmsnorm_kernel.
template <int CPL>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const bf16* __restrict__ x, const bf16* __restrict__ add,
                                                           const float* __restrict__ gain, bf16* __restrict__ res_out,
                                                           bf16* __restrict__ out, int64_t M, int64_t N, int64_t ldx,
                                                           int64_t ldo, float eps, int8_t* __restrict__ q,
                                                           float* __restrict__ qscale) {
  griddep_launch();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= M) return;
  const int nchunk = (int)(N >> 3);
  uint4 v[CPL];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < CPL; ++i) {
    const int c = lane + 32 * i;
    if (c < nchunk) v[i] = *reinterpret_cast<const uint4*>(x + r * ldx + c * 8);
  }
  if (add) {
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
      const int c = lane + 32 * i;
      if (c < nchunk) {
        float f[8], g[8];
        bf16x8_to_float(v[i], f);
        bf16x8_to_float(*reinterpret_cast<const uint4*>(add + r * ldx + c * 8), g);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += g[e];
        v[i] = float_to_bf16x8(f);
        if (res_out) *reinterpret_cast<uint4*>(res_out + r * ldx + c * 8) = v[i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < CPL; ++i) {
    if (lane + 32 * i < nchunk) {
      float f[8];
      bf16x8_to_float(v[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
    }
  }
  const float rstd = rsqrtf(warp_sum(ss) / (float)N + eps);
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < CPL; ++i) {
    const int c = lane + 32 * i;
    if (c < nchunk) {
      float f[8];
      bf16x8_to_float(v[i], f);
      const float4 g0 = *reinterpret_cast<const float4*>(gain + c * 8), g1 = *reinterpret_cast<const float4*>(gain + c * 8 + 4);
      f[0] *= rstd * g0.x; f[1] *= rstd * g0.y; f[2] *= rstd * g0.z; f[3] *= rstd * g0.w;
      f[4] *= rstd * g1.x; f[5] *= rstd * g1.y; f[6] *= rstd * g1.z; f[7] *= rstd * g1.w;
      v[i] = float_to_bf16x8(f);                       // the normalised row replaces the input in the registers
      if (out) *reinterpret_cast<uint4*>(out + r * ldo + c * 8) = v[i];
      if (q) {
        bf16x8_to_float(v[i], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
      }
    }
  }
  if (q) {   // int8 rows + scale of the bf16-rounded values (what quant_rows would compute from `out`)
    amax = warp_max(amax);
    const float sc = fmaxf(amax, 1e-8f) / 127.f, inv = 1.f / sc;
    if (lane == 0) qscale[r] = sc;
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
      const int c = lane + 32 * i;
      if (c < nchunk) {
        float f[8];
        bf16x8_to_float(v[i], f);
        uint32_t w[2] = {0u, 0u};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int qi = max(-127, min(127, __float2int_rn(f[e] * inv)));
          w[e >> 2] |= (uint32_t)(qi & 0xff) << (8 * (e & 3));
        }
        *reinterpret_cast<uint2*>(q + r * N + c * 8) = make_uint2(w[0], w[1]);
      }
    }
  }
}

// Pool slots and rotary rows of a prefill chunk: token t of the chunk sits at position pos0 + t, in page
// block_table[(pos0 + t) / block] at offset (pos0 + t) % block.  One launch instead of a string of small
// index operations per chunk.
__global__ void prefill_index_kernel(const int* __restrict__ block_table, int pos0, int T, int block,
                                     int* __restrict__ slots, int* __restrict__ ridx) {
  griddep_launch();
  griddep_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const int p = pos0 + t;
  slots[t] = block_table[p / block] * block + p % block;
  if (ridx) ridx[t] = p;
}

// out[m, i] = silu(gu[m, i]) * gu[m, I + i]
__global__ void swiglu_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int64_t I,
                              int64_t ldg, int64_t ldo, int64_t total_chunks) {
  griddep_launch();
  griddep_wait();
  const int64_t cpr = I >> 3;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_chunks;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = idx / cpr, c = idx % cpr;
    float g[8], u[8];
    bf16x8_to_float(*reinterpret_cast<const uint4*>(gu + m * ldg + c * 8), g);
    bf16x8_to_float(*reinterpret_cast<const uint4*>(gu + m * ldg + I + c * 8), u);
#pragma unroll
    for (int i = 0; i < 8; ++i) g[i] = silu_f(g[i]) * u[i];
    *reinterpret_cast<uint4*>(out + m * ldo + c * 8) = float_to_bf16x8(g);
  }
}

// LayerNorm with bias (vision tower): out = (x - mean) * rsqrt(var + eps) * w + b
__global__ void layernorm_kernel(const bf16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                 bf16* __restrict__ out, int64_t N, int64_t ldx, int64_t ldo, float eps) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* row = reinterpret_cast<float*>(smem_raw);
  __shared__ float red[32];
  griddep_launch();
  griddep_wait();
  const int64_t r = blockIdx.x;
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < N; i += blockDim.x) { row[i] = __bfloat162float(x[r * ldx + i]); s += row[i]; }
  const float mean = block_sum(s, red) / (float)N;
  float v = 0.f;
  for (int64_t i = threadIdx.x; i < N; i += blockDim.x) { const float d = row[i] - mean; v += d * d; }
  const float rstd = rsqrtf(block_sum(v, red) / (float)N + eps);
  for (int64_t i = threadIdx.x; i < N; i += blockDim.x)
    out[r * ldo + i] = __float2bfloat16((row[i] - mean) * rstd * w[i] + b[i]);
}

// tanh-approximated GELU, in place capable
__global__ void gelu_tanh_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, int64_t n) {
  griddep_launch();
  griddep_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(x[i]);
    out[i] = __float2bfloat16(0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v))));
  }
}

// argmax over rows of fp32 logits; ties resolve to the lowest index (torch.argmax order).
// Two stages in one launch: kArgmaxParts CTAs per row each reduce a slice into a (value, index)
// partial in scratch memory, and the last CTA to arrive (atomic ticket) reduces the partials,
// writes the token and re-arms the ticket, so the scratch can be reused by the next launch.
constexpr int kArgmaxParts = 64;

__device__ __forceinline__ void argmax_pair(float& best, int64_t& idx, float ov, int64_t oi) {
  if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
}

__device__ __forceinline__ void argmax_block(float& best, int64_t& idx, float* bv, int64_t* bi) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
    argmax_pair(best, idx, ov, oi);
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) { bv[w] = best; bi[w] = idx; }
  __syncthreads();
  best = lane < nw ? bv[lane] : -INFINITY;
  idx = lane < nw ? bi[lane] : 0x7fffffffffffffffLL;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
    argmax_pair(best, idx, ov, oi);
  }
}

// scratch layout per row: kArgmaxParts floats, kArgmaxParts int64, one unsigned ticket
struct ArgmaxScratch {
  float val[kArgmaxParts];
  int64_t idx[kArgmaxParts];
  unsigned int ticket;
  unsigned int pad;
};

__device__ __forceinline__ void argmax_body(const float* __restrict__ logits, int64_t* __restrict__ out,
                                            int64_t V, int64_t ld, ArgmaxScratch* scratch) {
  __shared__ float bv[32];
  __shared__ int64_t bi[32];
  __shared__ bool last;
  const int row = blockIdx.y, part = blockIdx.x;
  const float* r = logits + (int64_t)row * ld;
  const int64_t per = (V + kArgmaxParts - 1) / kArgmaxParts, b = part * per, e = min(V, b + per);
  float best = -INFINITY;
  int64_t idx = 0x7fffffffffffffffLL;
  for (int64_t i = b + threadIdx.x; i < e; i += blockDim.x) argmax_pair(best, idx, r[i], i);
  argmax_block(best, idx, bv, bi);
  ArgmaxScratch* sc = scratch + row;
  if (threadIdx.x == 0) {
    sc->val[part] = best;
    sc->idx[part] = idx;
    __threadfence();
    last = atomicAdd(&sc->ticket, 1u) == kArgmaxParts - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  best = -INFINITY;
  idx = 0x7fffffffffffffffLL;
  if (threadIdx.x < kArgmaxParts) {
    best = *((volatile float*)&sc->val[threadIdx.x]);
    idx = *((volatile int64_t*)&sc->idx[threadIdx.x]);
  }
  argmax_block(best, idx, bv, bi);
  if (threadIdx.x == 0) {
    out[row] = idx;
    sc->ticket = 0;
  }
}

__global__ void __launch_bounds__(256) argmax_kernel(const float* __restrict__ logits, int64_t* __restrict__ out,
                                                      int64_t V, int64_t ld, ArgmaxScratch* scratch) {
  griddep_launch();
  griddep_wait();
  argmax_body(logits, out, V, ld, scratch);
}

// ---- allocation-free argmax ---------------------------------------------------------------------
// Same two-stage reduction, but the partials and tickets live in a file-scope device array that the
// library carries itself, so the caller provides nothing but its logits and the output.  The array
// is sized for kArgmaxStaticRows rows (about 50 KB per GPU that loads the library, held until the
// process exits).  Device code names the array directly; host code must not pass the symbol itself
// to a kernel (on the host it is only a stand-in), it asks the runtime for the device address once
// per device (cb_argmax_static below).
constexpr int kArgmaxStaticRows = 64;
static __device__ __align__(256) ArgmaxScratch g_argmax_static[kArgmaxStaticRows];

__global__ void __launch_bounds__(256) argmax_static_kernel(const float* __restrict__ logits,
                                                             int64_t* __restrict__ out, int64_t V, int64_t ld,
                                                             ArgmaxScratch* scratch) {
  griddep_launch();
  griddep_wait();
  argmax_body(logits, out, V, ld, scratch);
}

// Temperature sampling by inverse CDF: p = softmax(logits / T); token = first i with cdf(i) > u.
// One CTA per row; u[row] is a uniform random number supplied by the host (so that every
// tensor-parallel rank draws the same token from the same logits).
__global__ void sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                              const float* __restrict__ u, int64_t* __restrict__ out, int64_t V, int64_t ld) {
  __shared__ float red[32];
  __shared__ float chunk_sum[1024];
  griddep_launch();
  griddep_wait();
  const float* row = logits + (int64_t)blockIdx.x * ld;
  const float T = temperature[blockIdx.x];
  const int tid = threadIdx.x, nt = blockDim.x;
  float mx = -INFINITY;
  for (int64_t i = tid; i < V; i += nt) mx = fmaxf(mx, row[i]);
  mx = block_max(mx, red);
  if (!(T > 0.f)) {  // greedy row inside a sampled batch
    int64_t idx = 0x7fffffffffffffffLL;
    for (int64_t i = tid; i < V; i += nt) if (row[i] == mx && i < idx) idx = i;
    __shared__ unsigned long long best;
    if (tid == 0) best = ~0ull;
    __syncthreads();
    atomicMin(&best, (unsigned long long)idx);
    __syncthreads();
    if (tid == 0) out[blockIdx.x] = (int64_t)best;
    return;
  }
  // contiguous span per thread so the CDF order is the index order
  const int64_t per = (V + nt - 1) / nt, b = (int64_t)tid * per, e = min(V, b + per);
  const float inv = 1.f / T;
  float s = 0.f;
  for (int64_t i = b; i < e; ++i) s += __expf((row[i] - mx) * inv);
  chunk_sum[tid] = s;
  const float total = block_sum(s, red);
  __syncthreads();
  if (tid == 0) {
    const float target = u[blockIdx.x] * total;
    float cum = 0.f;
    int t = 0;
    for (; t < nt - 1; ++t) { if (cum + chunk_sum[t] > target) break; cum += chunk_sum[t]; }
    int64_t bb = (int64_t)t * per, ee = min(V, bb + per), pick = min(V - 1, max(bb, ee - 1));
    for (int64_t i = bb; i < ee; ++i) {
      cum += __expf((row[i] - mx) * inv);
      if (cum > target) { pick = i; break; }
    }
    out[blockIdx.x] = pick;
  }
}

// dst[i] = src[i] for `n16` 16-byte words per (blockIdx.y) pair from index lists: copies
// `count` blocks of `block_bytes` bytes: dst_base + dst_idx[j]*block_bytes <- src_base + src_idx[j]*block_bytes
__global__ void block_copy_kernel(unsigned char* __restrict__ dst, const unsigned char* __restrict__ src,
                                  const int64_t* __restrict__ dst_idx, const int64_t* __restrict__ src_idx,
                                  int64_t block_bytes) {
  griddep_launch();
  griddep_wait();
  const int64_t j = blockIdx.y;
  const uint4* s = reinterpret_cast<const uint4*>(src + src_idx[j] * block_bytes);
  uint4* d = reinterpret_cast<uint4*>(dst + dst_idx[j] * block_bytes);
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < (block_bytes >> 4);
       c += (int64_t)gridDim.x * blockDim.x)
    d[c] = s[c];
}

}  // namespace

CB_EXPORT int cb_embed_gather(const void* table, const void* tokens, void* out, int64_t T, int64_t H,
                              int64_t V, void* stream) {
  if (H % 8) return CB_ERR_SHAPE;
  if (T == 0) return 0;
  return (int)cb_launch(embed_gather_kernel, dim3((unsigned)T), dim3(256), 0, (cudaStream_t)stream,
                        (const bf16*)table, (const int64_t*)tokens, (bf16*)out, H, V);
}

CB_EXPORT int cb_rmsnorm_q(const void* x, const void* add, const void* gain, void* res_out, void* out,
                           int64_t M, int64_t N, int64_t ldx, int64_t ldo, float eps, void* q, void* qscale, void* stream);
CB_EXPORT int cb_rmsnorm(const void* x, const void* add, const void* gain, void* res_out, void* out,
                         int64_t M, int64_t N, int64_t ldx, int64_t ldo, float eps, void* stream) {
  if (!out) return CB_ERR_ARG;
  return cb_rmsnorm_q(x, add, gain, res_out, out, M, N, ldx, ldo, eps, nullptr, nullptr, stream);
}
// As cb_rmsnorm, plus the int8 rows q [M, N] and their scales qscale [M] (see the kernel); out may be null.
CB_EXPORT int cb_rmsnorm_q(const void* x, const void* add, const void* gain, void* res_out, void* out,
                           int64_t M, int64_t N, int64_t ldx, int64_t ldo, float eps, void* q, void* qscale, void* stream) {
  if (N % 8 || N * 4 > 200 * 1024) return CB_ERR_SHAPE;
  if ((q == nullptr) != (qscale == nullptr) || (!out && !q)) return CB_ERR_ARG;
  if (M == 0) return 0;
  if (M >= 256 && ldx % 8 == 0 && (!out || ldo % 8 == 0) && ((uintptr_t)gain & 15) == 0 && ((uintptr_t)q & 7) == 0) {   // a prefill chunk: one warp per row
    const dim3 grid((unsigned)((M + 7) / 8));
#define CB_RMS_ROWS(CPL_)                                                                                      \
  return (int)cb_launch(rmsnorm_rows_kernel<CPL_>, grid, dim3(256), 0, (cudaStream_t)stream, (const bf16*)x,   \
                        (const bf16*)add, (const float*)gain, (bf16*)res_out, (bf16*)out, M, N, ldx, ldo, eps,  \
                        (int8_t*)q, (float*)qscale)
    if (N <= 8 * 32 * 4) CB_RMS_ROWS(4);
    if (N <= 8 * 32 * 8) CB_RMS_ROWS(8);
    if (N <= 8 * 32 * 12) CB_RMS_ROWS(12);
    if (N <= 8 * 32 * 20) CB_RMS_ROWS(20);
#undef CB_RMS_ROWS
  }
  const size_t smem = (size_t)N * 4;
  if (smem + 2048 > 48 * 1024) {   // the 48 KB default also has to hold the static shared memory
    cudaError_t e = cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = N >= 2048 ? 256 : 128;
  return (int)cb_launch(rmsnorm_kernel, dim3((unsigned)M), dim3(threads), smem, (cudaStream_t)stream,
                        (const bf16*)x, (const bf16*)add, (const float*)gain, (bf16*)res_out, (bf16*)out,
                        N, ldx, ldo, eps, (int8_t*)q, (float*)qscale);
}

CB_EXPORT int cb_layernorm(const void* x, const void* w, const void* b, void* out, int64_t M, int64_t N, int64_t ldx,
                           int64_t ldo, float eps, void* stream) {
  if (M == 0) return 0;
  if (N * 4 > 200 * 1024) return CB_ERR_SHAPE;
  const size_t smem = (size_t)N * 4;
  if (smem + 2048 > 48 * 1024) {   // the 48 KB default also has to hold the static shared memory
    cudaError_t e = cudaFuncSetAttribute(layernorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cb_launch(layernorm_kernel, dim3((unsigned)M), dim3(256), smem, (cudaStream_t)stream, (const bf16*)x,
                        (const float*)w, (const float*)b, (bf16*)out, N, ldx, ldo, eps);
}

CB_EXPORT int cb_gelu_tanh(const void* x, void* out, int64_t n, void* stream) {
  if (n == 0) return 0;
  const int64_t blocks = min((n + 255) / 256, (int64_t)148 * 8);
  return (int)cb_launch(gelu_tanh_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const bf16*)x,
                        (bf16*)out, n);
}

CB_EXPORT int cb_prefill_index(const void* block_table, int64_t pos0, int64_t T, int64_t block, void* slots, void* ridx,
                               void* stream) {
  if (T == 0) return 0;
  if (T < 0 || pos0 < 0 || block < 1 || !block_table || !slots) return CB_ERR_ARG;
  return (int)cb_launch(prefill_index_kernel, dim3((unsigned)((T + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
                        (const int*)block_table, (int)pos0, (int)T, (int)block, (int*)slots, (int*)ridx);
}

CB_EXPORT int cb_swiglu(const void* gu, void* out, int64_t M, int64_t I, int64_t ldg, int64_t ldo,
                        void* stream) {
  if (I % 8 || ldg % 8 || ldo % 8) return CB_ERR_SHAPE;
  const int64_t total = M * (I >> 3);
  if (total == 0) return 0;
  const int64_t blocks = min((total + 255) / 256, (int64_t)148 * 8);
  return (int)cb_launch(swiglu_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream,
                        (const bf16*)gu, (bf16*)out, I, ldg, ldo, total);
}

// scratch: cb_argmax_scratch_bytes(M) bytes, zero-initialised once by the caller.
CB_EXPORT int64_t cb_argmax_scratch_bytes(int64_t M) { return M * (int64_t)sizeof(ArgmaxScratch); }

CB_EXPORT int cb_argmax(const void* logits, void* out, int64_t M, int64_t V, int64_t ld, void* scratch,
                        void* stream) {
  if (M == 0) return 0;
  if (!scratch) return CB_ERR_ARG;
  return (int)cb_launch(argmax_kernel, dim3(kArgmaxParts, (unsigned)M), dim3(256), 0, (cudaStream_t)stream,
                        (const float*)logits, (int64_t*)out, V, ld, (ArgmaxScratch*)scratch);
}

// See no_alloc.h. Allocation-free variant of cb_argmax: no cudaMalloc / cudaFree / library
// allocation on any call.  The first call on a device looks up the device address of the static
// scratch and clears its tickets (with that device current); make that first call outside any
// stream capture.
static ArgmaxScratch* g_argmax_static_ptr[64] = {};

CB_EXPORT int cb_argmax_static(const void* logits, void* out, int64_t M, int64_t V, int64_t ld, void* stream) {
  if (M == 0) return 0;
  if (!logits || !out || V < 1) return CB_ERR_ARG;
  if (M < 0 || M > kArgmaxStaticRows) return CB_ERR_SHAPE;   // beyond the built-in scratch: use cb_argmax
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return CB_ERR_ARG;
  if (!g_argmax_static_ptr[dev]) {
    ArgmaxScratch* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_argmax_static);
    if (e != cudaSuccess) return (int)e;
    if (!p) return CB_ERR_DRIVER;
    // tickets must start at zero; the kernel re-arms them itself after every launch
    e = cudaMemsetAsync(p, 0, sizeof(ArgmaxScratch) * kArgmaxStaticRows, (cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    g_argmax_static_ptr[dev] = p;
  }
  return (int)cb_launch(argmax_static_kernel, dim3(kArgmaxParts, (unsigned)M), dim3(256), 0, (cudaStream_t)stream,
                        (const float*)logits, (int64_t*)out, V, ld, g_argmax_static_ptr[dev]);
}

CB_EXPORT int64_t cb_argmax_static_max_rows() { return kArgmaxStaticRows; }

CB_EXPORT int cb_sample(const void* logits, const void* temperature, const void* u, void* out, int64_t M,
                        int64_t V, int64_t ld, void* stream) {
  if (M == 0) return 0;
  return (int)cb_launch(sample_kernel, dim3((unsigned)M), dim3(1024), 0, (cudaStream_t)stream,
                        (const float*)logits, (const float*)temperature, (const float*)u, (int64_t*)out, V, ld);
}

CB_EXPORT int cb_block_copy(void* dst, const void* src, const void* dst_idx, const void* src_idx,
                            int64_t count, int64_t block_bytes, void* stream) {
  if (block_bytes % 16) return CB_ERR_SHAPE;
  if (count == 0) return 0;
  const int64_t bx = min((int64_t)64, ((block_bytes >> 4) + 255) / 256);
  return (int)cb_launch(block_copy_kernel, dim3((unsigned)bx, (unsigned)count), dim3(256), 0,
                        (cudaStream_t)stream, (unsigned char*)dst, (const unsigned char*)src,
                        (const int64_t*)dst_idx, (const int64_t*)src_idx, block_bytes);
}

// Feed the sampled tokens back and advance the positions of the live rows (positions >= 0) by one:
// lets greedy steps run back to back with no host round trip and no framework kernels in between.
namespace {
__global__ void advance_rows_kernel(int64_t* tokens, const int64_t* next, int* positions, int* rope_pos, int M) {
  griddep_launch();
  griddep_wait();
  const int m = threadIdx.x;
  if (m >= M) return;
  tokens[m] = next[m];
  if (positions[m] >= 0) {
    positions[m] += 1;
    rope_pos[m] += 1;
  }
}
}  // namespace
CB_EXPORT int cb_advance_rows(void* tokens, const void* next, void* positions, void* rope_pos, int64_t M, void* stream) {
  if (!tokens || !next || !positions || !rope_pos || M < 1 || M > 1024) return CB_ERR_ARG;
  return (int)cb_launch(advance_rows_kernel, dim3(1), dim3((unsigned)((M + 31) / 32 * 32)), 0, (cudaStream_t)stream,
                        (int64_t*)tokens, (const int64_t*)next, (int*)positions, (int*)rope_pos, (int)M);
}
