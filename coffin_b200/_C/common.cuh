// Shared device/host helpers for the sm_100a kernel library.
//
// Every exported entry point is `extern "C" int cb_<name>(..., void* stream)`: raw device
// pointers, 64-bit integer sizes, float scalars, the CUDA stream last, and an int status
// (0 = launched; a cudaError_t value or a CB_ERR_* code otherwise).  The Python side binds
// them with ctypes, so no torch header is compiled and the library links only cudart.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define CB_EXPORT extern "C" __attribute__((visibility("default")))

enum CbError : int {
  CB_OK = 0,
  CB_ERR_SHAPE = 10001,      // unsupported size / alignment
  CB_ERR_ARG = 10002,        // null pointer or bad mode
  CB_ERR_DRIVER = 10003,     // driver entry point lookup failed
  CB_ERR_TIMEOUT = 10004,    // a bounded device-side wait ran out (status word set)
};

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

#define CB_CHECK_LAUNCH()                          \
  do {                                             \
    cudaError_t e__ = cudaGetLastError();          \
    if (e__ != cudaSuccess) return (int)e__;       \
  } while (0)

// ---- programmatic dependent launch -------------------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may start while its
// predecessor drains; it must execute griddep_wait() before touching anything the predecessor
// wrote (or writing anything the predecessor reads).  Without the attribute both are no-ops.
//
// Step trace (diagnostic): when a trace buffer is installed, thread 0 of block 0 of every kernel
// stamps %globaltimer when it enters (griddep_launch) and when its dependency has resolved
// (griddep_wait).  Kernels of one stream run in order, so the n-th entry stamp and the n-th ready
// stamp belong to the n-th kernel, and the time between two consecutive ready stamps is the span a
// kernel really occupies inside a CUDA graph with programmatic dependent launch - something a
// serialising profiler cannot show.  Layout: [0] entry count, [1] ready count, then (entry, ready)
// pairs.  Every translation unit holds its own pointer (no relocatable device code); the setters
// register themselves at load time.
namespace cbtrace {
constexpr int kMaxEvents = 8192;
static __device__ unsigned long long* buf = nullptr;
__device__ __forceinline__ void stamp(int which) {
  if ((threadIdx.x | threadIdx.y | blockIdx.x | blockIdx.y | blockIdx.z) != 0) return;
  unsigned long long* b = buf;
  if (!b) return;
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  const unsigned long long i = atomicAdd(b + which, 1ull);
  if (i < (unsigned long long)kMaxEvents) b[2 + 2 * i + which] = t;
}
}  // namespace cbtrace
extern "C" void cb_trace_register(void (*setter)(unsigned long long*));
extern "C" void cb_trace_name(const void* kernel);
extern int g_cb_trace_names;
namespace cbtrace {
static void set_tu(unsigned long long* p) { cudaMemcpyToSymbol(buf, &p, sizeof(p)); }
struct Registrar { Registrar() { cb_trace_register(&set_tu); } };
static Registrar registrar;
}  // namespace cbtrace

__device__ __forceinline__ void griddep_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  cbtrace::stamp(1);
}
__device__ __forceinline__ void griddep_launch() {
  cbtrace::stamp(0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Global switch (set from Python): launch with the PDL attribute or as plain launches.
extern int g_cb_use_pdl;

template <typename... KArgs, typename... Args>
static inline cudaError_t cb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_cb_use_pdl ? 1 : 0;
  if (g_cb_trace_names) cb_trace_name((const void*)kernel);
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- small math ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `red` is >= 32 floats of shared memory. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(t);
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// 8 bf16 (one 16-byte vector) <-> 8 floats
__device__ __forceinline__ void bf16x8_to_float(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint32_t pack_bf162(float a, float b) {
  bf162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ uint4 float_to_bf16x8(const float* f) {
  return make_uint4(pack_bf162(f[0], f[1]), pack_bf162(f[2], f[3]), pack_bf162(f[4], f[5]),
                    pack_bf162(f[6], f[7]));
}
// streaming 16-byte load that does not pollute L1 (weights are read exactly once)
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
