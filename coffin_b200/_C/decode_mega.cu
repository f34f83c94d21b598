// One decode step of the dense hybrid model as ONE persistent, cooperatively launched kernel.
//
// A decode step of a single sequence is a chain of ~160 dependent, individually tiny kernels; each
// boundary costs 4-5 us of drain, launch and ramp even inside a CUDA graph with programmatic
// dependent launch, and a tensor-parallel step adds a pull kernel per all-reduce site.  Here the
// step is one grid of one 512-thread CTA per SM that walks the phases of every layer
//
//   in-proj (add + RMSNorm prologue) | mixer (delta-net step, or split-KV attention | merge) |
//   out-proj (gated-norm prologue)   | gate/up (add + RMSNorm prologue, SwiGLU epilogue) | down
//
// and finally lm_head + arg-max, separated by a device-side grid barrier (one atomic per CTA on a
// monotonic counter, bounded spin on %globaltimer).  The launch is cooperative, so all CTAs are
// resident or the launch fails; a barrier that does not complete within the limit sets the status
// word, after which no later wait spins and the kernel drains and returns.  While a CTA waits at a
// barrier the L2 is already fetching its slab of the next projection's weights
// (cp.async.bulk.prefetch.L2), so the HBM stream does not stop at phase boundaries.
//
// Projections: a warp feeds 16-byte global loads of weight rows straight into mma.m16n8k16 as the A
// operand (the k index is permuted the same way for the activation, as in gemv_mma.cu).  With M
// activation rows only M of the 8 B columns would be used, so the other columns carry k-slices: the
// 16 A rows are (2M weight rows) x (8/M k-slices), the 8 B columns are (M batch rows) x (8/M
// k-slices), and the products that pair equal slices are summed.  A work group is therefore 2M
// weight rows; a CTA owns a contiguous run of groups (its weights are one contiguous slab) and its
// 16 warps split the run's (group, k-step) items evenly, leaving partial sums in shared memory that
// are added in a fixed order - results do not depend on timing.
//
// Tensor parallel: the finalising thread of a row-parallel projection stores its partial value into
// every rank's inbox ({value, epoch} pairs, tp.cuh) and at once pulls the other ranks' values of the
// same element, so the all-reduce is part of the projection's epilogue and costs no extra barrier.
// The vocabulary-parallel arg-max travels the same way (one {value, index} pair per rank and row).
//
// Role in the reference: the idea of its persistent "mega" kernel with a software grid barrier
// (backends/corex/kernels/mega.cu:79-119, docs/DECODE-LAUNCH-LEDGER.md:27-40,164-184), taken to the
// whole step and to the multi-GPU exchange.
#include <string.h>
#include "sm100.cuh"
#include "tp.cuh"

namespace {

constexpr int kThreads = 512, kWarps = 16;
constexpr int kLaunchThreads = kThreads;
constexpr int kBlock = 64;     // tokens per KV block
constexpr int kRing = 16;      // conv ring depth
constexpr int kU = 8;          // (group, k-step) items in flight per lane (two 16-byte loads each)
constexpr int kTileLd = 9;     // padded row length of a warp's 16 x 8 accumulator tile in shared memory
constexpr int kMaxSplit = 64;
constexpr unsigned long long kBarWaitNs = 2000000000ull;

// Weight ring.  Barriers, prologues and mixers do not touch the weights, yet with plain loads the HBM
// stream stops at every one of them and has to ramp up again (~1-2 us per phase, ~130 phases per
// step).  With the ring every warp keeps its next few batches of weight fragments in flight into its
// own stages of shared memory with bulk asynchronous copies (cp.async.bulk, completion counted on an
// mbarrier): whenever it has consumed a batch it issues the copy of the batch `stages` ahead, and
// that look-ahead walks the step's whole schedule of projections, so before a warp enters a grid
// barrier the first batches of the NEXT projection are already under way and land while it waits.
// A stage holds one batch of one warp: kUR k-steps of its 16 A rows (two weight rows x k-slices), each
// row a contiguous run of kUR * 64 bytes, rows padded to 64 B mod 128 so that a warp's 16-byte fragment
// loads hit distinct banks.
constexpr int kUR = 4;                          // k-steps per ring batch
constexpr int kRowStride = kUR * 64 + 64;       // bytes between the 16 rows of a stage
constexpr int kStageBytes = 16 * kRowStride;    // 5120
constexpr int kMaxStages = 4;
constexpr int kMaxLayers = 96;

struct MegaLayer {
  const bf16* w_in; const bf16* w_out; const bf16* w_gu; const bf16* w_down;
  const float* in_gain; const float* post_gain;
  const float* conv_w; const float* A_log; const float* dt_bias; const float* norm_w;   // delta net
  const float* qg; const float* kg;                                                     // attention
  bf16* ring; float* state;       // delta net: [slots, 16, conv_dim], [slots, nv, dk, dv]
  bf16* kpool; bf16* vpool;       // attention: [pool slots, nkv, hd]
  int kind;                       // 0 = delta net, 1 = attention
  int n_in;                       // rows of w_in
};

struct MegaArgs {
  const MegaLayer* layers;
  const bf16* embed; const int64_t* tokens_in;
  const int* slots;
  const int* block_table;
  const float* cos; const float* sin;
  const float* final_gain; const bf16* lm_head;
  int64_t* tokens; int* positions; int* rope_pos;      // advanced in place when `advance` is set
  bf16* res0; bf16* res1;          // [M, H] residual stream, ping-pong
  float* h;                        // [M, H] output of the row-parallel projections
  bf16* proj;                      // [M, ld_proj]
  float* mix;                      // [M, mixw] mixer output before the output projection
  bf16* inter;                     // [M, I]
  float* part_o; float* part_ml;   // attention split partials [M, nh, nsplit, hd], [M, nh, nsplit, 2]
  float* logits;                   // [M, ld_logits] (local vocabulary slice)
  float* cand;                     // [grid, M, 2] per-CTA arg-max candidates
  int64_t* next;                   // [M]
  unsigned* bar;                   // [0] arrival counter, [1] its value when the kernel starts
  int* status;
  unsigned long long* trace;       // optional: %globaltimer of CTA 0 at every phase boundary (diagnostic)
  unsigned long long wait_ns;
  int n_layers, M, H, I, ld_proj, ld_logits, ldbt;
  int nk, nv, dk, dv, nh, nkv, rot, nsplit, vocab_local, vocab_total, vocab_off;
  int part_floats;                 // capacity of the partial-sum area in shared memory (floats)
  int xs_elems;                    // capacity of the activation area (bf16 elements)
  int advance;                     // 1: feed the sampled tokens back and advance the positions
  int use_res0;                    // 1: the step starts from res0 (a staged hidden state), not the embedding
  int prefetch;                    // > 0: KB per CTA of the next projection's slab requested into L2 before each barrier
  int tp_on;
  int hd;                          // attention head dim (the kernel's HD)
  int ring_stages;                 // 0: workers load weights themselves; 2..4: stages per warp of the weight ring
  float eps, scale_log2;
  TpComm tp;
};

// ------------------------------------------------------------------------------------------------
// small device helpers
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16(v)); }
// L2 load of one bf16 written earlier in this kernel by another CTA (L1 is not coherent across SMs)
__device__ __forceinline__ float ldcg_bf16(const bf16* p) {
  return __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(p))));
}

// CTA-wide barrier of the 512 threads.
__device__ __forceinline__ void cta_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }
__device__ __forceinline__ float wsum512(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_sum(v);
  cta_sync();
  if (lane == 0) red[w] = v;
  cta_sync();
  float t = (lane < kWarps) ? red[lane] : 0.f;
  return warp_sum(t);
}

struct Ctx {
  unsigned bar_target;     // counter value that completes the next barrier
  unsigned epoch;          // tensor-parallel epoch of this step
  int n_bar;               // barriers passed (every CTA passes the same number)
  int n_stamp;             // trace entries written
};
__device__ __forceinline__ void stamp(const MegaArgs& a, Ctx& c) {
  if (a.trace && blockIdx.x == 0 && threadIdx.x == 0) a.trace[c.n_stamp++] = tp_now_ns();
}

// Grid barrier: every CTA adds one to a monotonic counter and waits until it has reached this
// barrier's target.  Bounded: gives up after the limit (status 48) and never spins again once the
// status word is set, so a CTA that cannot make progress costs an error, not a hung GPU.
__device__ __forceinline__ void grid_barrier(const MegaArgs& a, Ctx& c) {
  cta_sync();
  c.bar_target += gridDim.x;
  c.n_bar += 1;
  if (threadIdx.x == 0) {
    // one release-add publishes everything this CTA wrote before the barrier (the CTA barrier above
    // orders the other threads' writes before it); the acquire loads below pair with the other CTAs' adds
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(a.bar), "r"(1u) : "memory");
    if (!tp_status_set(a.status)) {
      const unsigned long long limit = a.wait_ns ? a.wait_ns : kBarWaitNs;
      unsigned long long t0 = 0;
      unsigned spins = 0;
      while ((int)(ld_acquire_gpu(a.bar) - c.bar_target) < 0) {
        if ((++spins & 63u) == 0) {
          if (tp_status_set(a.status)) break;
          const unsigned long long now = tp_now_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > limit) { atomicCAS(a.status, 0, 48); break; }
        }
      }
    }
  }
  cta_sync();
}

// Ask the L2 for a contiguous slab (16-byte aligned, size a multiple of 16).  One thread.
__device__ __forceinline__ void l2_prefetch(const void* p, int64_t bytes, int64_t cap) {
  bytes = bytes > cap ? (cap & ~(int64_t)15) : bytes;
  while (bytes > 0) {
    const uint32_t n = (uint32_t)(bytes > (1 << 24) ? (1 << 24) : bytes);
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(n) : "memory");
    p = reinterpret_cast<const char*>(p) + n;
    bytes -= n;
  }
}

// ------------------------------------------------------------------------------------------------
// Projection phase.
struct Proj {
  const bf16* W;     // [rows_total, K]
  int rows_total;    // rows of W (loads are clamped to the last one)
  int K;
  int groups;        // work groups of the whole projection
  int rg;            // weight rows a group advances by (2M, or M with SwiGLU)
  int hi_base;       // row offset of the "high" half of the A tile (M, or I with SwiGLU)
  int mode;          // 0: bf16 out, 1: fp32 out (row-parallel, tensor-parallel exchange), 2: SwiGLU bf16 out, 3: fp32 logits + arg-max
  void* out; int ldo;
  int n_out;         // valid output columns (N, or I with SwiGLU)
  int site;          // tensor-parallel site (mode 1)
};

__device__ __forceinline__ int xs_pad(int Ks) { return ((Ks * 2) & 127) == 0 ? 32 : 0; }   // elements

__device__ __forceinline__ void proj_range(const Proj& p, int& G0, int& G1) {
  G0 = (int)((int64_t)blockIdx.x * p.groups / gridDim.x);
  G1 = (int)((int64_t)(blockIdx.x + 1) * p.groups / gridDim.x);
}

// Request this CTA's slab of a coming projection into L2 (called by one thread before a barrier).
__device__ __noinline__ void proj_prefetch(const Proj& p, int cap_kb) {
  const int64_t cap = (int64_t)cap_kb * 1024 / (p.mode == 2 ? 2 : 1);
  int G0, G1;
  proj_range(p, G0, G1);
  if (G1 <= G0) return;
  const bool swiglu = p.mode == 2;
  const int64_t r0 = (int64_t)G0 * p.rg, r1 = min((int64_t)G1 * p.rg, (int64_t)(swiglu ? p.hi_base : p.rows_total));
  if (r1 > r0) l2_prefetch(p.W + r0 * p.K, (r1 - r0) * p.K * 2, cap);
  if (swiglu && r1 > r0) l2_prefetch(p.W + (p.hi_base + r0) * p.K, (r1 - r0) * p.K * 2, cap);
}

// The activation rows are in shared memory, cut into M * S segments (batch row m, k-slice s) of
// K / S elements each, padded so that the eight segments a warp reads at once fall into distinct
// bank groups.
// The (group, k-step) items of one worker warp in one projection, cut into batches of at most `cap`
// k-steps that never cross a group.  The workers and the producer warp walk the same sequence.
struct BatchIter {
  int it, i1, gl, pb, P, G0, gl_first;
  __device__ __forceinline__ void init(const Proj& p, int M, int warp) {
    const int S = 8 / M, Ks = p.K / S;
    P = (Ks + 31) >> 5;
    int G1;
    proj_range(p, G0, G1);
    const int items = (G1 - G0) * P;
    const int ipw = (items + kWarps - 1) / kWarps;
    it = min(items, warp * ipw);
    i1 = min(items, it + ipw);
    gl = P ? it / P : 0;
    pb = it - gl * P;
    gl_first = gl;
  }
  __device__ __forceinline__ bool done() const { return it >= i1; }
  // next batch: `n` k-steps of group `gl` starting at step `pb`; seg_end: the warp's share of the group ends with it
  __device__ __forceinline__ void peek(int cap, int& n, bool& seg_end) const {
    const int pe = min(P, pb + (i1 - it));
    n = min(cap, pe - pb);
    seg_end = pb + n == pe;
  }
  __device__ __forceinline__ void advance(int n) {
    pb += n;
    it += n;
    if (pb == P) { pb = 0; ++gl; }
  }
};

struct Ring {
  unsigned char* base;      // [kWarps][stages][kStageBytes]
  uint64_t* full;           // [kWarps][kMaxStages]
  int stages;               // 0: off
  unsigned bc;              // batches this warp has consumed since the kernel started
  unsigned issued;          // batches whose copies it has issued
  int ph;                   // projection (in program order) the look-ahead is in
  bool active;              // the look-ahead has not reached the end of the step
  BatchIter it;             // look-ahead position
  Proj p;                   // its projection
};
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(sm100::smem_u32(dst)), "l"(src), "r"(bytes), "r"(sm100::smem_u32(bar)) : "memory");
}
// Bounded wait of a worker warp for its stage; gives up (status 49) after the limit and never spins
// once the status word is set.
__device__ __forceinline__ void ring_wait_full(const MegaArgs& a, uint64_t* bar, uint32_t parity) {
  if (sm100::mbar_try(bar, parity)) return;
  if (tp_status_set(a.status)) return;
  const unsigned long long t0 = tp_now_ns(), limit = a.wait_ns ? a.wait_ns : kBarWaitNs;
  unsigned spins = 0;
  while (!sm100::mbar_try(bar, parity)) {
    if ((++spins & 15u) == 0) {
      if (tp_status_set(a.status)) return;
      if (tp_now_ns() - t0 > limit) { atomicCAS(a.status, 0, 49); return; }
    }
  }
}

// Streaming half of a projection: this CTA's run of groups through the tensor cores, partial sums of
// every (warp, segment) left in shared memory.  Kept apart from the epilogue so that its registers
// are allocated for the hot loop alone.
// ------------------------------------------------------------------------------------------------
// The projections of a step in program order: 4 per layer (in, out, gate|up, down), then the head.
__device__ __forceinline__ Proj make_proj(const MegaArgs& a, const bf16* W, int rows_total, int K, int n_out, int mode,
                                          void* out, int ldo, int site) {
  Proj p;
  p.W = W; p.rows_total = rows_total; p.K = K; p.mode = mode; p.out = out; p.ldo = ldo; p.n_out = n_out; p.site = site;
  if (mode == 2) { p.rg = a.M; p.hi_base = n_out; p.groups = (n_out + a.M - 1) / a.M; }
  else { p.rg = 2 * a.M; p.hi_base = a.M; p.groups = (n_out + 2 * a.M - 1) / (2 * a.M); }
  return p;
}
__device__ __forceinline__ Proj proj_of(const MegaArgs& a, const MegaLayer* layers, int ph) {
  const int H = a.H;
  if (ph >= 4 * a.n_layers) return make_proj(a, a.lm_head, a.vocab_local, H, a.vocab_local, 3, a.logits, a.ld_logits, -1);
  const int li = ph >> 2, k = ph & 3;
  const MegaLayer& L = layers[li];
  const int mixw = L.kind == 0 ? a.nv * a.dv : a.nh * a.hd;
  if (k == 0) return make_proj(a, L.w_in, L.n_in, H, L.n_in, 0, a.proj, a.ld_proj, -1);
  if (k == 1) return make_proj(a, L.w_out, H, mixw, H, 1, a.h, H, 2 * li);
  if (k == 2) return make_proj(a, L.w_gu, 2 * a.I, H, a.I, 2, a.inter, a.I, -1);
  return make_proj(a, L.w_down, H, a.I, H, 1, a.h, H, 2 * li + 1);
}

// One step of a warp's look-ahead: issue the copies of its next batch (16 rows, one per lane 0..15) into
// the stage that batch will be read from, and move on, across projections, to the batch after it.
__device__ __forceinline__ void ring_settle(const MegaArgs& a, const MegaLayer* layers, Ring& r, int warp) {
  const int n_ph = 4 * a.n_layers + 1;
  while (r.active && r.it.done()) {
    if (++r.ph >= n_ph) { r.active = false; break; }
    r.p = proj_of(a, layers, r.ph);
    r.it.init(r.p, a.M, warp);
  }
}
__device__ __forceinline__ void ring_issue(const MegaArgs& a, const MegaLayer* layers, Ring& r, int warp, int lane) {
  if (!r.active) return;
  const int S = 8 / a.M, K = r.p.K, Ks = K / S;
  int n;
  bool seg_end;
  r.it.peek(kUR, n, seg_end);
  const unsigned st = r.issued % (unsigned)r.stages;
  const uint32_t row_bytes = (uint32_t)(min(n * 32, Ks - r.it.pb * 32) * 2);
  uint64_t* fullb = r.full + warp * kMaxStages + st;
  if (lane == 0) sm100::mbar_expect_tx(fullb, 16u * row_bytes);
  __syncwarp();
  if (lane < 16) {
    const int g = lane & 7, hi = lane >> 3;
    const int64_t rbase = (int64_t)(r.it.G0 + r.it.gl) * r.p.rg + g / S + (hi ? r.p.hi_base : 0);
    const int64_t row = min(rbase, (int64_t)r.p.rows_total - 1);
    const bf16* src = r.p.W + row * K + (int64_t)(g % S) * Ks + r.it.pb * 32;
    unsigned char* dst = r.base + ((size_t)warp * r.stages + st) * kStageBytes + lane * kRowStride;
    bulk_g2s(dst, src, row_bytes, fullb);
  }
  r.it.advance(n);
  r.issued += 1;
  ring_settle(a, layers, r, warp);
}

__device__ __forceinline__ void proj_flush(const float* acc, float* tile, float* dst, int M, int S, int MM2, int lane, int g, int t) {
  // C[i][n] pairs weight-row slot / slice of A row i with batch row / slice of B column n; the products
  // of equal slices are the k-slices of one output
  tile[g * kTileLd + 2 * t] = acc[0];
  tile[g * kTileLd + 2 * t + 1] = acc[1];
  tile[(g + 8) * kTileLd + 2 * t] = acc[2];
  tile[(g + 8) * kTileLd + 2 * t + 1] = acc[3];
  __syncwarp();
  for (int o = lane; o < MM2; o += 32) {
    const int wr = o / M, m = o % M;
    const int ib = wr < M ? wr * S : 8 + (wr - M) * S, nb = m * S;
    float v = 0.f;
    for (int sidx = 0; sidx < S; ++sidx) v += tile[(ib + sidx) * kTileLd + nb + sidx];
    dst[o] = v;
  }
  __syncwarp();
}

__device__ __noinline__ void proj_stream(const MegaArgs& a, const MegaLayer* layers, const Proj& p, const bf16* xs, float* part,
                                         float* tile_s, Ring& ring) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int M = a.M, S = 8 / M, K = p.K, Ks = K / S, MM2 = 2 * M * M;   // Ks: a multiple of 8
  const int seg_ld = Ks + xs_pad(Ks);
  BatchIter bi;
  bi.init(p, M, warp);
  int G0, G1;
  proj_range(p, G0, G1);
  const int items = (G1 - G0) * bi.P;
  const int ipw2 = (items + kWarps - 1) / kWarps;
  const int maxseg = ipw2 > 0 ? (ipw2 + bi.P - 1) / bi.P + 1 : 1;
  const int wr_lo = g / S, sl = g % S;
  const int64_t lane_koff = (int64_t)sl * Ks + t * 8;
  const bf16* xlane = xs + (int64_t)g * seg_ld + t * 8;
  float* tile = tile_s + warp * 16 * kTileLd;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (ring.stages > 0) {
    // ---- weights arrive through this warp's stages of the ring ---------------------------------------
    while (!bi.done()) {
      int n;
      bool seg_end;
      bi.peek(kUR, n, seg_end);
      const unsigned st = ring.bc % (unsigned)ring.stages, par = (ring.bc / (unsigned)ring.stages) & 1u;
      ring_wait_full(a, ring.full + warp * kMaxStages + st, par);
      const unsigned char* sb = ring.base + ((size_t)warp * ring.stages + st) * kStageBytes;
#pragma unroll
      for (int u = 0; u < kUR; ++u) {
        const int q = bi.pb + u;
        const bool ok = u < n && q * 32 + t * 8 < Ks;
        const uint4 lo = ok ? *reinterpret_cast<const uint4*>(sb + g * kRowStride + u * 64 + t * 16) : zero;
        const uint4 hi = ok ? *reinterpret_cast<const uint4*>(sb + (g + 8) * kRowStride + u * 64 + t * 16) : zero;
        const uint4 xv = ok ? *reinterpret_cast<const uint4*>(xlane + q * 32) : zero;
        mma16816(acc, lo.x, hi.x, lo.y, hi.y, xv.x, xv.y);
        mma16816(acc, lo.z, hi.z, lo.w, hi.w, xv.z, xv.w);
      }
      __syncwarp();                 // every lane has its fragments: the stage may be refilled
      ring.bc += 1;
      ring_issue(a, layers, ring, warp, lane);
      if (seg_end) {
        proj_flush(acc, tile, part + ((int64_t)warp * maxseg + (bi.gl - bi.gl_first)) * MM2, M, S, MM2, lane, g, t);
        acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
      }
      bi.advance(n);
    }
    return;
  }
  // ---- the warp loads its weights itself: kU pairs of 16-byte loads issued before the first multiply ----
  while (!bi.done()) {
    int n;
    bool seg_end;
    bi.peek(kU, n, seg_end);
    const int64_t rbase = (int64_t)(bi.G0 + bi.gl) * p.rg + wr_lo;
    const bf16* wlo = p.W + min(rbase, (int64_t)p.rows_total - 1) * K + lane_koff;
    const bf16* whi = p.W + min(rbase + p.hi_base, (int64_t)p.rows_total - 1) * K + lane_koff;
    uint4 lo[kU], hi[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int q = bi.pb + u;
      // past the batch, or in the ragged last k-step of a slice (Ks not a multiple of 32): zeros
      const bool ok = u < n && q * 32 + t * 8 < Ks;
      lo[u] = ok ? ld_stream(wlo + q * 32) : zero;
      hi[u] = ok ? ld_stream(whi + q * 32) : zero;
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int q = bi.pb + u;
      const bool ok = u < n && q * 32 + t * 8 < Ks;
      const uint4 xv = ok ? *reinterpret_cast<const uint4*>(xlane + q * 32) : zero;
      mma16816(acc, lo[u].x, hi[u].x, lo[u].y, hi[u].y, xv.x, xv.y);
      mma16816(acc, lo[u].z, hi[u].z, lo[u].w, hi[u].w, xv.z, xv.w);
    }
    if (seg_end) {
      proj_flush(acc, tile, part + ((int64_t)warp * maxseg + (bi.gl - bi.gl_first)) * MM2, M, S, MM2, lane, g, t);
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
    }
    bi.advance(n);
  }
}

__device__ __noinline__ void proj_run(const MegaArgs& a, const Ctx& c, const Proj& p, const bf16* xs, float* part, float* tile_s,
                         float* red, Ring& ring, const MegaLayer* layers) {
  proj_stream(a, layers, p, xs, part, tile_s, ring);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int M = a.M, S = 8 / M, Ks = p.K / S, P = (Ks + 31) >> 5, MM2 = 2 * M * M;
  int G0, G1;
  proj_range(p, G0, G1);
  const int ng = G1 - G0, items = ng * P;
  const int ipw = (items + kWarps - 1) / kWarps;
  const int maxseg = ipw > 0 ? (ipw + P - 1) / P + 1 : 1;
  cta_sync();
  // ---- finalise: fixed-order sum over the warps that touched a group, then the epilogue ----------
  auto group_sum = [&](int gl, int r) -> float {
    const int w0 = (gl * P) / ipw, w1 = (gl * P + P - 1) / ipw;
    float v = 0.f;
    for (int w = w0; w <= w1; ++w) v += part[((int64_t)w * maxseg + (gl - (w * ipw) / P)) * MM2 + r];
    return v;
  };
  if (p.mode == 2) {
    bf16* out = reinterpret_cast<bf16*>(p.out);
    for (int o = tid; o < ng * M * M; o += kThreads) {
      const int gl = o / (M * M), r = o % (M * M), j = r / M, m = r % M;
      const int col = (G0 + gl) * M + j;
      if (col < p.n_out) {
        const float gate = group_sum(gl, r), up = group_sum(gl, r + M * M);
        out[(int64_t)m * p.ldo + col] = __float2bfloat16(silu_f(gate) * up);
      }
    }
  } else if (p.mode == 3) {
    float* out = reinterpret_cast<float*>(p.out);
    float best[8];
    int bidx[8];
#pragma unroll
    for (int m = 0; m < 8; ++m) { best[m] = -INFINITY; bidx[m] = 0x7fffffff; }
    for (int o = tid; o < ng * MM2; o += kThreads) {
      const int gl = o / MM2, r = o % MM2, wr = r / M, m = r % M;
      const int col = (G0 + gl) * 2 * M + wr;
      if (col < p.n_out) {
        const float v = group_sum(gl, r);
        out[(int64_t)m * p.ldo + col] = v;
#pragma unroll
        for (int mm = 0; mm < 8; ++mm)
          if (mm == m && (v > best[mm] || (v == best[mm] && col < bidx[mm]))) { best[mm] = v; bidx[mm] = col; }
      }
    }
    // CTA-wide arg-max per batch row (ties to the lowest index)
    float* cv = red;                     // [kWarps][8] values, then [kWarps][8] indices
    int* ci = reinterpret_cast<int*>(red + kWarps * 8);
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      float v = best[m];
      int ix = bidx[m];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, off);
        const int oi = __shfl_xor_sync(0xffffffffu, ix, off);
        if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
      }
      if (lane == 0) { cv[warp * 8 + m] = v; ci[warp * 8 + m] = ix; }
    }
    cta_sync();
    if (tid < M) {
      float v = -INFINITY;
      int ix = 0x7fffffff;
      for (int w = 0; w < kWarps; ++w) {
        const float ov = cv[w * 8 + tid];
        const int oi = ci[w * 8 + tid];
        if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
      }
      a.cand[((int64_t)blockIdx.x * M + tid) * 2] = v;
      a.cand[((int64_t)blockIdx.x * M + tid) * 2 + 1] = __int_as_float(ix);
    }
  } else {
    for (int o = tid; o < ng * MM2; o += kThreads) {
      const int gl = o / MM2, r = o % MM2, wr = r / M, m = r % M;
      const int col = (G0 + gl) * 2 * M + wr;
      if (col < p.n_out) {
        float v = group_sum(gl, r);
        if (p.mode == 0) {
          reinterpret_cast<bf16*>(p.out)[(int64_t)m * p.ldo + col] = __float2bfloat16(v);
        } else {
          if (a.tp_on) {
            // all-reduce inside the epilogue: store the partial value on every rank, then add the ranks'
            // values of this element in rank order (bounded wait on the data-carried epochs)
            const int64_t off = (int64_t)m * p.n_out + col;
            const int64_t elem = ((int64_t)p.site * a.tp.world + a.tp.rank) * a.tp.slot_floats + off;
#pragma unroll
            for (int q = 0; q < kTpMaxWorld; ++q)
              if (q < a.tp.world) tp_st_pair(a.tp.inbox[q], elem, v, c.epoch);
            float s = 0.f;
            for (int r2 = 0; r2 < a.tp.world; ++r2) {
              const int64_t e2 = ((int64_t)p.site * a.tp.world + r2) * a.tp.slot_floats + off;
              unsigned long long pv = tp_ld_pair(a.tp.my_inbox, e2);
              if ((unsigned)(pv >> 32) != c.epoch && !tp_status_set(a.status)) {
                const unsigned long long t0 = tp_now_ns(), limit = a.tp.wait_ns ? a.tp.wait_ns : kTpWaitNs;
                unsigned spins = 0;
                while ((unsigned)(pv >> 32) != c.epoch) {
                  if ((++spins & 63u) == 0) {
                    if (tp_status_set(a.status)) break;
                    if (tp_now_ns() - t0 > limit) { atomicCAS(a.status, 0, 16 + r2); break; }
                  }
                  pv = tp_ld_pair(a.tp.my_inbox, e2);
                }
              }
              s += __uint_as_float((unsigned)pv);
            }
            v = s;
          }
          reinterpret_cast<float*>(p.out)[(int64_t)m * p.ldo + col] = v;
        }
      }
    }
  }
}

// Element k of batch row m in the segmented activation layout.
__device__ __forceinline__ int xs_index(int m, int k, int S, int Ks, int seg_ld) {
  return (m * S + k / Ks) * seg_ld + k % Ks;
}

// Prologue of in-proj / gate-up / lm_head: x = RMSNorm(res_in + add) * gain into shared memory; CTA 0
// also writes the new residual.  `res_in` rows may come from the embedding table (`tok` != null).
__device__ __noinline__ void prologue_norm(const MegaArgs& a, const bf16* res_in, const int64_t* tok, const float* add,
                              const float* gain, bf16* res_out, int K, bf16* xs, float* red) {
  const int tid = threadIdx.x, M = a.M, S = 8 / M, Ks = K / S, seg_ld = Ks + xs_pad(Ks);
  const int nchunk = K >> 3;
  for (int m = 0; m < M; ++m) {
    const bf16* src = res_in + (int64_t)m * K;
    if (tok) {
      int64_t tk = tok[m];
      tk = tk < 0 ? 0 : (tk >= a.vocab_total ? a.vocab_total - 1 : tk);
      src = a.embed + tk * K;
    }
    if (nchunk <= kThreads) {
      // one 8-element chunk per thread: residual, addend and gain are requested together and the row
      // stays in registers between the sum of squares and the scaling (one pass, one reduction)
      const bool ok = tid < nchunk;
      float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float4 g0 = make_float4(0.f, 0.f, 0.f, 0.f), g1 = g0;
      if (ok) {
        const uint4 rv = __ldcg(reinterpret_cast<const uint4*>(src + tid * 8));
        float4 q0 = make_float4(0.f, 0.f, 0.f, 0.f), q1 = q0;
        if (add) {
          q0 = __ldcg(reinterpret_cast<const float4*>(add + (int64_t)m * K + tid * 8));
          q1 = __ldcg(reinterpret_cast<const float4*>(add + (int64_t)m * K + tid * 8 + 4));
        }
        g0 = *reinterpret_cast<const float4*>(gain + tid * 8);
        g1 = *reinterpret_cast<const float4*>(gain + tid * 8 + 4);
        bf16x8_to_float(rv, f);
        if (add) {
          f[0] = round_bf16(f[0] + q0.x); f[1] = round_bf16(f[1] + q0.y); f[2] = round_bf16(f[2] + q0.z); f[3] = round_bf16(f[3] + q0.w);
          f[4] = round_bf16(f[4] + q1.x); f[5] = round_bf16(f[5] + q1.y); f[6] = round_bf16(f[6] + q1.z); f[7] = round_bf16(f[7] + q1.w);
        }
        if (res_out && blockIdx.x == 0) *reinterpret_cast<uint4*>(res_out + (int64_t)m * K + tid * 8) = float_to_bf16x8(f);
      }
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
      const float rstd = rsqrtf(wsum512(ss, red) / (float)K + a.eps);
      if (ok) {
        f[0] *= rstd * g0.x; f[1] *= rstd * g0.y; f[2] *= rstd * g0.z; f[3] *= rstd * g0.w;
        f[4] *= rstd * g1.x; f[5] *= rstd * g1.y; f[6] *= rstd * g1.z; f[7] *= rstd * g1.w;
        *reinterpret_cast<uint4*>(xs + xs_index(m, tid * 8, S, Ks, seg_ld)) = float_to_bf16x8(f);
      }
      continue;
    }
    float ss = 0.f;
    for (int cidx = tid; cidx < nchunk; cidx += kThreads) {
      float f[8];
      bf16x8_to_float(__ldcg(reinterpret_cast<const uint4*>(src + cidx * 8)), f);
      if (add) {
        const float4 q0 = __ldcg(reinterpret_cast<const float4*>(add + (int64_t)m * K + cidx * 8));
        const float4 q1 = __ldcg(reinterpret_cast<const float4*>(add + (int64_t)m * K + cidx * 8 + 4));
        f[0] = round_bf16(f[0] + q0.x); f[1] = round_bf16(f[1] + q0.y); f[2] = round_bf16(f[2] + q0.z); f[3] = round_bf16(f[3] + q0.w);
        f[4] = round_bf16(f[4] + q1.x); f[5] = round_bf16(f[5] + q1.y); f[6] = round_bf16(f[6] + q1.z); f[7] = round_bf16(f[7] + q1.w);
      }
      const uint4 packed = float_to_bf16x8(f);
      *reinterpret_cast<uint4*>(xs + xs_index(m, cidx * 8, S, Ks, seg_ld)) = packed;
      if (res_out && blockIdx.x == 0) *reinterpret_cast<uint4*>(res_out + (int64_t)m * K + cidx * 8) = packed;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    const float rstd = rsqrtf(wsum512(ss, red) / (float)K + a.eps);
    for (int cidx = tid; cidx < nchunk; cidx += kThreads) {
      float f[8];
      uint4* px = reinterpret_cast<uint4*>(xs + xs_index(m, cidx * 8, S, Ks, seg_ld));
      bf16x8_to_float(*px, f);
      const float4 g0 = *reinterpret_cast<const float4*>(gain + cidx * 8);
      const float4 g1 = *reinterpret_cast<const float4*>(gain + cidx * 8 + 4);
      f[0] *= rstd * g0.x; f[1] *= rstd * g0.y; f[2] *= rstd * g0.z; f[3] *= rstd * g0.w;
      f[4] *= rstd * g1.x; f[5] *= rstd * g1.y; f[6] *= rstd * g1.z; f[7] *= rstd * g1.w;
      *px = float_to_bf16x8(f);
    }
  }
  cta_sync();
}

// Prologue of the delta-net output projection: gated RMSNorm over each value head of the raw mixer
// output (fp32), times silu(z) with z from the input projection (q | k | v | z | b | a).
__device__ __noinline__ void prologue_gdn_act(const MegaArgs& a, const MegaLayer& L, bf16* xs) {
  const int tid = threadIdx.x, M = a.M, S = 8 / M, K = a.nv * a.dv, Ks = K / S, seg_ld = Ks + xs_pad(Ks);
  const int n8 = K >> 3, lph = a.dv >> 3;             // chunks per row; chunks (= lanes) per head
  const int conv_dim = 2 * a.nk * a.dk + a.nv * a.dv;
  for (int m = 0; m < M; ++m) {
    for (int base = 0; base < n8; base += kThreads) {
      const int idx = base + tid;
      const bool ok = idx < n8;
      float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (ok) {
        const float4 q0 = __ldcg(reinterpret_cast<const float4*>(a.mix + (int64_t)m * K + idx * 8));
        const float4 q1 = __ldcg(reinterpret_cast<const float4*>(a.mix + (int64_t)m * K + idx * 8 + 4));
        f[0] = q0.x; f[1] = q0.y; f[2] = q0.z; f[3] = q0.w; f[4] = q1.x; f[5] = q1.y; f[6] = q1.z; f[7] = q1.w;
      }
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
      for (int off = lph >> 1; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
      if (ok) {
        const int col = idx * 8, j = col % a.dv;
        const float r = rsqrtf(ss / (float)a.dv + a.eps);
        float zf[8];
        bf16x8_to_float(__ldcg(reinterpret_cast<const uint4*>(a.proj + (int64_t)m * a.ld_proj + conv_dim + col)), zf);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = f[i] * r * L.norm_w[j + i] * silu_f(zf[i]);
        *reinterpret_cast<uint4*>(xs + xs_index(m, col, S, Ks, seg_ld)) = float_to_bf16x8(f);
      }
    }
  }
  cta_sync();
}

// Prologue that copies fp32 rows (merged attention output) or bf16 rows (SwiGLU output) into the
// segmented activation layout.
__device__ __noinline__ void prologue_copy_f32(const MegaArgs& a, const float* src, int K, bf16* xs) {
  const int M = a.M, S = 8 / M, Ks = K / S, seg_ld = Ks + xs_pad(Ks), n8 = K >> 3;
  for (int i = threadIdx.x; i < M * n8; i += kThreads) {
    const int m = i / n8, col = (i % n8) * 8;
    const float4 q0 = __ldcg(reinterpret_cast<const float4*>(src + (int64_t)m * K + col));
    const float4 q1 = __ldcg(reinterpret_cast<const float4*>(src + (int64_t)m * K + col + 4));
    const float f[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    *reinterpret_cast<uint4*>(xs + xs_index(m, col, S, Ks, seg_ld)) = float_to_bf16x8(f);
  }
  cta_sync();
}
__device__ __noinline__ void prologue_copy_bf16(const MegaArgs& a, const bf16* src, int64_t lds, int K, bf16* xs) {
  const int M = a.M, S = 8 / M, Ks = K / S, seg_ld = Ks + xs_pad(Ks), n8 = K >> 3;
  for (int i = threadIdx.x; i < M * n8; i += kThreads) {
    const int m = i / n8, col = (i % n8) * 8;
    *reinterpret_cast<uint4*>(xs + xs_index(m, col, S, Ks, seg_ld)) =
        __ldcg(reinterpret_cast<const uint4*>(src + (int64_t)m * lds + col));
  }
  cta_sync();
}

// ------------------------------------------------------------------------------------------------
// Delta-net step.  A unit is (batch row, value head, block of 32 value columns): 16 warps = 16 groups
// of DK/16 state rows, a lane owns one column.  The gated norm over the whole head is left to the
// output projection's prologue, so the columns of a head can be spread over CTAs.
template <int DK>
__device__ __noinline__ void gdn_phase(const MegaArgs& a, const MegaLayer& L, float* sm) {
  constexpr int RPT = DK / kWarps;
  const int tid = threadIdx.x, j = tid & 31, rg = tid >> 5;
  const int DV = a.dv, ncb = DV >> 5, rep = a.nv / a.nk;
  const int kdim = a.nk * DK, conv_dim = 2 * kdim + a.nv * DV;
  float* q_s = sm;                  // [DK]
  float* k_s = q_s + DK;            // [DK]
  float* v_s = k_s + DK;            // [32]
  float* scal = v_s + 32;           // [4]
  float* sk = scal + 4;             // [kWarps][32]
  float* sq = sk + kWarps * 32;     // [kWarps][32]
  const int units = a.M * a.nv * ncb;
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int m = u / (a.nv * ncb), h = (u / ncb) % a.nv, cb = u % ncb, kh = h / rep;
    const int slot = a.slots[m];
    if (slot < 0) continue;                       // padded row (uniform over the CTA)
    const int pos = a.positions[m];
    float* sp = L.state + (((int64_t)slot * a.nv + h) * DK + rg * RPT) * DV + cb * 32 + j;
    float s[RPT];
#pragma unroll
    for (int r = 0; r < RPT; ++r) s[r] = __ldcg(sp + (int64_t)r * DV);
    const bf16* prow = a.proj + (int64_t)m * a.ld_proj;
    bf16* ring = L.ring + (int64_t)slot * kRing * conv_dim;
    // ---- causal conv + SiLU on this unit's q, k (whole key head) and v (32 columns) channels -----
    if (tid < 2 * DK + 32) {
      int ch;
      bool own;
      if (tid < DK) { ch = kh * DK + tid; own = (h % rep) == 0 && cb == 0; }
      else if (tid < 2 * DK) { ch = kdim + kh * DK + (tid - DK); own = (h % rep) == 0 && cb == 0; }
      else { ch = 2 * kdim + h * DV + cb * 32 + (tid - 2 * DK); own = true; }
      const float4 w = *reinterpret_cast<const float4*>(L.conv_w + (int64_t)ch * 4);
      const float xn = ldcg_bf16(prow + ch);
      float x1 = 0.f, x2 = 0.f, x3 = 0.f;
      if (pos >= 1) x1 = ldcg_bf16(ring + (int64_t)((pos - 1) & (kRing - 1)) * conv_dim + ch);
      if (pos >= 2) x2 = ldcg_bf16(ring + (int64_t)((pos - 2) & (kRing - 1)) * conv_dim + ch);
      if (pos >= 3) x3 = ldcg_bf16(ring + (int64_t)((pos - 3) & (kRing - 1)) * conv_dim + ch);
      const float v = silu_f(w.x * x3 + w.y * x2 + w.z * x1 + w.w * xn);
      if (own) ring[(int64_t)(pos & (kRing - 1)) * conv_dim + ch] = __float2bfloat16(xn);   // exact: xn is a bf16 value
      if (tid < DK) q_s[tid] = v;
      else if (tid < 2 * DK) k_s[tid - DK] = v;
      else v_s[tid - 2 * DK] = v;
    }
    cta_sync();
    if (tid < 96) {
      const int w = tid >> 5;
      float acc = 0.f;
      for (int i = j; i < DK; i += 32) {
        const float qa = q_s[i], ka = k_s[i];
        acc += (w == 0) ? qa * qa : (w == 1) ? ka * ka : qa * ka;
      }
      acc = warp_sum(acc);
      if (j == 0) scal[w] = acc;
    }
    float pk = 0.f, pq = 0.f;
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      pk = fmaf(s[r], k_s[rg * RPT + r], pk);
      pq = fmaf(s[r], q_s[rg * RPT + r], pq);
    }
    sk[rg * 32 + j] = pk;
    sq[rg * 32 + j] = pq;
    cta_sync();
    const float rq = rsqrtf(scal[0] + 1e-6f) * rsqrtf((float)DK), rk = rsqrtf(scal[1] + 1e-6f);
    const float kq = scal[2] * rq * rk;
    const float bl = ldcg_bf16(prow + conv_dim + a.nv * DV + h);
    const float al = ldcg_bf16(prow + conv_dim + a.nv * DV + a.nv + h);
    const float beta = sigmoid_f(bl);
    const float alpha = __expf(-__expf(L.A_log[h]) * softplus_f(al + L.dt_bias[h]));
    float Sk = 0.f, Sq = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) { Sk += sk[w * 32 + j]; Sq += sq[w * 32 + j]; }
    Sk *= rk;
    Sq *= rq;
    const float d = (v_s[j] - alpha * Sk) * beta;
    const float o = alpha * Sq + kq * d;
#pragma unroll
    for (int r = 0; r < RPT; ++r) sp[(int64_t)r * DV] = fmaf(k_s[rg * RPT + r] * rk, d, alpha * s[r]);
    if (rg == 0) a.mix[(int64_t)m * a.nv * DV + h * DV + cb * 32 + j] = o;
    cta_sync();
  }
}

// ------------------------------------------------------------------------------------------------
// Attention, first half: one unit per (batch row, kv head, key split).  Key tiles of 64 are strided
// over the splits; the split that owns the tile holding the current position first norms, rotates and
// appends this token's K/V.  16 warps take 4 keys each per iteration, merge pairwise through shared
// memory and leave one partial (o, m, l) per query head.
template <int HD>
__device__ __forceinline__ void norm_rope_lane(float* x, const float* gain, const float* cs, const float* sn, int rot,
                                               float eps, int lane) {
  constexpr int EPL = HD / 32;
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < EPL; ++e) ss += x[e] * x[e];
  const float r = rsqrtf(warp_sum(ss) / (float)HD + eps);
#pragma unroll
  for (int e = 0; e < EPL; ++e) x[e] *= r * gain[lane * EPL + e];
  const int half = rot >> 1, plane = half / EPL;
#pragma unroll
  for (int e = 0; e < EPL; ++e) {
    const float other = __shfl_xor_sync(0xffffffffu, x[e], plane);
    const int i = lane * EPL + e;
    if (i < rot) {
      const float cc = cs[i], s = sn[i];
      x[e] = (i < half) ? x[e] * cc - other * s : x[e] * cc + other * s;
    }
  }
}
template <int EPL>
__device__ __forceinline__ void kv_load(const bf16* p, uint32_t* w) {
  if (EPL == 8) {
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(p));
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
  } else {
#pragma unroll
    for (int e = 0; e < EPL / 2; ++e) w[e] = __ldcg(reinterpret_cast<const uint32_t*>(p) + e);
  }
}

template <int HD, int REP>
__device__ __noinline__ void attn_phase(const MegaArgs& a, const MegaLayer& L, float* sm) {
  constexpr int EPL = HD / 32, WPL = EPL / 2, KPW = 4;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* q_s = sm;                                   // [REP][HD]
  float* mo = q_s + REP * HD;                        // [kWarps / 2][REP][HD]
  float* mml = mo + (kWarps / 2) * REP * HD;         // [kWarps / 2][REP][2]
  const int ns = a.nsplit, units = a.M * a.nkv * ns;
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int m = u / (a.nkv * ns), kvh = (u / ns) % a.nkv, split = u % ns;
    const int pos = a.positions[m];
    float* po = a.part_o + (((int64_t)m * a.nh + kvh * REP) * ns + split) * HD;
    float* pml = a.part_ml + (((int64_t)m * a.nh + kvh * REP) * ns + split) * 2;
    if (pos < 0) {                                   // padded row: an empty partial
      for (int i = tid; i < REP * 2; i += kThreads) pml[(int64_t)(i >> 1) * ns * 2 + (i & 1)] = (i & 1) ? 0.f : -INFINITY;
      continue;
    }
    const bf16* prow = a.proj + (int64_t)m * a.ld_proj;
    const int rp = a.rope_pos[m];
    const float* cs = a.cos + (int64_t)rp * a.rot;
    const float* sn = a.sin + (int64_t)rp * a.rot;
    const int* bt = a.block_table + (int64_t)m * a.ldbt;
    for (int r = warp; r < REP; r += kWarps) {
      float x[EPL];
      const bf16* src = prow + (int64_t)(kvh * REP + r) * 2 * HD + lane * EPL;
      uint32_t raw[WPL];
      kv_load<EPL>(src, raw);
#pragma unroll
      for (int e = 0; e < WPL; ++e) { x[2 * e] = bf_lo(raw[e]); x[2 * e + 1] = bf_hi(raw[e]); }
      norm_rope_lane<HD>(x, L.qg, cs, sn, a.rot, a.eps, lane);
#pragma unroll
      for (int e = 0; e < EPL; ++e) q_s[r * HD + lane * EPL + e] = x[e] * a.scale_log2;
    }
    if ((pos / kBlock) % ns == split) {
      const int64_t slot = (int64_t)bt[pos / kBlock] * kBlock + pos % kBlock;
      if (warp == kWarps - 1) {
        float x[EPL];
        uint32_t raw[WPL];
        kv_load<EPL>(prow + (int64_t)a.nh * 2 * HD + (int64_t)kvh * HD + lane * EPL, raw);
#pragma unroll
        for (int e = 0; e < WPL; ++e) { x[2 * e] = bf_lo(raw[e]); x[2 * e + 1] = bf_hi(raw[e]); }
        norm_rope_lane<HD>(x, L.kg, cs, sn, a.rot, a.eps, lane);
        uint32_t* dst = reinterpret_cast<uint32_t*>(L.kpool + (slot * a.nkv + kvh) * HD + lane * EPL);
#pragma unroll
        for (int e = 0; e < WPL; ++e) dst[e] = pack_bf162(x[2 * e], x[2 * e + 1]);
      } else if (warp == kWarps - 2) {
        uint32_t raw[WPL];
        kv_load<EPL>(prow + (int64_t)a.nh * 2 * HD + (int64_t)(a.nkv + kvh) * HD + lane * EPL, raw);
        uint32_t* dst = reinterpret_cast<uint32_t*>(L.vpool + (slot * a.nkv + kvh) * HD + lane * EPL);
#pragma unroll
        for (int e = 0; e < WPL; ++e) dst[e] = raw[e];
      }
      __threadfence_block();
    }
    cta_sync();
    float q[REP][EPL], o[REP][EPL], mx[REP], l[REP];
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      mx[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) { q[r][e] = q_s[r * HD + lane * EPL + e]; o[r][e] = 0.f; }
    }
    const int ntiles = pos / kBlock + 1;
    const int nloc = split < ntiles ? (ntiles - 1 - split) / ns + 1 : 0;
    const int nj = nloc * kBlock;
    const int niter = (nj + kWarps * KPW - 1) / (kWarps * KPW);
    for (int it = 0; it < niter; ++it) {
      uint32_t kf[KPW][WPL], vf[KPW][WPL];
      bool okk[KPW];
#pragma unroll
      for (int uu = 0; uu < KPW; ++uu) {
        const int jj = it * (kWarps * KPW) + warp * KPW + uu;
        const int kt = split + (jj / kBlock) * ns, i = jj % kBlock;
        okk[uu] = jj < nj && kt * kBlock + i <= pos;
        if (okk[uu]) {
          const int64_t row = ((int64_t)bt[kt] * kBlock + i) * a.nkv + kvh;
          kv_load<EPL>(L.kpool + row * HD + lane * EPL, kf[uu]);
          kv_load<EPL>(L.vpool + row * HD + lane * EPL, vf[uu]);
        }
      }
#pragma unroll
      for (int r = 0; r < REP; ++r) {
        float d[KPW];
#pragma unroll
        for (int uu = 0; uu < KPW; ++uu) {
          float sdot = 0.f;
          if (okk[uu]) {
#pragma unroll
            for (int e = 0; e < WPL; ++e) {
              sdot = fmaf(q[r][2 * e], bf_lo(kf[uu][e]), sdot);
              sdot = fmaf(q[r][2 * e + 1], bf_hi(kf[uu][e]), sdot);
            }
          }
          d[uu] = sdot;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
          for (int uu = 0; uu < KPW; ++uu) d[uu] += __shfl_xor_sync(0xffffffffu, d[uu], off);
        }
        float mn = mx[r];
#pragma unroll
        for (int uu = 0; uu < KPW; ++uu) {
          if (!okk[uu]) d[uu] = -INFINITY;
          mn = fmaxf(mn, d[uu]);
        }
        if (mn == -INFINITY) continue;
        const float cc = exp2f(mx[r] - mn);
        float pw[KPW], ps = 0.f;
#pragma unroll
        for (int uu = 0; uu < KPW; ++uu) { pw[uu] = exp2f(d[uu] - mn); ps += pw[uu]; }
        l[r] = l[r] * cc + ps;
        mx[r] = mn;
#pragma unroll
        for (int e = 0; e < WPL; ++e) {
          float a0 = o[r][2 * e] * cc, a1 = o[r][2 * e + 1] * cc;
#pragma unroll
          for (int uu = 0; uu < KPW; ++uu)
            if (okk[uu]) { a0 = fmaf(pw[uu], bf_lo(vf[uu][e]), a0); a1 = fmaf(pw[uu], bf_hi(vf[uu][e]), a1); }
          o[r][2 * e] = a0; o[r][2 * e + 1] = a1;
        }
      }
    }
    // ---- merge the 16 warps pairwise through shared memory ---------------------------------------
#pragma unroll
    for (int step = kWarps / 2; step > 0; step >>= 1) {
      if (warp >= step && warp < 2 * step) {
#pragma unroll
        for (int r = 0; r < REP; ++r) {
#pragma unroll
          for (int e = 0; e < EPL; ++e) mo[((warp - step) * REP + r) * HD + lane * EPL + e] = o[r][e];
          if (lane == 0) { mml[((warp - step) * REP + r) * 2] = mx[r]; mml[((warp - step) * REP + r) * 2 + 1] = l[r]; }
        }
      }
      cta_sync();
      if (warp < step) {
#pragma unroll
        for (int r = 0; r < REP; ++r) {
          const float m2 = mml[(warp * REP + r) * 2], l2 = mml[(warp * REP + r) * 2 + 1];
          const float mn = fmaxf(mx[r], m2);
          const float c1 = mn == -INFINITY ? 0.f : exp2f(mx[r] - mn);
          const float c2 = mn == -INFINITY ? 0.f : exp2f(m2 - mn);
#pragma unroll
          for (int e = 0; e < EPL; ++e) o[r][e] = o[r][e] * c1 + mo[(warp * REP + r) * HD + lane * EPL + e] * c2;
          l[r] = l[r] * c1 + l2 * c2;
          mx[r] = mn;
        }
      }
      cta_sync();
    }
    if (warp == 0) {
#pragma unroll
      for (int r = 0; r < REP; ++r) {
#pragma unroll
        for (int e = 0; e < EPL; ++e) po[(int64_t)r * ns * HD + lane * EPL + e] = o[r][e];
        if (lane == 0) {
          pml[(int64_t)r * ns * 2] = mx[r];
          pml[(int64_t)r * ns * 2 + 1] = l[r];
        }
      }
    }
    cta_sync();
  }
}

// Attention, second half: one unit per (batch row, query head) merges the split partials, applies the
// sigmoid output gate and writes the fp32 row that the output projection's prologue converts.
template <int HD>
__device__ __noinline__ void attn_merge_phase(const MegaArgs& a, float* sm) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* sc_s = sm;                 // [kMaxSplit]
  float* l_s = sc_s + kMaxSplit;    // [kMaxSplit]
  float* linv = l_s + kMaxSplit;    // [1] (padded to 4)
  float* pacc = linv + 4;           // [kThreads / HD][HD] = kThreads partial sums
  const int ns = a.nsplit, units = a.M * a.nh;
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int m = u / a.nh, h = u % a.nh;
    const float* bo = a.part_o + ((int64_t)m * a.nh + h) * ns * HD;
    const float* bml = a.part_ml + ((int64_t)m * a.nh + h) * ns * 2;
    if (tid < ns) {
      sc_s[tid] = __ldcg(bml + tid * 2);
      l_s[tid] = __ldcg(bml + tid * 2 + 1);
    }
    cta_sync();
    if (warp == 0) {
      float Mx = -INFINITY;
      for (int sp = lane; sp < ns; sp += 32) Mx = fmaxf(Mx, sc_s[sp]);
      Mx = warp_max(Mx);
      float Lsum = 0.f;
      for (int sp = lane; sp < ns; sp += 32) {
        const float cc = Mx == -INFINITY ? 0.f : exp2f(sc_s[sp] - Mx);
        sc_s[sp] = cc;
        Lsum += l_s[sp] * cc;
      }
      Lsum = warp_sum(Lsum);
      if (lane == 0) linv[0] = Lsum > 0.f ? 1.f / Lsum : 0.f;
    }
    cta_sync();
    // kThreads / HD thread groups share the sum over the splits (independent loads, a few per thread)
    constexpr int NP = kThreads / HD;
    const int d = tid % HD, pt = tid / HD;
    float acc = 0.f;
#pragma unroll 4
    for (int sp = pt; sp < ns; sp += NP) acc = fmaf(__ldcg(bo + (int64_t)sp * HD + d), sc_s[sp], acc);
    pacc[pt * HD + d] = acc;
    cta_sync();
    if (tid < HD) {
      float tot = 0.f;
#pragma unroll
      for (int q = 0; q < NP; ++q) tot += pacc[q * HD + tid];
      const float gate = ldcg_bf16(a.proj + (int64_t)m * a.ld_proj + (int64_t)h * 2 * HD + HD + tid);
      // rounded to bf16 by the output projection's prologue, as the multi-kernel path rounds it
      a.mix[(int64_t)m * a.nh * HD + h * HD + tid] = tot * linv[0] * sigmoid_f(gate);
    }
    cta_sync();
  }
}

// ------------------------------------------------------------------------------------------------
// The step.
template <int DK, int HD, int REP>
__global__ void __launch_bounds__(kLaunchThreads, 1) decode_mega_kernel(const MegaArgs a) {
  // shared memory: [activation rows | mixer scratch] [partial sums] [accumulator tiles] [reductions]
  //                [layer table] [ring barriers] [weight ring]
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);
  float* part = reinterpret_cast<float*>(smem_raw + (((size_t)a.xs_elems * 2 + 255) & ~(size_t)255));
  float* tile_s = part + a.part_floats;                       // [kWarps][16][kTileLd]
  float* red = tile_s + kWarps * 16 * kTileLd;                // [kWarps * 16] reductions / arg-max staging
  MegaLayer* layers_s = reinterpret_cast<MegaLayer*>(red + kWarps * 16);
  uint64_t* ring_bars = reinterpret_cast<uint64_t*>(layers_s + a.n_layers);          // full[16][kMaxStages]
  unsigned char* ring_base = reinterpret_cast<unsigned char*>(
      ((uintptr_t)(ring_bars + kWarps * kMaxStages) + 127) & ~(uintptr_t)127);
  float* phase_sm = reinterpret_cast<float*>(smem_raw);       // mixer phases reuse the activation area
  const int tid = threadIdx.x, M = a.M, H = a.H;
  // the per-layer table is read by every phase: one copy into shared memory instead of cold global reads
  {
    const int words = a.n_layers * (int)(sizeof(MegaLayer) / 4);
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a.layers);
    uint32_t* dst = reinterpret_cast<uint32_t*>(layers_s);
    for (int i = tid; i < words; i += kThreads) dst[i] = __ldg(src + i);
  }
  Ring ring;
  ring.base = ring_base;
  ring.full = ring_bars;
  ring.stages = a.ring_stages;
  ring.bc = ring.issued = 0;
  ring.ph = 0;
  ring.active = false;
  if (tid == 0 && ring.stages > 0) {
    for (int i = 0; i < kWarps * kMaxStages; ++i) sm100::mbar_init(ring.full + i, 1);
    sm100::mbar_fence_init();
  }
  cta_sync();                                                 // table and barriers are ready
  if (ring.stages > 0) {
    // fill the warp's stages with its first batches of the step
    ring.active = true;
    ring.p = proj_of(a, layers_s, 0);
    ring.it.init(ring.p, M, tid >> 5);
    ring_settle(a, layers_s, ring, tid >> 5);
    for (int i = 0; i < ring.stages; ++i) ring_issue(a, layers_s, ring, tid >> 5, tid & 31);
  }
  Ctx c;
  c.bar_target = __ldcg(a.bar + 1);
  c.n_bar = 0;
  c.n_stamp = 0;
  c.epoch = a.tp_on ? __ldcg(a.tp.epoch) + 1u : 0u;
  auto make_proj = [&](const bf16* W, int rows_total, int K, int n_out, int mode, void* out, int ldo, int site) {
    return ::make_proj(a, W, rows_total, K, n_out, mode, out, ldo, site);
  };
  bf16* res_cur = a.res0;
  bf16* res_nxt = a.res1;
  bool have_h = false;
  stamp(a, c);
  for (int li = 0; li < a.n_layers; ++li) {
    const MegaLayer& L = layers_s[li];
    const bool lin = L.kind == 0;
    const int mixw = lin ? a.nv * a.dv : a.nh * HD;
    // ---- A: input projection -------------------------------------------------------------------
    const Proj pin = make_proj(L.w_in, L.n_in, H, L.n_in, 0, a.proj, a.ld_proj, -1);
    const Proj pout = make_proj(L.w_out, H, mixw, H, 1, a.h, H, 2 * li);
    const Proj pgu = make_proj(L.w_gu, 2 * a.I, H, a.I, 2, a.inter, a.I, -1);
    const Proj pdown = make_proj(L.w_down, H, a.I, H, 1, a.h, H, 2 * li + 1);
    if (li == 0 && !a.use_res0) prologue_norm(a, nullptr, a.tokens_in, nullptr, L.in_gain, res_nxt, H, xs, red);
    else prologue_norm(a, res_cur, nullptr, have_h ? a.h : nullptr, L.in_gain, res_nxt, H, xs, red);
    stamp(a, c);
    { bf16* t = res_cur; res_cur = res_nxt; res_nxt = t; }
    proj_run(a, c, pin, xs, part, tile_s, red, ring, layers_s);
    stamp(a, c);
    if (a.prefetch && tid == 0) proj_prefetch(pout, a.prefetch);
    grid_barrier(a, c);
    stamp(a, c);
    // ---- B: mixer ---------------------------------------------------------------------------------
    if (lin) {
      gdn_phase<DK>(a, L, phase_sm);
    } else {
      attn_phase<HD, REP>(a, L, phase_sm);
      grid_barrier(a, c);
      attn_merge_phase<HD>(a, phase_sm);
    }
    stamp(a, c);
    if (a.prefetch && tid == 0) proj_prefetch(pgu, a.prefetch);
    grid_barrier(a, c);
    stamp(a, c);
    // ---- C: output projection (+ all-reduce) ---------------------------------------------------------
    if (lin) prologue_gdn_act(a, L, xs);
    else prologue_copy_f32(a, a.mix, mixw, xs);
    stamp(a, c);
    proj_run(a, c, pout, xs, part, tile_s, red, ring, layers_s);
    stamp(a, c);
    grid_barrier(a, c);
    stamp(a, c);
    // ---- D: gate | up with SwiGLU ----------------------------------------------------------------
    prologue_norm(a, res_cur, nullptr, a.h, L.post_gain, res_nxt, H, xs, red);
    stamp(a, c);
    { bf16* t = res_cur; res_cur = res_nxt; res_nxt = t; }
    proj_run(a, c, pgu, xs, part, tile_s, red, ring, layers_s);
    stamp(a, c);
    if (a.prefetch && tid == 0) proj_prefetch(pdown, a.prefetch);
    grid_barrier(a, c);
    stamp(a, c);
    // ---- E: down projection (+ all-reduce) ---------------------------------------------------------
    prologue_copy_bf16(a, a.inter, a.I, a.I, xs);
    stamp(a, c);
    proj_run(a, c, pdown, xs, part, tile_s, red, ring, layers_s);
    stamp(a, c);
    if (a.prefetch && tid == 0) {
      if (li + 1 < a.n_layers) {
        const MegaLayer& Ln = layers_s[li + 1];
        proj_prefetch(make_proj(Ln.w_in, Ln.n_in, H, Ln.n_in, 0, nullptr, 0, -1), a.prefetch);
      } else {
        proj_prefetch(make_proj(a.lm_head, a.vocab_local, H, a.vocab_local, 3, nullptr, 0, -1), a.prefetch);
      }
    }
    grid_barrier(a, c);
    stamp(a, c);
    have_h = true;
  }
  // ---- lm_head + arg-max -----------------------------------------------------------------------------
  const Proj phead = make_proj(a.lm_head, a.vocab_local, H, a.vocab_local, 3, a.logits, a.ld_logits, -1);
  prologue_norm(a, res_cur, nullptr, have_h ? a.h : nullptr, a.final_gain, res_nxt, H, xs, red);
  stamp(a, c);
  proj_run(a, c, phead, xs, part, tile_s, red, ring, layers_s);
  stamp(a, c);
  grid_barrier(a, c);
  stamp(a, c);
  if (blockIdx.x == 0) {
    // reduce the CTAs' candidates (ties to the lowest index); one warp per batch row
    const int lane = tid & 31, warp = tid >> 5;
    if (warp < M) {
      float v = -INFINITY;
      int ix = 0x7fffffff;
      for (int b = lane; b < (int)gridDim.x; b += 32) {
        const float ov = __ldcg(a.cand + ((int64_t)b * M + warp) * 2);
        const int oi = __float_as_int(__ldcg(a.cand + ((int64_t)b * M + warp) * 2 + 1));
        if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, off);
        const int oi = __shfl_xor_sync(0xffffffffu, ix, off);
        if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
      }
      if (a.tp_on && lane == 0) {
        // vocabulary-parallel arg-max: every rank sends {value, global index} to every rank and keeps the
        // best of all ranks (ties to the lowest index, so all ranks agree)
        const int site = 2 * a.n_layers;
        ix = ix == 0x7fffffff ? ix : ix + a.vocab_off;
        const int64_t base = ((int64_t)site * a.tp.world + a.tp.rank) * a.tp.slot_floats + warp * 2;
        for (int q = 0; q < a.tp.world; ++q) {
          tp_st_pair(a.tp.inbox[q], base, v, c.epoch);
          tp_st_pair(a.tp.inbox[q], base + 1, __int_as_float(ix), c.epoch);
        }
        v = -INFINITY;
        ix = 0x7fffffff;
        for (int r2 = 0; r2 < a.tp.world; ++r2) {
          const int64_t e2 = ((int64_t)site * a.tp.world + r2) * a.tp.slot_floats + warp * 2;
          unsigned long long pv[2];
          for (int w2 = 0; w2 < 2; ++w2) {
            pv[w2] = tp_ld_pair(a.tp.my_inbox, e2 + w2);
            if ((unsigned)(pv[w2] >> 32) != c.epoch && !tp_status_set(a.status)) {
              const unsigned long long t0 = tp_now_ns(), limit = a.tp.wait_ns ? a.tp.wait_ns : kTpWaitNs;
              unsigned spins = 0;
              while ((unsigned)(pv[w2] >> 32) != c.epoch) {
                if ((++spins & 63u) == 0) {
                  if (tp_status_set(a.status)) break;
                  if (tp_now_ns() - t0 > limit) { atomicCAS(a.status, 0, 16 + r2); break; }
                }
                pv[w2] = tp_ld_pair(a.tp.my_inbox, e2 + w2);
              }
            }
          }
          const float ov = __uint_as_float((unsigned)pv[0]);
          const int oi = (int)(unsigned)pv[1];
          if (ov > v || (ov == v && oi < ix)) { v = ov; ix = oi; }
        }
      }
      if (lane == 0) {
        const int64_t tok = ix == 0x7fffffff ? 0 : ix;
        a.next[warp] = tok;
        if (a.advance) {
          a.tokens[warp] = tok;
          if (a.positions[warp] >= 0) { a.positions[warp] += 1; a.rope_pos[warp] += 1; }
        }
      }
    }
    if (tid == 0) {
      // the counter has advanced by n_bar * grid: the next launch starts from there
      a.bar[1] = c.bar_target;
      if (a.tp_on) *const_cast<unsigned*>(a.tp.epoch) = c.epoch;
    }
  }
}

typedef void (*MegaFn)(const MegaArgs);
struct MegaVariant { int dk, hd, rep; MegaFn fn; };
const MegaVariant kVariants[] = {
    {128, 256, 2, decode_mega_kernel<128, 256, 2>}, {128, 256, 3, decode_mega_kernel<128, 256, 3>},
    {128, 256, 4, decode_mega_kernel<128, 256, 4>}, {128, 256, 6, decode_mega_kernel<128, 256, 6>},
    {64, 64, 2, decode_mega_kernel<64, 64, 2>},
};
MegaFn find_variant(int dk, int hd, int rep) {
  for (const MegaVariant& v : kVariants)
    if (v.dk == dk && v.hd == hd && v.rep == rep) return v.fn;
  return nullptr;
}
}  // namespace

CB_EXPORT int cb_decode_mega_args_size() { return (int)sizeof(MegaArgs); }
CB_EXPORT int cb_decode_mega_layer_size() { return (int)sizeof(MegaLayer); }
CB_EXPORT int cb_decode_mega_supported(int64_t dk, int64_t hd, int64_t rep) {
  return find_variant((int)dk, (int)hd, (int)rep) ? 1 : 0;
}
// Shared memory beyond the activation and partial-sum areas (accumulator tiles + reduction staging).
CB_EXPORT int cb_decode_mega_fixed_smem(int64_t n_layers, int64_t ring_stages) {
  return (int)((kWarps * 16 * kTileLd + kWarps * 16) * sizeof(float)) + 256 + (int)(n_layers * sizeof(MegaLayer)) +
         kWarps * kMaxStages * 8 + 128 + (int)(kWarps * ring_stages * kStageBytes);
}

// Grid size of a cooperative launch with `smem` bytes of dynamic shared memory: one CTA per SM, or 0
// when not even one CTA fits.
CB_EXPORT int cb_decode_mega_grid(int64_t dk, int64_t hd, int64_t rep, int64_t smem) {
  MegaFn fn = find_variant((int)dk, (int)hd, (int)rep);
  if (!fn) return 0;
  if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  int dev = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kLaunchThreads, (size_t)smem) != cudaSuccess || per_sm < 1) {
    cudaGetLastError();
    return 0;
  }
  return sms;
}

// One decode step.  `args` is a host copy of MegaArgs (layers, buffers and the barrier words live in
// device memory).  Launched cooperatively: either every CTA is resident or the launch fails.
CB_EXPORT int cb_decode_mega(const void* args, int64_t dk, int64_t hd, int64_t rep, int64_t grid, int64_t smem,
                             void* stream) {
  if (!args || grid < 1) return CB_ERR_ARG;
  MegaFn fn = find_variant((int)dk, (int)hd, (int)rep);
  if (!fn) return CB_ERR_SHAPE;
  MegaArgs a;
  memcpy(&a, args, sizeof(a));
  if (a.M != 1 && a.M != 2 && a.M != 4 && a.M != 8) return CB_ERR_SHAPE;
  if (a.nsplit < 1 || a.nsplit > kMaxSplit || a.dv % 32 || a.dv > 256) return CB_ERR_SHAPE;
  if (a.n_layers > kMaxLayers || a.ring_stages < 0 || a.ring_stages > kMaxStages || a.ring_stages == 1) return CB_ERR_SHAPE;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kLaunchThreads);
  cfg.dynamicSmemBytes = (size_t)smem;
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (g_cb_trace_names) cb_trace_name((const void*)fn);
  return (int)cudaLaunchKernelEx(&cfg, fn, a);
}
