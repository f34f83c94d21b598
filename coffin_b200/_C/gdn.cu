// Gated DeltaNet (linear attention) kernels.
//
// Decode: ONE launch per layer does causal conv1d + SiLU, head prep (L2 norm, beta, log decay),
// the gated delta-rule update of the fp32 recurrent state, and the gated RMSNorm of the output.
// The reference runs these as 4-5 launches with fp32 scratch between them
// (models/qwen35/linear_attn.py:358-396; kernels backends/corex/kernels/linear_attn.cu:172-744,
// delta.cu:86-194).  Prefill: the chunked (UT-transform) form of ops/delta.py:57-178 as two
// kernels: the per-chunk triangular system, which also computes conv + SiLU, the q/k norms, beta and
// the log decay from the raw projection rows, and the sequential inter-chunk scan (bf16 operands on
// mma.m16n8k16, fp32 state in registers, a three-stage ring of whole-chunk operand sets); the
// earlier forms (a prep kernel of its own, TF32 products, SIMT) stay selectable for A/B runs.
//
// Conv memory is a ring of the last 16 raw projection rows per sequence slot, indexed by
// position & 15: a step writes only slot pos&15 and reads the three before it, so the CTAs of
// value heads that share a key head never race, and a speculative verify of up to 12 tokens
// can be rolled back without restoring the window.
#include "common.cuh"

namespace {

constexpr int kRing = 16;
constexpr int kChunk = 64;

struct GdnDecodeArgs {
  const bf16* proj;       // [M*ntok, ldp]: q | k | v | z | b | a
  int64_t ldp;
  const float* conv_w;    // [conv_dim, 4], oldest tap first
  const float* A_log;     // [nv]
  const float* dt_bias;   // [nv]
  const float* norm_w;    // [dv]
  bf16* ring;             // [slots, 16, conv_dim]
  float* state;           // [slots, nv, dk, dv]
  const int* slots;       // [M] state slot per row, < 0 = padded row
  const int* positions;   // [M] position of the row's first token
  bf16* out;              // [M*ntok, ldo]
  int64_t ldo;
  float* record;          // optional [M, rec_w, nv, dk+dv+1]
  int rec_w;
  int ntok;               // tokens per row (1 = decode, c = verify chain)
  int write_state;        // 0: leave the state untouched (verify; commit replays the record)
  int gate_sigmoid;       // output gate: 0 = silu(z) (Qwen3.5), 1 = sigmoid(z) (Qwen4-exp option)
  int nk, nv, rep;
  float eps;
};

// MINB = 2: the same kernel compiled for two resident CTAs per SM, used when a batch of rows
// launches many more CTAs than there are SMs.
template <int DK, int DV, int MINB = 1>
__global__ void __launch_bounds__(4 * DV, MINB) gdn_decode_kernel(const GdnDecodeArgs a) {
  constexpr int G = 4, RPT = DK / G, NT = 4 * DV;
  __shared__ float q_s[DK], k_s[DK], v_s[DV];
  __shared__ float sk[G][DV], sq[G][DV];
  __shared__ float scal[4];
  __shared__ float red[32];
  const int h = blockIdx.x, m = blockIdx.y, kh = h / a.rep;
  const int tid = threadIdx.x, j = tid % DV, grp = tid / DV;
  const int kdim = a.nk * DK, conv_dim = 2 * kdim + a.nv * DV;
  const int slot = a.slots[m];
  if (slot < 0) return;
  const int pos0 = a.positions[m];

  // The recurrent state was written by this layer's previous step, long complete: fetch it
  // before waiting for the projection kernel.
  float* sp = a.state + (((int64_t)slot * a.nv + h) * DK + grp * RPT) * DV + j;
  float s[RPT];
  griddep_launch();
#pragma unroll
  for (int r = 0; r < RPT; ++r) s[r] = sp[(int64_t)r * DV];
  griddep_wait();

  const float nexpA = -__expf(a.A_log[h]), dtb = a.dt_bias[h];
  const float nw = a.norm_w[j];
  bf16* ring = a.ring + (int64_t)slot * kRing * conv_dim;

  for (int t = 0; t < a.ntok; ++t) {
    const int pos = pos0 + t;
    const bf16* prow = a.proj + ((int64_t)m * a.ntok + t) * a.ldp;
    // ---- causal conv + SiLU on this head's q, k, v channels ---------------------------
    if (tid < 2 * DK + DV) {
      int c;
      bool own;
      if (tid < DK) { c = kh * DK + tid; own = (h % a.rep) == 0; }
      else if (tid < 2 * DK) { c = kdim + kh * DK + (tid - DK); own = (h % a.rep) == 0; }
      else { c = 2 * kdim + h * DV + (tid - 2 * DK); own = true; }
      const float4 w = *reinterpret_cast<const float4*>(a.conv_w + (int64_t)c * 4);
      const bf16 xn = prow[c];
      // tokens of this launch older than t come from the projection rows, the rest from the ring
      float x3 = 0.f, x2 = 0.f, x1 = 0.f;
      if (t >= 1) x1 = __bfloat162float(prow[c - a.ldp]);
      else if (pos >= 1) x1 = __bfloat162float(ring[(int64_t)((pos - 1) & (kRing - 1)) * conv_dim + c]);
      if (t >= 2) x2 = __bfloat162float(prow[c - 2 * a.ldp]);
      else if (pos >= 2) x2 = __bfloat162float(ring[(int64_t)((pos - 2) & (kRing - 1)) * conv_dim + c]);
      if (t >= 3) x3 = __bfloat162float(prow[c - 3 * a.ldp]);
      else if (pos >= 3) x3 = __bfloat162float(ring[(int64_t)((pos - 3) & (kRing - 1)) * conv_dim + c]);
      const float v = silu_f(w.x * x3 + w.y * x2 + w.z * x1 + w.w * __bfloat162float(xn));
      if (own) ring[(int64_t)(pos & (kRing - 1)) * conv_dim + c] = xn;
      if (tid < DK) q_s[tid] = v;
      else if (tid < 2 * DK) k_s[tid - DK] = v;
      else v_s[tid - 2 * DK] = v;
    }
    __syncthreads();
    // ---- head prep: sum q^2, sum k^2, k.q ------------------------------------------------
    if (tid < 96) {
      const int w = tid >> 5, lane = tid & 31;
      float acc = 0.f;
      for (int i = lane; i < DK; i += 32) {
        const float qa = q_s[i], ka = k_s[i];
        acc += (w == 0) ? qa * qa : (w == 1) ? ka * ka : qa * ka;
      }
      acc = warp_sum(acc);
      if (lane == 0) scal[w] = acc;
    }
    __syncthreads();
    const float rq = rsqrtf(scal[0] + 1e-6f) * rsqrtf((float)DK), rk = rsqrtf(scal[1] + 1e-6f);
    const float kq = scal[2] * rq * rk;
    const float bl = __bfloat162float(prow[conv_dim + a.nv * DV + h]);
    const float al = __bfloat162float(prow[conv_dim + a.nv * DV + a.nv + h]);
    const float beta = sigmoid_f(bl);
    const float alpha = __expf(nexpA * softplus_f(al + dtb));
    // ---- S^T k and S^T q over this thread's rows -----------------------------------------
    float pk = 0.f, pq = 0.f;
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      pk = fmaf(s[r], k_s[grp * RPT + r], pk);
      pq = fmaf(s[r], q_s[grp * RPT + r], pq);
    }
    sk[grp][j] = pk;
    sq[grp][j] = pq;
    __syncthreads();
    const float Sk = (sk[0][j] + sk[1][j] + sk[2][j] + sk[3][j]) * rk;
    const float Sq = (sq[0][j] + sq[1][j] + sq[2][j] + sq[3][j]) * rq;
    const float d = (v_s[j] - alpha * Sk) * beta;
    const float o = alpha * Sq + kq * d;
#pragma unroll
    for (int r = 0; r < RPT; ++r) s[r] = fmaf(k_s[grp * RPT + r] * rk, d, alpha * s[r]);
    if (a.record) {
      float* rec = a.record + (((int64_t)m * a.rec_w + t) * a.nv + h) * (DK + DV + 1);
      if (tid < DK) rec[tid] = k_s[tid] * rk;
      if (grp == 0) rec[DK + j] = d;
      if (tid == 0) rec[DK + DV] = alpha;
    }
    // ---- gated RMSNorm over the head ---------------------------------------------------
    const float ms = block_sum(grp == 0 ? o * o : 0.f, red) / (float)DV;
    if (grp == 0) {
      const float z = __bfloat162float(prow[conv_dim + h * DV + j]);
      a.out[((int64_t)m * a.ntok + t) * a.ldo + h * DV + j] =
          __float2bfloat16(o * rsqrtf(ms + a.eps) * nw * (a.gate_sigmoid ? sigmoid_f(z) : silu_f(z)));
    }
    __syncthreads();
  }
  if (a.write_state) {
#pragma unroll
    for (int r = 0; r < RPT; ++r) sp[(int64_t)r * DV] = s[r];
  }
  (void)NT;
}

// state[slot] = replay of the first steps[m] recorded updates on state[slot] (verify leaves the
// state untouched, so the base is the state itself).
template <int DK, int DV>
__global__ void __launch_bounds__(4 * DV) gdn_commit_kernel(float* state, const float* record,
                                                            const int* slots, const int* steps,
                                                            int rec_w, int nv) {
  constexpr int G = 4, RPT = DK / G;
  const int h = blockIdx.x, m = blockIdx.y, j = threadIdx.x % DV, grp = threadIdx.x / DV;
  griddep_launch();
  griddep_wait();
  const int slot = slots[m], n = steps[m];
  if (slot < 0 || n <= 0) return;
  float* sp = state + (((int64_t)slot * nv + h) * DK + grp * RPT) * DV + j;
  float s[RPT];
#pragma unroll
  for (int r = 0; r < RPT; ++r) s[r] = sp[(int64_t)r * DV];
  for (int t = 0; t < n && t < rec_w; ++t) {
    const float* rec = record + (((int64_t)m * rec_w + t) * nv + h) * (DK + DV + 1);
    const float alpha = rec[DK + DV], d = rec[DK + j];
#pragma unroll
    for (int r = 0; r < RPT; ++r) s[r] = fmaf(rec[grp * RPT + r], d, alpha * s[r]);
  }
#pragma unroll
  for (int r = 0; r < RPT; ++r) sp[(int64_t)r * DV] = s[r];
}

// ---------------------------------------------------------------------------------------
// Prefill prep: conv + SiLU, q/k normalisation, beta and g for a chunk of tokens.
constexpr int kPrepTok = 4;   // tokens per CTA of the prefill prep kernel (512 CTAs for a 2048-token chunk)
struct GdnPrepArgs {
  const bf16* proj; int64_t ldp;
  const float* conv_w; const float* A_log; const float* dt_bias;
  const bf16* ring;        // this sequence's ring [16, conv_dim]
  float* qn; float* kn;    // [nk, Tp, DK]
  float* v;                // [nv, Tp, DV]
  float* beta; float* g;   // [nv, Tp]
  int T, Tp, pos0, nk, nv;
};

template <int DK, int DV>
__global__ void __launch_bounds__(256) gdn_prep_kernel(const GdnPrepArgs a) {
  // One CTA per tile of kPrepTok tokens, one warp per head task.  A lane owns four adjacent channels
  // (8-byte loads of the projection rows, 16-byte stores) and slides the 4-tap window over the tile's
  // tokens in registers, so a row is read once per tile instead of once per tap.
  griddep_launch();
  griddep_wait();
  constexpr int TT = kPrepTok;
  const int t0 = blockIdx.x * TT, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kdim = a.nk * DK, conv_dim = 2 * kdim + a.nv * DV;
  const int ntask = 2 * a.nk + a.nv + 1;
  for (int task = warp; task < ntask; task += 8) {
    if (task == ntask - 1) {  // beta / g for every (value head, token of the tile)
      for (int idx = lane; idx < a.nv * TT; idx += 32) {
        const int h = idx / TT, t = t0 + idx % TT;
        float b = 0.f, gg = 0.f;
        if (t < a.T) {
          const bf16* prow = a.proj + (int64_t)t * a.ldp + conv_dim + a.nv * DV;
          b = sigmoid_f(__bfloat162float(prow[h]));
          gg = -__expf(a.A_log[h]) * softplus_f(__bfloat162float(prow[a.nv + h]) + a.dt_bias[h]);
        }
        if (t < a.Tp) {
          a.beta[(int64_t)h * a.Tp + t] = b;
          a.g[(int64_t)h * a.Tp + t] = gg;
        }
      }
      continue;
    }
    int cbase, width, head, kind;  // kind 0 = q, 1 = k, 2 = v
    if (task < a.nk) { kind = 0; head = task; cbase = head * DK; width = DK; }
    else if (task < 2 * a.nk) { kind = 1; head = task - a.nk; cbase = kdim + head * DK; width = DK; }
    else { kind = 2; head = task - 2 * a.nk; cbase = 2 * kdim + head * DV; width = DV; }
    const int i0 = lane * 4;
    const bool act = i0 < width;
    const int c = cbase + i0;
    float w[4][4];                       // [channel][tap]
    float win[3][4];                     // the three rows before the current token
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 wj = act ? *reinterpret_cast<const float4*>(a.conv_w + (int64_t)(c + j) * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
      w[j][0] = wj.x; w[j][1] = wj.y; w[j][2] = wj.z; w[j][3] = wj.w;
    }
    // all TT + 3 rows of the tile are requested before anything is computed or stored (the stores below
    // may alias the loads as far as the compiler knows, so it would not hoist them itself): eleven
    // independent 8-byte loads in flight per lane instead of one
    uint2 raw[TT + 3];
#pragma unroll
    for (int r = 0; r < TT + 3; ++r) {
      const int tt = t0 - 3 + r, pp = a.pos0 + tt;
      raw[r] = make_uint2(0u, 0u);
      if (act) {
        if (tt >= 0) { if (tt < a.T) raw[r] = *reinterpret_cast<const uint2*>(a.proj + (int64_t)tt * a.ldp + c); }
        else if (pp >= 0) raw[r] = *reinterpret_cast<const uint2*>(a.ring + (int64_t)(pp & (kRing - 1)) * conv_dim + c);
      }
    }
    auto load_row = [&](int r, float* x) {          // conv input row r of the tile window (row 0 = token t0 - 3)
      // a bf16 is the upper half of the fp32 with the same value
      x[0] = __uint_as_float(raw[r].x << 16); x[1] = __uint_as_float(raw[r].x & 0xffff0000u);
      x[2] = __uint_as_float(raw[r].y << 16); x[3] = __uint_as_float(raw[r].y & 0xffff0000u);
    };
    load_row(0, win[0]);
    load_row(1, win[1]);
    load_row(2, win[2]);
    float* dbase = (kind == 0 ? a.qn : kind == 1 ? a.kn : a.v) + (int64_t)head * a.Tp * width;
#pragma unroll
    for (int k = 0; k < TT; ++k) {
      const int t = t0 + k;
      float cur[4], val[4];
      load_row(k + 3, cur);
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        val[j] = (act && t < a.T) ? silu_f(w[j][0] * win[0][j] + w[j][1] * win[1][j] + w[j][2] * win[2][j] + w[j][3] * cur[j]) : 0.f;
        ss += val[j] * val[j];
        win[0][j] = win[1][j]; win[1][j] = win[2][j]; win[2][j] = cur[j];
      }
      float scale = 1.f;
      if (kind < 2) {
        ss = warp_sum(ss);
        scale = rsqrtf(ss + 1e-6f) * (kind == 0 ? rsqrtf((float)DK) : 1.f);
      }
      if (act && t < a.Tp)
        *reinterpret_cast<float4*>(dbase + (int64_t)t * width + i0) = make_float4(val[0] * scale, val[1] * scale, val[2] * scale, val[3] * scale);
    }
  }
}

// ring[(pos0 + t) & 15] = proj[t] for the last min(T, 16) tokens of the chunk
__global__ void gdn_ring_update_kernel(const bf16* proj, int64_t ldp, bf16* ring, int T, int pos0, int conv_dim) {
  griddep_launch();
  griddep_wait();
  const int first = max(0, T - kRing);
  const int t = first + blockIdx.x;
  if (t >= T) return;
  const uint4* src = reinterpret_cast<const uint4*>(proj + (int64_t)t * ldp);
  uint4* dst = reinterpret_cast<uint4*>(ring + (int64_t)((pos0 + t) & (kRing - 1)) * conv_dim);
  for (int c = threadIdx.x; c < (conv_dim >> 3); c += blockDim.x) dst[c] = src[c];
}

// ---------------------------------------------------------------------------------------
// Per-chunk triangular system. For chunk rows i (64) with cumulative log decay c_i:
//   Tm_ij = beta_i e^{c_i-c_j} k_i.k_j (j<i);  W = (I+Tm)^-1
//   nvv = W (beta V)  [64, DV];  kcd = W (beta e^c K) [64, DK];  ica_ij = q_i.k_j e^{c_i-c_j} (j<=i)
// and the scaled copies the scan needs: qe = q e^c, ke = k e^{c_L - c}, ecl = e^{c_L}.
struct GdnChunkArgs {
  const float* qn; const float* kn; const float* v; const float* beta; const float* g;
  float* nvv;   // [nv, nc, 64, DV]
  float* kcd;   // [nv, nc, 64, DK]
  float* ica;   // [nv, nc, 64, 64]
  float* qe;    // [nv, nc, 64, DK]
  float* ke;    // [nv, nc, 64, DK]
  float* ecl;   // [nv, nc]
  int Tp, nc, rep;
  // fused form (the prepare kernel takes conv + SiLU, the q/k normalisation, beta and g from the raw
  // projection rows itself; qn / kn / v / beta / g above are then unused)
  const bf16* proj; int64_t ldp; const float* conv_w; const float* A_log; const float* dt_bias; const bf16* ring;
  int T, pos0, nk, nv;
};

template <int DK, int DV>
__global__ void __launch_bounds__(256) gdn_chunk_prepare_kernel(const GdnChunkArgs a) {
  constexpr int L = kChunk, LDK = DK + 4, LDV = DV + 4, LDL = L + 1;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* Ks = reinterpret_cast<float*>(smem_raw);   // [L][LDK]
  float* Qs = Ks + L * LDK;                         // [L][LDK]  (later: beta e^c K)
  float* Vs = Qs + L * LDK;                         // [L][LDV]  (beta V)
  float* Tm = Vs + L * LDV;                         // [L][LDL]
  float* Wi = Tm + L * LDL;                         // [L][LDL]
  float* cs = Wi + L * LDL;                         // [L] cumulative log decay
  float* bs = cs + L;                               // [L] beta
  griddep_launch();
  griddep_wait();
  const int n = blockIdx.x, h = blockIdx.y, kh = h / a.rep, tid = threadIdx.x;
  const int64_t t0 = (int64_t)n * L;
  const float* kp = a.kn + ((int64_t)kh * a.Tp + t0) * DK;
  const float* qp = a.qn + ((int64_t)kh * a.Tp + t0) * DK;
  const float* vp = a.v + ((int64_t)h * a.Tp + t0) * DV;
  for (int idx = tid; idx < L * DK / 4; idx += 256) {
    const int i = idx / (DK / 4), c = (idx % (DK / 4)) * 4;
    *reinterpret_cast<float4*>(Ks + i * LDK + c) = *reinterpret_cast<const float4*>(kp + (int64_t)i * DK + c);
    *reinterpret_cast<float4*>(Qs + i * LDK + c) = *reinterpret_cast<const float4*>(qp + (int64_t)i * DK + c);
  }
  for (int idx = tid; idx < L * DV / 4; idx += 256) {
    const int i = idx / (DV / 4), c = (idx % (DV / 4)) * 4;
    *reinterpret_cast<float4*>(Vs + i * LDV + c) = *reinterpret_cast<const float4*>(vp + (int64_t)i * DV + c);
  }
  if (tid < 32) {  // inclusive scan of g over the 64 rows
    const float g0 = a.g[(int64_t)h * a.Tp + t0 + tid], g1 = a.g[(int64_t)h * a.Tp + t0 + 32 + tid];
    float x0 = g0, x1 = g1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float y0 = __shfl_up_sync(0xffffffffu, x0, o), y1 = __shfl_up_sync(0xffffffffu, x1, o);
      if (tid >= o) { x0 += y0; x1 += y1; }
    }
    const float tot0 = __shfl_sync(0xffffffffu, x0, 31);
    cs[tid] = x0;
    cs[32 + tid] = x1 + tot0;
    bs[tid] = a.beta[(int64_t)h * a.Tp + t0 + tid];
    bs[32 + tid] = a.beta[(int64_t)h * a.Tp + t0 + 32 + tid];
  }
  __syncthreads();
  // ---- K K^T and Q K^T: 4x4 register tiles ---------------------------------------------
  {
    const int ti = tid / 16, tj = tid % 16;
    float kk[4][4] = {}, qk[4][4] = {};
    for (int c = 0; c < DK; c += 4) {
      float4 ki[4], qi[4], kj[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        ki[x] = *reinterpret_cast<const float4*>(Ks + (ti * 4 + x) * LDK + c);
        qi[x] = *reinterpret_cast<const float4*>(Qs + (ti * 4 + x) * LDK + c);
        kj[x] = *reinterpret_cast<const float4*>(Ks + (tj * 4 + x) * LDK + c);
      }
#pragma unroll
      for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < 4; ++y) {
          kk[x][y] += ki[x].x * kj[y].x + ki[x].y * kj[y].y + ki[x].z * kj[y].z + ki[x].w * kj[y].w;
          qk[x][y] += qi[x].x * kj[y].x + qi[x].y * kj[y].y + qi[x].z * kj[y].z + qi[x].w * kj[y].w;
        }
    }
    float* icap = a.ica + ((int64_t)h * a.nc + n) * L * L;
#pragma unroll
    for (int x = 0; x < 4; ++x)
#pragma unroll
      for (int y = 0; y < 4; ++y) {
        const int i = ti * 4 + x, jj = tj * 4 + y;
        const float dec = (jj <= i) ? __expf(cs[i] - cs[jj]) : 0.f;
        Tm[i * LDL + jj] = (jj < i) ? bs[i] * dec * kk[x][y] : 0.f;
        icap[i * L + jj] = dec * qk[x][y];
      }
  }
  __syncthreads();
  // ---- scaled copies for the scan, then overwrite Qs <- beta e^c K, Vs <- beta V -------
  {
    float* qep = a.qe + ((int64_t)h * a.nc + n) * L * DK;
    float* kep = a.ke + ((int64_t)h * a.nc + n) * L * DK;
    const float cl = cs[L - 1];
    for (int idx = tid; idx < L * DK; idx += 256) {
      const int i = idx / DK, c = idx % DK;
      const float ec = __expf(cs[i]);
      const float kv = Ks[i * LDK + c];
      qep[idx] = Qs[i * LDK + c] * ec;
      kep[idx] = kv * __expf(cl - cs[i]);
      Qs[i * LDK + c] = bs[i] * ec * kv;
    }
    for (int idx = tid; idx < L * DV; idx += 256) {
      const int i = idx / DV, c = idx % DV;
      Vs[i * LDV + c] *= bs[i];
    }
    if (tid == 0) a.ecl[(int64_t)h * a.nc + n] = __expf(cl);
  }
  // ---- W = (I + Tm)^-1 by forward substitution, one column per thread ------------------
  if (tid < L) {
    const int c = tid;
    for (int i = 0; i < L; ++i) {
      float acc = (i == c) ? 1.f : 0.f;
      for (int jj = c; jj < i; ++jj) acc -= Tm[i * LDL + jj] * Wi[jj * LDL + c];
      Wi[i * LDL + c] = (i >= c) ? acc : 0.f;
    }
  }
  __syncthreads();
  // ---- nvv = W (beta V), kcd = W (beta e^c K) ---------------------------------------------
  {
    float* nvp = a.nvv + ((int64_t)h * a.nc + n) * L * DV;
    float* kcp = a.kcd + ((int64_t)h * a.nc + n) * L * DK;
    // thread -> 4 rows x 4 cols tiles over [64 x (DV + DK)]
    constexpr int NCOL = (DV + DK) / 4;
    for (int tile = tid; tile < 16 * NCOL; tile += 256) {
      const int ti = tile / NCOL, tc = tile % NCOL;
      const bool isv = tc < DV / 4;
      const float* B = isv ? (Vs + tc * 4) : (Qs + (tc - DV / 4) * 4);
      const int ldb = isv ? LDV : LDK;
      float acc[4][4] = {};
      const int imax = ti * 4 + 3;
      for (int l = 0; l <= imax; ++l) {
        const float4 b = *reinterpret_cast<const float4*>(B + l * ldb);
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const float w = Wi[(ti * 4 + x) * LDL + l];
          acc[x][0] += w * b.x; acc[x][1] += w * b.y; acc[x][2] += w * b.z; acc[x][3] += w * b.w;
        }
      }
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const float4 o = make_float4(acc[x][0], acc[x][1], acc[x][2], acc[x][3]);
        if (isv) *reinterpret_cast<float4*>(nvp + (ti * 4 + x) * DV + tc * 4) = o;
        else *reinterpret_cast<float4*>(kcp + (ti * 4 + x) * DK + (tc - DV / 4) * 4) = o;
      }
    }
  }
}

// Sequential scan over chunks for one (value head, DVS-column slice) of the state.
//   U = nvv - kcd S ;  O = qe S + ica U ;  S <- ecl S + ke^T U
struct GdnScanArgs {
  const float* nvv; const float* kcd; const float* ica; const float* qe; const float* ke; const float* ecl;
  float* state;   // this sequence's state [nv, DK, DV] (read as S0, written as S_final)
  float* out;     // [T, nv*DV] fp32
  int T, nc, nv;
};

template <int DK, int DV, int DVS>
__global__ void __launch_bounds__(256) gdn_chunk_scan_kernel(const GdnScanArgs a) {
  constexpr int L = kChunk, LDK = DK + 4, LDS = DVS + 4, LDL = L + 4;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* S = reinterpret_cast<float*>(smem_raw);  // [DK][LDS]
  float* A1 = S + DK * LDS;                       // [L][LDK] kcd, then ke
  float* A2 = A1 + L * LDK;                       // [L][LDK] qe
  float* Ic = A2 + L * LDK;                       // [L][LDL]
  float* U = Ic + L * LDL;                        // [L][LDS]
  griddep_launch();
  griddep_wait();
  const int h = blockIdx.x, sl = blockIdx.y, tid = threadIdx.x;
  const int col0 = sl * DVS;
  float* sp = a.state + (int64_t)h * DK * DV + col0;
  for (int idx = tid; idx < DK * DVS; idx += 256) S[(idx / DVS) * LDS + idx % DVS] = sp[(int64_t)(idx / DVS) * DV + idx % DVS];
  // thread tiles: (64 x DVS) outputs -> rows ty*RT.., cols tx*4.. ; (DK x DVS) -> rows ty*RS..
  constexpr int TX = DVS / 4, TY = 256 / TX, RT = L / TY, RS = DK / TY;
  static_assert(L % TY == 0 && DK % TY == 0, "tile");
  const int tx = tid % TX, ty = tid / TX;
  for (int n = 0; n < a.nc; ++n) {
    const int64_t base = (int64_t)h * a.nc + n;
    __syncthreads();
    for (int idx = tid; idx < L * DK / 4; idx += 256) {
      const int i = idx / (DK / 4), c = (idx % (DK / 4)) * 4;
      *reinterpret_cast<float4*>(A1 + i * LDK + c) = *reinterpret_cast<const float4*>(a.kcd + base * L * DK + (int64_t)i * DK + c);
      *reinterpret_cast<float4*>(A2 + i * LDK + c) = *reinterpret_cast<const float4*>(a.qe + base * L * DK + (int64_t)i * DK + c);
    }
    for (int idx = tid; idx < L * L / 4; idx += 256) {
      const int i = idx / (L / 4), c = (idx % (L / 4)) * 4;
      *reinterpret_cast<float4*>(Ic + i * LDL + c) = *reinterpret_cast<const float4*>(a.ica + base * L * L + (int64_t)i * L + c);
    }
    __syncthreads();
    // U = nvv - kcd S ; Oacc = qe S
    float u[RT][4], o[RT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
      const float4 nv4 = *reinterpret_cast<const float4*>(a.nvv + base * L * DV + (int64_t)(ty * RT + r) * DV + col0 + tx * 4);
      u[r][0] = nv4.x; u[r][1] = nv4.y; u[r][2] = nv4.z; u[r][3] = nv4.w;
      o[r][0] = o[r][1] = o[r][2] = o[r][3] = 0.f;
    }
    for (int k = 0; k < DK; ++k) {
      const float4 sv = *reinterpret_cast<const float4*>(S + k * LDS + tx * 4);
#pragma unroll
      for (int r = 0; r < RT; ++r) {
        const float ak = A1[(ty * RT + r) * LDK + k], aq = A2[(ty * RT + r) * LDK + k];
        u[r][0] -= ak * sv.x; u[r][1] -= ak * sv.y; u[r][2] -= ak * sv.z; u[r][3] -= ak * sv.w;
        o[r][0] += aq * sv.x; o[r][1] += aq * sv.y; o[r][2] += aq * sv.z; o[r][3] += aq * sv.w;
      }
    }
#pragma unroll
    for (int r = 0; r < RT; ++r)
      *reinterpret_cast<float4*>(U + (ty * RT + r) * LDS + tx * 4) = make_float4(u[r][0], u[r][1], u[r][2], u[r][3]);
    __syncthreads();
    // ke replaces kcd in A1 (kcd no longer needed)
    for (int idx = tid; idx < L * DK / 4; idx += 256) {
      const int i = idx / (DK / 4), c = (idx % (DK / 4)) * 4;
      *reinterpret_cast<float4*>(A1 + i * LDK + c) = *reinterpret_cast<const float4*>(a.ke + base * L * DK + (int64_t)i * DK + c);
    }
    // O += ica U (lower triangular: l <= row)
    for (int l = 0; l < L; ++l) {
      const float4 uv = *reinterpret_cast<const float4*>(U + l * LDS + tx * 4);
#pragma unroll
      for (int r = 0; r < RT; ++r) {
        const float c = Ic[(ty * RT + r) * LDL + l];
        o[r][0] += c * uv.x; o[r][1] += c * uv.y; o[r][2] += c * uv.z; o[r][3] += c * uv.w;
      }
    }
#pragma unroll
    for (int r = 0; r < RT; ++r) {
      const int64_t t = (int64_t)n * L + ty * RT + r;
      if (t < a.T)
        *reinterpret_cast<float4*>(a.out + t * a.nv * DV + (int64_t)h * DV + col0 + tx * 4) =
            make_float4(o[r][0], o[r][1], o[r][2], o[r][3]);
    }
    __syncthreads();
    // S <- ecl S + ke^T U
    const float el = a.ecl[base];
    float sacc[RS][4];
#pragma unroll
    for (int r = 0; r < RS; ++r) {
      const float4 sv = *reinterpret_cast<const float4*>(S + (ty * RS + r) * LDS + tx * 4);
      sacc[r][0] = sv.x * el; sacc[r][1] = sv.y * el; sacc[r][2] = sv.z * el; sacc[r][3] = sv.w * el;
    }
    for (int l = 0; l < L; ++l) {
      const float4 uv = *reinterpret_cast<const float4*>(U + l * LDS + tx * 4);
#pragma unroll
      for (int r = 0; r < RS; ++r) {
        const float kv = A1[l * LDK + ty * RS + r];
        sacc[r][0] += kv * uv.x; sacc[r][1] += kv * uv.y; sacc[r][2] += kv * uv.z; sacc[r][3] += kv * uv.w;
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < RS; ++r)
      *reinterpret_cast<float4*>(S + (ty * RS + r) * LDS + tx * 4) = make_float4(sacc[r][0], sacc[r][1], sacc[r][2], sacc[r][3]);
  }
  __syncthreads();
  for (int idx = tid; idx < DK * DVS; idx += 256) sp[(int64_t)(idx / DVS) * DV + idx % DVS] = S[(idx / DVS) * LDS + idx % DVS];
}

// ---------------------------------------------------------------------------------------------
// Tensor-core versions of the two chunk kernels.  The products are small (64x64x128, 64x128x32)
// but there are eight of them per (chunk, head); as fp32 SIMT loops they made the delta-net layers
// the largest part of a prefill.  Operands stay fp32 in shared memory and go to the tensor cores as
// TF32 (mma.m16n8k8, fp32 accumulate): no conversion pass, and the state itself is never rounded -
// only its copy that enters a product.  Leading dimensions are chosen so that fragment loads are
// bank-conflict free: an operand read "row = g, k = t" wants ld = 4 (mod 32), one read "k = t,
// column = g" wants ld = 8 (mod 32).
__device__ __forceinline__ void mma_tf32(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// A fragment of rows r0+g / r0+g+8, columns k0+t / k0+t+4 of a row-major matrix
__device__ __forceinline__ void frag_a(const float* M, int ld, int r0, int k0, int g, int t, uint32_t* a) {
  const float* p = M + (r0 + g) * ld + k0 + t;
  a[0] = __float_as_uint(p[0]);
  a[1] = __float_as_uint(p[8 * ld]);
  a[2] = __float_as_uint(p[4]);
  a[3] = __float_as_uint(p[8 * ld + 4]);
}
// A fragment of the transpose: element (row, k) = M[k][row]
__device__ __forceinline__ void frag_at(const float* M, int ld, int r0, int k0, int g, int t, uint32_t* a) {
  const float* p = M + (k0 + t) * ld + r0 + g;
  a[0] = __float_as_uint(p[0]);
  a[1] = __float_as_uint(p[8]);
  a[2] = __float_as_uint(p[4 * ld]);
  a[3] = __float_as_uint(p[4 * ld + 8]);
}
// B fragment (k = k0+t / k0+t+4, column c0+g) of a row-major [K][N] matrix
__device__ __forceinline__ void frag_b(const float* M, int ld, int k0, int c0, int g, int t, uint32_t* b) {
  const float* p = M + (k0 + t) * ld + c0 + g;
  b[0] = __float_as_uint(p[0]);
  b[1] = __float_as_uint(p[4 * ld]);
}
// B fragment of the transpose: element (k, column) = M[column][k]
__device__ __forceinline__ void frag_bt(const float* M, int ld, int k0, int c0, int g, int t, uint32_t* b) {
  const float* p = M + (c0 + g) * ld + k0 + t;
  b[0] = __float_as_uint(p[0]);
  b[1] = __float_as_uint(p[4]);
}

template <int DK, int DV>
struct PrepTcLayout {
  static constexpr int L = kChunk, LDA = DK + 4, LDB = DK + 8, LDV = DV + 8, LDL = L + 4;
  // R1 [L][max(LDA, LDV)]: K as a row operand, later V (k-major operand of the last product)
  // R2 [L][LDB]: Q as a row operand (leading dimension LDA), later e^c K as a k-major operand
  // Tm, Wi [L][LDL]; cs, bs [L].  105 KB for 128-wide heads: two CTAs per SM.
  static constexpr int LD1 = LDA > LDV ? LDA : LDV;
  static constexpr size_t floats = (size_t)L * LD1 + (size_t)L * LDB + (size_t)2 * L * LDL + 2 * L;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Causal 4-tap conv + SiLU of NT consecutive tokens (first token t_first of the chunk whose rows are proj,
// earlier rows come from the ring) for the four channels c..c+3 of this lane.  All NT + 3 rows are
// requested before anything is computed.  val[k][j]: token t_first + k, channel c + j; rows past T give 0.
template <int NT>
__device__ __forceinline__ void conv_tokens(const bf16* proj, int64_t ldp, const bf16* ring, int conv_dim, const float* conv_w,
                                            int c, bool act, int t_first, int T, int pos0, float (*val)[4]) {
  float w[4][4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float4 wj = act ? *reinterpret_cast<const float4*>(conv_w + (int64_t)(c + j) * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    w[j][0] = wj.x; w[j][1] = wj.y; w[j][2] = wj.z; w[j][3] = wj.w;
  }
  uint2 raw[NT + 3];
#pragma unroll
  for (int r = 0; r < NT + 3; ++r) {
    const int tt = t_first - 3 + r, pp = pos0 + tt;
    raw[r] = make_uint2(0u, 0u);
    if (act) {
      if (tt >= 0) { if (tt < T) raw[r] = *reinterpret_cast<const uint2*>(proj + (int64_t)tt * ldp + c); }
      else if (pp >= 0) raw[r] = *reinterpret_cast<const uint2*>(ring + (int64_t)(pp & (kRing - 1)) * conv_dim + c);
    }
  }
#pragma unroll
  for (int k = 0; k < NT; ++k) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float x[4];
#pragma unroll
      for (int tap = 0; tap < 4; ++tap) {
        const uint32_t word = (j < 2) ? raw[k + tap].x : raw[k + tap].y;
        x[tap] = (j & 1) ? __uint_as_float(word & 0xffff0000u) : __uint_as_float(word << 16);
      }
      val[k][j] = (act && t_first + k < T) ? silu_f(w[j][0] * x[0] + w[j][1] * x[1] + w[j][2] * x[2] + w[j][3] * x[3]) : 0.f;
    }
  }
}

// FUSE: the q / k / v rows, beta and g are computed here from the raw projection rows (what gdn_prep_kernel
// does as a launch of its own, with an fp32 round trip through memory).
// BF: kcd, qe, ke and ica leave as bf16 (same element offsets in the same regions) for the bf16 scan below;
// the triangular system itself is still solved from TF32 products in fp32.
template <int DK, int DV, bool BF = false, bool FUSE = false>
__global__ void __launch_bounds__(256, 2) gdn_chunk_prepare_tc_kernel(const GdnChunkArgs a) {
  using Lay = PrepTcLayout<DK, DV>;
  constexpr int L = kChunk, LDA = Lay::LDA, LDB = Lay::LDB, LDV = Lay::LDV, LDL = Lay::LDL;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* R1 = reinterpret_cast<float*>(smem_raw);
  float* R2 = R1 + L * Lay::LD1;
  float* Tm = R2 + L * LDB;
  float* Wi = Tm + L * LDL;
  float* cs = Wi + L * LDL;
  float* bs = cs + L;
  float* Ks = R1;          // phase 1-3
  float* Qs = R2;          // phase 1-2
  float* Kb = R2;          // phase 4-5
  float* Vs = R1;          // phase 5
  griddep_launch();
  griddep_wait();
  const int n = blockIdx.x, h = blockIdx.y, kh = h / a.rep, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int64_t t0 = (int64_t)n * L;
  const float* kp = a.kn + ((int64_t)kh * a.Tp + t0) * DK;
  const float* qp = a.qn + ((int64_t)kh * a.Tp + t0) * DK;
  const float* vp = a.v + ((int64_t)h * a.Tp + t0) * DV;
  const int kdim = a.nk * DK, conv_dim = 2 * kdim + a.nv * DV;
  if (FUSE) {
    // warp w: tokens 8w .. 8w+7 of the chunk, a lane owns four adjacent channels of the key head
    const int i0 = lane * 4;
    const bool act = i0 < DK;
    const int tf = (int)t0 + warp * 8;
#pragma unroll
    for (int kind = 0; kind < 2; ++kind) {              // 0: q, 1: k
      float val[8][4];
      conv_tokens<8>(a.proj, a.ldp, a.ring, conv_dim, a.conv_w, kind * kdim + kh * DK + i0, act, tf, a.T, a.pos0, val);
      float* dstm = kind ? Ks : Qs;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float ss = warp_sum(val[k][0] * val[k][0] + val[k][1] * val[k][1] + val[k][2] * val[k][2] + val[k][3] * val[k][3]);
        const float sc = rsqrtf(ss + 1e-6f) * (kind == 0 ? rsqrtf((float)DK) : 1.f);
        if (act) *reinterpret_cast<float4*>(dstm + (warp * 8 + k) * LDA + i0) = make_float4(val[k][0] * sc, val[k][1] * sc, val[k][2] * sc, val[k][3] * sc);
      }
    }
  } else {
    for (int idx = tid; idx < L * DK / 4; idx += 256) {
      const int i = idx / (DK / 4), c = (idx % (DK / 4)) * 4;
      *reinterpret_cast<float4*>(Ks + i * LDA + c) = *reinterpret_cast<const float4*>(kp + (int64_t)i * DK + c);
      *reinterpret_cast<float4*>(Qs + i * LDA + c) = *reinterpret_cast<const float4*>(qp + (int64_t)i * DK + c);
    }
  }
  if (tid < 32) {  // inclusive scan of g over the 64 rows
    float g0, g1, be0, be1;
    if (FUSE) {
      const float al = -__expf(a.A_log[h]), db = a.dt_bias[h];
      const int64_t ta = t0 + tid, tb = ta + 32;
      const bf16* pa = a.proj + ta * a.ldp + conv_dim + a.nv * DV;
      const bf16* pb = a.proj + tb * a.ldp + conv_dim + a.nv * DV;
      g0 = g1 = be0 = be1 = 0.f;
      if (ta < a.T) { be0 = sigmoid_f(__bfloat162float(pa[h])); g0 = al * softplus_f(__bfloat162float(pa[a.nv + h]) + db); }
      if (tb < a.T) { be1 = sigmoid_f(__bfloat162float(pb[h])); g1 = al * softplus_f(__bfloat162float(pb[a.nv + h]) + db); }
    } else {
      g0 = a.g[(int64_t)h * a.Tp + t0 + tid]; g1 = a.g[(int64_t)h * a.Tp + t0 + 32 + tid];
      be0 = a.beta[(int64_t)h * a.Tp + t0 + tid]; be1 = a.beta[(int64_t)h * a.Tp + t0 + 32 + tid];
    }
    float x0 = g0, x1 = g1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float y0 = __shfl_up_sync(0xffffffffu, x0, o), y1 = __shfl_up_sync(0xffffffffu, x1, o);
      if (tid >= o) { x0 += y0; x1 += y1; }
    }
    const float tot0 = __shfl_sync(0xffffffffu, x0, 31);
    cs[tid] = x0;
    cs[32 + tid] = x1 + tot0;
    bs[tid] = be0;
    bs[32 + tid] = be1;
  }
  __syncthreads();
  // ---- K K^T and Q K^T: warp (row tile of 16) x (column half of 32) ----------------------------
  {
    const int r0 = (warp & 3) * 16, c0 = (warp >> 2) * 32;
    float kk[4][4] = {}, qk[4][4] = {};
    for (int k0 = 0; k0 < DK; k0 += 8) {
      uint32_t ak[4], aq[4];
      frag_a(Ks, LDA, r0, k0, g, t, ak);
      frag_a(Qs, LDA, r0, k0, g, t, aq);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t b[2];
        frag_bt(Ks, LDA, k0, c0 + j * 8, g, t, b);
        mma_tf32(kk[j], ak[0], ak[1], ak[2], ak[3], b[0], b[1]);
        mma_tf32(qk[j], aq[0], aq[1], aq[2], aq[3], b[0], b[1]);
      }
    }
    float* icap = a.ica + ((int64_t)h * a.nc + n) * L * L;
    bf16* icab = reinterpret_cast<bf16*>(a.ica) + ((int64_t)h * a.nc + n) * L * L;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = r0 + g + ((e & 2) ? 8 : 0), jj = c0 + j * 8 + 2 * t + (e & 1);
        const float dec = (jj <= i) ? __expf(cs[i] - cs[jj]) : 0.f;
        Tm[i * LDL + jj] = (jj < i) ? bs[i] * dec * kk[j][e] : 0.f;
        if (BF) icab[i * L + jj] = __float2bfloat16(dec * qk[j][e]);
        else icap[i * L + jj] = dec * qk[j][e];
      }
  }
  // ---- qe = e^c Q for the scan (Q's last use), zero the inverse ---------------------------------
  {
    float* qep = a.qe + ((int64_t)h * a.nc + n) * L * DK;
    bf16* qeb = reinterpret_cast<bf16*>(a.qe) + ((int64_t)h * a.nc + n) * L * DK;
    for (int idx = tid; idx < L * DK / 4; idx += 256) {
      const int i = idx / (DK / 4), c = (idx % (DK / 4)) * 4;
      const float ec = __expf(cs[i]);
      const float4 q = *reinterpret_cast<const float4*>(Qs + i * LDA + c);
      if (BF) *reinterpret_cast<uint2*>(qeb + (int64_t)i * DK + c) = make_uint2(pack_bf162(q.x * ec, q.y * ec), pack_bf162(q.z * ec, q.w * ec));
      else *reinterpret_cast<float4*>(qep + (int64_t)i * DK + c) = make_float4(q.x * ec, q.y * ec, q.z * ec, q.w * ec);
    }
    for (int idx = tid; idx < L * L; idx += 256) Wi[(idx / L) * LDL + idx % L] = 0.f;
  }
  __syncthreads();                                   // Tm complete, Q no longer needed
  // ---- W = (I + Tm)^-1, blocked: the four 16x16 diagonal blocks are inverted by forward
  // substitution (one warp each, one column per lane, 16 dependent rows instead of 64), then the
  // blocks below the diagonal follow level by level from  W_ij = -W_ii (sum_{k=j..i-1} T_ik W_kj).
  if (warp < 4 && lane < 16) {
    const int b0 = warp * 16, c = lane;
    for (int i = 0; i < 16; ++i) {
      float acc = (i == c) ? 1.f : 0.f;
      for (int jj = c; jj < i; ++jj) acc -= Tm[(b0 + i) * LDL + b0 + jj] * Wi[(b0 + jj) * LDL + b0 + c];
      if (i >= c) Wi[(b0 + i) * LDL + b0 + c] = acc;
    }
  }
  __syncthreads();
  {
    float* P = R2;                                    // scratch for the block sums (Q is gone, e^c K not yet there)
    for (int d = 1; d < 4; ++d) {
      const int npairs = 4 - d;
      // P_p = sum_{k=j}^{i-1} T_ik W_kj for the pairs (i = j + d, j)
      for (int idx = tid; idx < npairs * 256; idx += 256) {
        const int pr = idx >> 8, r = (idx >> 4) & 15, c = idx & 15;
        const int j = pr, i = pr + d;
        float acc = 0.f;
        for (int kk = j * 16; kk < i * 16; ++kk) acc += Tm[(i * 16 + r) * LDL + kk] * Wi[kk * LDL + j * 16 + c];
        P[idx] = acc;
      }
      __syncthreads();
      for (int idx = tid; idx < npairs * 256; idx += 256) {
        const int pr = idx >> 8, r = (idx >> 4) & 15, c = idx & 15;
        const int j = pr, i = pr + d;
        float acc = 0.f;
        for (int kk = 0; kk <= r; ++kk) acc += Wi[(i * 16 + r) * LDL + i * 16 + kk] * P[(pr << 8) + kk * 16 + c];
        Wi[(i * 16 + r) * LDL + j * 16 + c] = -acc;
      }
      __syncthreads();
    }
  }
  // ---- W <- W diag(beta) (both products below carry beta); ke and e^c K from K -------------------
  {
    for (int idx = tid; idx < L * L; idx += 256) Wi[(idx / L) * LDL + idx % L] *= bs[idx % L];
    float* kep = a.ke + ((int64_t)h * a.nc + n) * L * DK;
    bf16* keb = reinterpret_cast<bf16*>(a.ke) + ((int64_t)h * a.nc + n) * L * DK;
    const float cl = cs[L - 1];
    for (int idx = tid; idx < L * DK / 4; idx += 256) {
      const int i = idx / (DK / 4), c = (idx % (DK / 4)) * 4;
      const float ec = __expf(cs[i]), el = __expf(cl - cs[i]);
      const float4 k = *reinterpret_cast<const float4*>(Ks + i * LDA + c);
      if (BF) *reinterpret_cast<uint2*>(keb + (int64_t)i * DK + c) = make_uint2(pack_bf162(k.x * el, k.y * el), pack_bf162(k.z * el, k.w * el));
      else *reinterpret_cast<float4*>(kep + (int64_t)i * DK + c) = make_float4(k.x * el, k.y * el, k.z * el, k.w * el);
      *reinterpret_cast<float4*>(Kb + i * LDB + c) = make_float4(k.x * ec, k.y * ec, k.z * ec, k.w * ec);
    }
    if (tid == 0) a.ecl[(int64_t)h * a.nc + n] = __expf(cl);
  }
  __syncthreads();                                   // K is no longer needed: V takes its place
  // ---- nvv = W' V, kcd = W' (e^c K): warp (row tile) x (V or K half); W' is lower triangular ------
  {
    const int r0 = (warp & 3) * 16;
    const bool isv = (warp >> 2) == 0;
    if (isv) {                                       // the four V warps fetch V while the K warps multiply
      if (FUSE) {                                    // conv + SiLU of the value channels: 16 tokens per warp, 8 at a time
        const int i0 = lane * 4;
        const bool act = i0 < DV;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
          const int tl = warp * 16 + half * 8;
          float val[8][4];
          conv_tokens<8>(a.proj, a.ldp, a.ring, conv_dim, a.conv_w, 2 * kdim + h * DV + i0, act, (int)t0 + tl, a.T, a.pos0, val);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            if (act) *reinterpret_cast<float4*>(Vs + (tl + k) * LDV + i0) = make_float4(val[k][0], val[k][1], val[k][2], val[k][3]);
        }
      } else {
        for (int idx = tid; idx < L * DV / 4; idx += 128) {
          const int i = idx / (DV / 4), c = (idx % (DV / 4)) * 4;
          cp_async16(Vs + i * LDV + c, vp + (int64_t)i * DV + c);
        }
        cp_async_commit();
        cp_async_wait_all();
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    const float* B = isv ? Vs : Kb;
    const int ldb = isv ? LDV : LDB;
    constexpr int NT = (DV > DK ? DV : DK) / 8;
    const int nt = (isv ? DV : DK) / 8;
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
    for (int k0 = 0; k0 < r0 + 16; k0 += 8) {
      uint32_t aw[4];
      frag_a(Wi, LDL, r0, k0, g, t, aw);
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        if (j < nt) {
          uint32_t b[2];
          frag_b(B, ldb, k0, j * 8, g, t, b);
          mma_tf32(acc[j], aw[0], aw[1], aw[2], aw[3], b[0], b[1]);
        }
      }
    }
    float* dst = isv ? a.nvv + ((int64_t)h * a.nc + n) * L * DV : a.kcd + ((int64_t)h * a.nc + n) * L * DK;
    bf16* dstb = reinterpret_cast<bf16*>(a.kcd) + ((int64_t)h * a.nc + n) * L * DK;
    const int ldd = isv ? DV : DK;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      if (j < nt) {
        if (BF && !isv) {
          *reinterpret_cast<uint32_t*>(dstb + (r0 + g) * ldd + j * 8 + 2 * t) = pack_bf162(acc[j][0], acc[j][1]);
          *reinterpret_cast<uint32_t*>(dstb + (r0 + g + 8) * ldd + j * 8 + 2 * t) = pack_bf162(acc[j][2], acc[j][3]);
        } else {
          *reinterpret_cast<float2*>(dst + (r0 + g) * ldd + j * 8 + 2 * t) = make_float2(acc[j][0], acc[j][1]);
          *reinterpret_cast<float2*>(dst + (r0 + g + 8) * ldd + j * 8 + 2 * t) = make_float2(acc[j][2], acc[j][3]);
        }
      }
    }
  }
}

template <int DK, int DVS>
struct ScanTcLayout {
  static constexpr int L = kChunk, LDS = DVS + 8, LDA = DK + 4, LDT = DK + 8, LDL = L + 4;
  // S [DK][LDS], A1 = kcd [L][LDA], A2 = qe [L][LDA], A3 = ke [L][LDT] (read transposed), Ic [L][LDL], U [L][LDS]
  static constexpr size_t floats = (size_t)DK * LDS + (size_t)2 * L * LDA + (size_t)L * LDT + (size_t)L * LDL + (size_t)L * LDS;
};

template <int DK, int DV, int DVS>
__global__ void __launch_bounds__(256) gdn_chunk_scan_tc_kernel(const GdnScanArgs a) {
  using Lay = ScanTcLayout<DK, DVS>;
  constexpr int L = kChunk, LDS = Lay::LDS, LDA = Lay::LDA, LDT = Lay::LDT, LDL = Lay::LDL;
  constexpr int NRT = DK / 16;                 // row tiles of the state
  constexpr int CG = 8 / NRT;                  // column groups the 8 warps split the state update into
  constexpr int NTS = (DVS / 8) / CG;          // n-tiles per warp in the state update
  static_assert(DVS == 32 && (DK == 64 || DK == 128), "tiling");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* S = reinterpret_cast<float*>(smem_raw);
  float* A1 = S + DK * LDS;
  float* A2 = A1 + L * LDA;
  float* A3 = A2 + L * LDA;
  float* Ic = A3 + L * LDT;
  float* U = Ic + L * LDL;
  griddep_launch();
  griddep_wait();
  const int h = blockIdx.x, sl = blockIdx.y, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int col0 = sl * DVS;
  float* sp = a.state + (int64_t)h * DK * DV + col0;
  for (int idx = tid; idx < DK * DVS; idx += 256) S[(idx / DVS) * LDS + idx % DVS] = sp[(int64_t)(idx / DVS) * DV + idx % DVS];
  const int r0 = (warp & 3) * 16, ch = (warp >> 2) * 16;          // U / O tile of this warp: 16 rows x 16 columns
  const int s0 = (warp % NRT) * 16, sc0 = (warp / NRT) * (DVS / CG);   // state tile: 16 rows x NTS*8 columns
  // Operand loads are asynchronous copies in two groups, so that they overlap the products: kcd and
  // qe of chunk n+1 are fetched while chunk n runs its second half (they are free once U exists), ke
  // and ica of chunk n while it runs its first half (the previous chunk's state update was their
  // last reader).  Two barriers per chunk.
  auto load_a12 = [&](int n) {
    const int64_t base = (int64_t)h * a.nc + n;
    for (int idx = tid; idx < L * DK / 4; idx += 256) {
      const int i = idx / (DK / 4), c = (idx % (DK / 4)) * 4;
      const int64_t off = base * L * DK + (int64_t)i * DK + c;
      cp_async16(A1 + i * LDA + c, a.kcd + off);
      cp_async16(A2 + i * LDA + c, a.qe + off);
    }
    cp_async_commit();
  };
  auto load_a3i = [&](int n) {
    const int64_t base = (int64_t)h * a.nc + n;
    for (int idx = tid; idx < L * DK / 4; idx += 256) {
      const int i = idx / (DK / 4), c = (idx % (DK / 4)) * 4;
      cp_async16(A3 + i * LDT + c, a.ke + base * L * DK + (int64_t)i * DK + c);
    }
    for (int idx = tid; idx < L * L / 4; idx += 256) {
      const int i = idx / (L / 4), c = (idx % (L / 4)) * 4;
      cp_async16(Ic + i * LDL + c, a.ica + base * L * L + (int64_t)i * L + c);
    }
    cp_async_commit();
  };
  load_a12(0);
  for (int n = 0; n < a.nc; ++n) {
    const int64_t base = (int64_t)h * a.nc + n;
    cp_async_wait_all();
    __syncthreads();          // kcd, qe of this chunk visible; every warp has left the previous chunk
    load_a3i(n);
    const float el = a.ecl[base];
    float2 nv0[2], nv1[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float* nvp = a.nvv + base * L * DV + col0 + ch + j * 8 + 2 * t;
      nv0[j] = *reinterpret_cast<const float2*>(nvp + (int64_t)(r0 + g) * DV);
      nv1[j] = *reinterpret_cast<const float2*>(nvp + (int64_t)(r0 + g + 8) * DV);
    }
    // ---- accU = kcd S, accO = qe S ------------------------------------------------------------
    float accU[2][4] = {}, accO[2][4] = {};
    for (int k0 = 0; k0 < DK; k0 += 8) {
      uint32_t ak[4], aq[4];
      frag_a(A1, LDA, r0, k0, g, t, ak);
      frag_a(A2, LDA, r0, k0, g, t, aq);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint32_t b[2];
        frag_b(S, LDS, k0, ch + j * 8, g, t, b);
        mma_tf32(accU[j], ak[0], ak[1], ak[2], ak[3], b[0], b[1]);
        mma_tf32(accO[j], aq[0], aq[1], aq[2], aq[3], b[0], b[1]);
      }
    }
    // ---- U = nvv - accU -> shared ---------------------------------------------------------------
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      *reinterpret_cast<float2*>(U + (r0 + g) * LDS + ch + j * 8 + 2 * t) = make_float2(nv0[j].x - accU[j][0], nv0[j].y - accU[j][1]);
      *reinterpret_cast<float2*>(U + (r0 + g + 8) * LDS + ch + j * 8 + 2 * t) = make_float2(nv1[j].x - accU[j][2], nv1[j].y - accU[j][3]);
    }
    cp_async_wait_all();
    __syncthreads();          // U, ke and ica visible; kcd and qe are free
    if (n + 1 < a.nc) load_a12(n + 1);
    // ---- O += ica U (ica is lower triangular: k <= row) -----------------------------------------
    for (int k0 = 0; k0 < r0 + 16; k0 += 8) {
      uint32_t ai[4];
      frag_a(Ic, LDL, r0, k0, g, t, ai);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        uint32_t b[2];
        frag_b(U, LDS, k0, ch + j * 8, g, t, b);
        mma_tf32(accO[j], ai[0], ai[1], ai[2], ai[3], b[0], b[1]);
      }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int64_t ta = (int64_t)n * L + r0 + g, tb = ta + 8;
      float* op = a.out + (int64_t)h * DV + col0 + ch + j * 8 + 2 * t;
      if (ta < a.T) *reinterpret_cast<float2*>(op + ta * a.nv * DV) = make_float2(accO[j][0], accO[j][1]);
      if (tb < a.T) *reinterpret_cast<float2*>(op + tb * a.nv * DV) = make_float2(accO[j][2], accO[j][3]);
    }
    // ---- S <- ecl S + ke^T U: warp owns a 16-row tile of the state --------------------------------
    float accS[NTS][4];
#pragma unroll
    for (int j = 0; j < NTS; ++j) {
      const float2 x0 = *reinterpret_cast<const float2*>(S + (s0 + g) * LDS + sc0 + j * 8 + 2 * t);
      const float2 x1 = *reinterpret_cast<const float2*>(S + (s0 + g + 8) * LDS + sc0 + j * 8 + 2 * t);
      accS[j][0] = x0.x * el; accS[j][1] = x0.y * el; accS[j][2] = x1.x * el; accS[j][3] = x1.y * el;
    }
    for (int k0 = 0; k0 < L; k0 += 8) {
      uint32_t at[4];
      frag_at(A3, LDT, s0, k0, g, t, at);
#pragma unroll
      for (int j = 0; j < NTS; ++j) {
        uint32_t b[2];
        frag_b(U, LDS, k0, sc0 + j * 8, g, t, b);
        mma_tf32(accS[j], at[0], at[1], at[2], at[3], b[0], b[1]);
      }
    }
    // every warp has finished reading S for this chunk (the barrier after U); the tile is this warp's own
#pragma unroll
    for (int j = 0; j < NTS; ++j) {
      *reinterpret_cast<float2*>(S + (s0 + g) * LDS + sc0 + j * 8 + 2 * t) = make_float2(accS[j][0], accS[j][1]);
      *reinterpret_cast<float2*>(S + (s0 + g + 8) * LDS + sc0 + j * 8 + 2 * t) = make_float2(accS[j][2], accS[j][3]);
    }
  }
  __syncthreads();
  for (int idx = tid; idx < DK * DVS; idx += 256) sp[(int64_t)(idx / DVS) * DV + idx % DVS] = S[(idx / DVS) * LDS + idx % DVS];
}

// ---------------------------------------------------------------------------------------------
// bf16-operand scan.  The same recurrence with kcd, qe, ke, ica (written as bf16 by the prepare kernel)
// and the copies of S and U that enter a product rounded to bf16 (mma.m16n8k16, fp32 accumulate); the
// state itself stays fp32 in the registers of the warp that owns its tile, from the first chunk to the
// last.  Half-size operands make room for a three-stage ring of whole-chunk operand sets, so the loads
// of chunk n+2 are in flight while chunk n is multiplied: the TF32 scan could only look half a chunk
// ahead and spent most of a chunk waiting for L2.  Fragments come from ldmatrix (.trans where the
// stored layout has the reduction index in rows); row strides of 16 B (mod 128) keep them conflict free.
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t smem_u32addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async_wait_1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

template <int DK, int DVS>
struct ScanBfLayout {
  static constexpr int L = kChunk, LDA = DK + 8, LDL = L + 8, LDS = DVS + 8, STAGES = 3;
  // stage: kcd [L][LDA], qe [L][LDA], ke [L][LDA], ica [L][LDL] (bf16); then S copy [DK][LDS], U [L][LDS] (bf16)
  static constexpr size_t stage_bytes = 2 * ((size_t)3 * L * LDA + (size_t)L * LDL);
  static constexpr size_t bytes = STAGES * stage_bytes + 2 * ((size_t)DK * LDS + (size_t)L * LDS);
};

template <int DK, int DV, int DVS>
__global__ void __launch_bounds__(256) gdn_chunk_scan_bf_kernel(const GdnScanArgs a) {
  using Lay = ScanBfLayout<DK, DVS>;
  constexpr int L = kChunk, LDA = Lay::LDA, LDL = Lay::LDL, LDS = Lay::LDS, ST = Lay::STAGES;
  constexpr int NRT = DK / 16;                 // row tiles of the state
  constexpr int CG = 8 / NRT;                  // column groups the 8 warps split the state into
  constexpr int NTS = (DVS / 8) / CG;          // n-tiles of a warp's state tile (2 or 4)
  static_assert(DVS == 32 && (DK == 64 || DK == 128), "tiling");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Sb = reinterpret_cast<bf16*>(smem_raw + ST * Lay::stage_bytes);
  bf16* Ub = Sb + DK * LDS;
  griddep_launch();
  griddep_wait();
  const int h = blockIdx.x, sl = blockIdx.y, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int col0 = sl * DVS;
  const bf16* kcd = reinterpret_cast<const bf16*>(a.kcd);
  const bf16* qe = reinterpret_cast<const bf16*>(a.qe);
  const bf16* ke = reinterpret_cast<const bf16*>(a.ke);
  const bf16* ica = reinterpret_cast<const bf16*>(a.ica);
  auto load_chunk = [&](int n) {
    if (n < a.nc) {
      bf16* st = reinterpret_cast<bf16*>(smem_raw + (size_t)(n % ST) * Lay::stage_bytes);
      const int64_t base = (int64_t)h * a.nc + n;
      for (int idx = tid; idx < L * DK / 8; idx += 256) {
        const int i = idx / (DK / 8), c = (idx % (DK / 8)) * 8;
        const int64_t off = base * L * DK + (int64_t)i * DK + c;
        cp_async16(st + i * LDA + c, kcd + off);
        cp_async16(st + L * LDA + i * LDA + c, qe + off);
        cp_async16(st + 2 * L * LDA + i * LDA + c, ke + off);
      }
      for (int idx = tid; idx < L * L / 8; idx += 256) {
        const int i = idx / (L / 8), c = (idx % (L / 8)) * 8;
        cp_async16(st + 3 * L * LDA + i * LDL + c, ica + base * L * L + (int64_t)i * L + c);
      }
    }
    cp_async_commit();            // one group per chunk, empty past the end: the wait below counts groups
  };
  load_chunk(0);
  load_chunk(1);
  const int r0 = (warp & 3) * 16, ch = (warp >> 2) * 16;                // U / O tile of this warp: 16 rows x 16 columns
  const int s0 = (warp % NRT) * 16, sc0 = (warp / NRT) * (NTS * 8);    // state tile: 16 rows x NTS*8 columns
  // the warp's tile of the state: fp32 in registers for the whole scan, bf16 copy in shared memory
  float* sp = a.state + (int64_t)h * DK * DV + col0;
  float accS[NTS][4];
#pragma unroll
  for (int j = 0; j < NTS; ++j) {
    const float2 x0 = *reinterpret_cast<const float2*>(sp + (int64_t)(s0 + g) * DV + sc0 + j * 8 + 2 * t);
    const float2 x1 = *reinterpret_cast<const float2*>(sp + (int64_t)(s0 + g + 8) * DV + sc0 + j * 8 + 2 * t);
    accS[j][0] = x0.x; accS[j][1] = x0.y; accS[j][2] = x1.x; accS[j][3] = x1.y;
    *reinterpret_cast<uint32_t*>(Sb + (s0 + g) * LDS + sc0 + j * 8 + 2 * t) = pack_bf162(x0.x, x0.y);
    *reinterpret_cast<uint32_t*>(Sb + (s0 + g + 8) * LDS + sc0 + j * 8 + 2 * t) = pack_bf162(x1.x, x1.y);
  }
  // per-lane fragment addresses (element offsets inside a tile)
  const int a_row = (lane & 7) + ((lane >> 3) & 1) * 8, a_col = (lane >> 4) * 8;        // A, row-major
  const int t_row = (lane & 7) + ((lane >> 4) & 1) * 8, t_col = ((lane >> 3) & 1) * 8;  // A from transposed storage
  const int b_row = (lane & 7) + ((lane >> 3) & 1) * 8, b_col = (lane >> 4) * 8;        // B from [k][n] storage
  const uint32_t sb_u = smem_u32addr(Sb), ub_u = smem_u32addr(Ub);
  // nvv and e^{c_L} of the next chunk travel in registers, one chunk ahead
  float2 nv0[2], nv1[2];
  float el = 0.f;
  auto load_nv = [&](int n) {
    if (n < a.nc) {
      const int64_t base = (int64_t)h * a.nc + n;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float* nvp = a.nvv + base * L * DV + col0 + ch + j * 8 + 2 * t;
        nv0[j] = *reinterpret_cast<const float2*>(nvp + (int64_t)(r0 + g) * DV);
        nv1[j] = *reinterpret_cast<const float2*>(nvp + (int64_t)(r0 + g + 8) * DV);
      }
      el = a.ecl[base];
    }
  };
  load_nv(0);
  for (int n = 0; n < a.nc; ++n) {
    cp_async_wait_1();
    __syncthreads();          // chunk n's operands and the S copy are visible; every warp has left chunk n-1
    load_chunk(n + 2);
    const uint32_t st_u = smem_u32addr(smem_raw + (size_t)(n % ST) * Lay::stage_bytes);
    const uint32_t a1_u = st_u, a2_u = st_u + 2 * L * LDA, a3_u = st_u + 4 * L * LDA, ic_u = st_u + 6 * L * LDA;
    const float2 cnv0[2] = {nv0[0], nv0[1]}, cnv1[2] = {nv1[0], nv1[1]};
    const float cel = el;
    load_nv(n + 1);
    // ---- accU = kcd S, accO = qe S ------------------------------------------------------------
    float accU[2][4] = {}, accO[2][4] = {};
#pragma unroll
    for (int k0 = 0; k0 < DK; k0 += 16) {
      uint32_t ak[4], aq[4], b[4];
      ldsm_x4(a1_u + 2 * ((r0 + a_row) * LDA + k0 + a_col), ak);
      ldsm_x4(a2_u + 2 * ((r0 + a_row) * LDA + k0 + a_col), aq);
      ldsm_x4_t(sb_u + 2 * ((k0 + b_row) * LDS + ch + b_col), b);
      mma_bf16(accU[0], ak, b[0], b[1]);
      mma_bf16(accU[1], ak, b[2], b[3]);
      mma_bf16(accO[0], aq, b[0], b[1]);
      mma_bf16(accO[1], aq, b[2], b[3]);
    }
    // ---- U = nvv - accU -> shared (bf16) ----------------------------------------------------------
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      *reinterpret_cast<uint32_t*>(Ub + (r0 + g) * LDS + ch + j * 8 + 2 * t) = pack_bf162(cnv0[j].x - accU[j][0], cnv0[j].y - accU[j][1]);
      *reinterpret_cast<uint32_t*>(Ub + (r0 + g + 8) * LDS + ch + j * 8 + 2 * t) = pack_bf162(cnv1[j].x - accU[j][2], cnv1[j].y - accU[j][3]);
    }
    __syncthreads();          // U visible; every warp is done reading the S copy
    // ---- O += ica U (ica is lower triangular: k <= row) -----------------------------------------
    for (int k0 = 0; k0 < r0 + 16; k0 += 16) {
      uint32_t ai[4], b[4];
      ldsm_x4(ic_u + 2 * ((r0 + a_row) * LDL + k0 + a_col), ai);
      ldsm_x4_t(ub_u + 2 * ((k0 + b_row) * LDS + ch + b_col), b);
      mma_bf16(accO[0], ai, b[0], b[1]);
      mma_bf16(accO[1], ai, b[2], b[3]);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int64_t ta = (int64_t)n * L + r0 + g, tb = ta + 8;
      float* op = a.out + (int64_t)h * DV + col0 + ch + j * 8 + 2 * t;
      if (ta < a.T) *reinterpret_cast<float2*>(op + ta * a.nv * DV) = make_float2(accO[j][0], accO[j][1]);
      if (tb < a.T) *reinterpret_cast<float2*>(op + tb * a.nv * DV) = make_float2(accO[j][2], accO[j][3]);
    }
    // ---- S <- ecl S + ke^T U on the warp's own tile; refresh the bf16 copy -----------------------
#pragma unroll
    for (int j = 0; j < NTS; ++j) { accS[j][0] *= cel; accS[j][1] *= cel; accS[j][2] *= cel; accS[j][3] *= cel; }
#pragma unroll
    for (int k0 = 0; k0 < L; k0 += 16) {
      uint32_t at[4];
      ldsm_x4_t(a3_u + 2 * ((k0 + t_row) * LDA + s0 + t_col), at);
#pragma unroll
      for (int jj = 0; jj < NTS; jj += 2) {
        uint32_t b[4];
        ldsm_x4_t(ub_u + 2 * ((k0 + b_row) * LDS + sc0 + jj * 8 + b_col), b);
        mma_bf16(accS[jj], at, b[0], b[1]);
        mma_bf16(accS[jj + 1], at, b[2], b[3]);
      }
    }
#pragma unroll
    for (int j = 0; j < NTS; ++j) {
      *reinterpret_cast<uint32_t*>(Sb + (s0 + g) * LDS + sc0 + j * 8 + 2 * t) = pack_bf162(accS[j][0], accS[j][1]);
      *reinterpret_cast<uint32_t*>(Sb + (s0 + g + 8) * LDS + sc0 + j * 8 + 2 * t) = pack_bf162(accS[j][2], accS[j][3]);
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
#pragma unroll
  for (int j = 0; j < NTS; ++j) {
    *reinterpret_cast<float2*>(sp + (int64_t)(s0 + g) * DV + sc0 + j * 8 + 2 * t) = make_float2(accS[j][0], accS[j][1]);
    *reinterpret_cast<float2*>(sp + (int64_t)(s0 + g + 8) * DV + sc0 + j * 8 + 2 * t) = make_float2(accS[j][2], accS[j][3]);
  }
}

// out[t, h*DV + j] = bf16( o * rsqrt(mean_j o^2 + eps) * w[j] * silu(z) ), one warp per (t, h)
template <int DV>
__global__ void gdn_gated_norm_kernel(const float* o, const bf16* z, int64_t ldz, const float* w, bf16* out,
                                      int64_t ldo, int T, int nv, float eps, int gate_sigmoid) {
  griddep_launch();
  griddep_wait();
  const int lane = threadIdx.x & 31;
  const int64_t task = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (task >= (int64_t)T * nv) return;
  const int64_t t = task / nv;
  const int h = task % nv;
  constexpr int E = DV / 32;                 // consecutive elements per lane (2 or 4): vector loads and stores
  static_assert(E == 2 || E == 4, "head width");
  const int j0 = lane * E;
  float x[E], ss = 0.f;
  const float* op = o + (t * nv + h) * DV + j0;
  if (E == 4) { const float4 v = *reinterpret_cast<const float4*>(op); x[0] = v.x; x[1] = v.y; x[E - 2] = v.z; x[E - 1] = v.w; }
  else { const float2 v = *reinterpret_cast<const float2*>(op); x[0] = v.x; x[1] = v.y; }
#pragma unroll
  for (int e = 0; e < E; ++e) ss += x[e] * x[e];
  const float r = rsqrtf(warp_sum(ss) / (float)DV + eps);
  uint32_t zz[E / 2], oo[E / 2];
  const bf16* zp = z + t * ldz + h * DV + j0;
  if (E == 4) { const uint2 v = *reinterpret_cast<const uint2*>(zp); zz[0] = v.x; zz[E / 2 - 1] = v.y; }
  else zz[0] = *reinterpret_cast<const uint32_t*>(zp);
#pragma unroll
  for (int e = 0; e < E; e += 2) {
    const float z0 = __uint_as_float(zz[e / 2] << 16), z1 = __uint_as_float(zz[e / 2] & 0xffff0000u);
    const float g0 = gate_sigmoid ? sigmoid_f(z0) : silu_f(z0), g1 = gate_sigmoid ? sigmoid_f(z1) : silu_f(z1);
    oo[e / 2] = pack_bf162(x[e] * r * w[j0 + e] * g0, x[e + 1] * r * w[j0 + e + 1] * g1);
  }
  bf16* dp = out + t * ldo + h * DV + j0;
  if (E == 4) *reinterpret_cast<uint2*>(dp) = make_uint2(oo[0], oo[E / 2 - 1]);
  else *reinterpret_cast<uint32_t*>(dp) = oo[0];
}

template <int DK, int DV>
size_t chunk_prepare_smem() {
  return sizeof(float) * (size_t)(2 * kChunk * (DK + 4) + kChunk * (DV + 4) + 2 * kChunk * (kChunk + 1) + 2 * kChunk);
}
template <int DK, int DVS>
size_t chunk_scan_smem() {
  return sizeof(float) * (size_t)(DK * (DVS + 4) + 2 * kChunk * (DK + 4) + kChunk * (kChunk + 4) + kChunk * (DVS + 4));
}

int g_gdn_tc = 3;    // chunk kernels: 3 = prep fused into the TF32 prepare + bf16-operand scan, 2 = the same with the
                     // prep kernel as a launch of its own, 1 = TF32 for both, 0 = fp32 SIMT versions

template <typename K>
int set_smem(K kern, size_t smem) {
  if (smem + 2048 > 48 * 1024) {   // the 48 KB default also has to hold the static shared memory
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

}  // namespace

CB_EXPORT int cb_gdn_decode(const void* proj, int64_t ldp, const void* conv_w, const void* A_log,
                            const void* dt_bias, const void* norm_w, void* ring, void* state,
                            const void* slots, const void* positions, void* out, int64_t ldo,
                            void* record, int64_t rec_w, int64_t M, int64_t ntok, int64_t write_state,
                            int64_t nk, int64_t nv, int64_t dk, int64_t dv, float eps, int64_t gate_sigmoid,
                            void* stream) {
  if (nv % nk || M < 1 || ntok < 1 || ntok > 12) return CB_ERR_SHAPE;
  GdnDecodeArgs a;
  a.gate_sigmoid = (int)gate_sigmoid;
  a.proj = (const bf16*)proj; a.ldp = ldp; a.conv_w = (const float*)conv_w; a.A_log = (const float*)A_log;
  a.dt_bias = (const float*)dt_bias; a.norm_w = (const float*)norm_w; a.ring = (bf16*)ring;
  a.state = (float*)state; a.slots = (const int*)slots; a.positions = (const int*)positions;
  a.out = (bf16*)out; a.ldo = ldo; a.record = (float*)record; a.rec_w = (int)rec_w; a.ntok = (int)ntok;
  a.write_state = (int)write_state; a.nk = (int)nk; a.nv = (int)nv; a.rep = (int)(nv / nk); a.eps = eps;
  dim3 grid((unsigned)nv, (unsigned)M);
  if (dk == 128 && dv == 128 && nv * M > 2 * 148)
    return (int)cb_launch(gdn_decode_kernel<128, 128, 2>, grid, dim3(512), 0, (cudaStream_t)stream, a);
  if (dk == 128 && dv == 128) return (int)cb_launch(gdn_decode_kernel<128, 128>, grid, dim3(512), 0, (cudaStream_t)stream, a);
  if (dk == 64 && dv == 64) return (int)cb_launch(gdn_decode_kernel<64, 64>, grid, dim3(256), 0, (cudaStream_t)stream, a);
  return CB_ERR_SHAPE;
}

// 3: conv / norm / beta / g inside the TF32 prepare kernel + bf16-operand scan with a three-stage operand ring
// (default); 2: the same with the prep kernel launched separately; 1: TF32 chunk kernels; 0: the fp32 SIMT versions.
CB_EXPORT int cb_set_gdn_tc(int64_t mode) { g_gdn_tc = mode < 0 ? 0 : (mode > 3 ? 3 : (int)mode); return 0; }

CB_EXPORT int cb_gdn_commit(void* state, const void* record, const void* slots, const void* steps,
                            int64_t rec_w, int64_t M, int64_t nv, int64_t dk, int64_t dv, void* stream) {
  dim3 grid((unsigned)nv, (unsigned)M);
  if (dk == 128 && dv == 128)
    return (int)cb_launch(gdn_commit_kernel<128, 128>, grid, dim3(512), 0, (cudaStream_t)stream, (float*)state,
                          (const float*)record, (const int*)slots, (const int*)steps, (int)rec_w, (int)nv);
  if (dk == 64 && dv == 64)
    return (int)cb_launch(gdn_commit_kernel<64, 64>, grid, dim3(256), 0, (cudaStream_t)stream, (float*)state,
                          (const float*)record, (const int*)slots, (const int*)steps, (int)rec_w, (int)nv);
  return CB_ERR_SHAPE;
}

// Whole prefill chain for one sequence chunk of T tokens starting at pos0.
// scratch (fp32) must hold cb_gdn_prefill_scratch(T, ...) floats.
CB_EXPORT int64_t cb_gdn_prefill_scratch(int64_t T, int64_t nk, int64_t nv, int64_t dk, int64_t dv) {
  const int64_t nc = (T + kChunk - 1) / kChunk, Tp = nc * kChunk;
  return 2 * nk * Tp * dk + nv * Tp * dv + 2 * nv * Tp       // qn kn v beta g
         + nv * nc * kChunk * (dv + 3 * dk + kChunk) + ((nv * nc + 3) & ~(int64_t)3)  // nvv kcd qe ke ica ecl
         + T * nv * dv;                                        // scan output
}

CB_EXPORT int cb_gdn_prefill(const void* proj, int64_t ldp, const void* conv_w, const void* A_log,
                             const void* dt_bias, const void* norm_w, void* ring_seq, void* state_seq,
                             void* scratch, void* out, int64_t ldo, int64_t T, int64_t pos0, int64_t nk,
                             int64_t nv, int64_t dk, int64_t dv, float eps, int64_t gate_sigmoid, void* stream) {
  if (T < 1 || nv % nk) return CB_ERR_SHAPE;
  // the ring update moves whole 16-byte vectors of a projection row
  if (ldp % 8 || (2 * nk * dk + nv * dv) % 8 || ((uintptr_t)proj & 15) || ((uintptr_t)ring_seq & 15)) return CB_ERR_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t nc = (T + kChunk - 1) / kChunk, Tp = nc * kChunk;
  const int conv_dim = (int)(2 * nk * dk + nv * dv);
  float* p = (float*)scratch;
  float* qn = p; p += nk * Tp * dk;
  float* kn = p; p += nk * Tp * dk;
  float* v = p; p += nv * Tp * dv;
  float* beta = p; p += nv * Tp;
  float* g = p; p += nv * Tp;
  float* nvv = p; p += nv * nc * kChunk * dv;
  float* kcd = p; p += nv * nc * kChunk * dk;
  float* qe = p; p += nv * nc * kChunk * dk;
  float* ke = p; p += nv * nc * kChunk * dk;
  float* ica = p; p += nv * nc * kChunk * kChunk;
  float* ecl = p; p += (nv * nc + 3) & ~(int64_t)3;
  float* o = p;
  GdnPrepArgs pa{(const bf16*)proj, ldp, (const float*)conv_w, (const float*)A_log, (const float*)dt_bias,
                 (const bf16*)ring_seq, qn, kn, v, beta, g, (int)T, (int)Tp, (int)pos0, (int)nk, (int)nv};
  GdnChunkArgs ca{qn, kn, v, beta, g, nvv, kcd, ica, qe, ke, ecl, (int)Tp, (int)nc, (int)(nv / nk),
                  (const bf16*)proj, ldp, (const float*)conv_w, (const float*)A_log, (const float*)dt_bias,
                  (const bf16*)ring_seq, (int)T, (int)pos0, (int)nk, (int)nv};
  GdnScanArgs sa{nvv, kcd, ica, qe, ke, ecl, (float*)state_seq, o, (int)T, (int)nc, (int)nv};
  cudaError_t e;
  int rc;
#define GDN_PREFILL(DK_, DV_, DVS_)                                                                      \
  do {                                                                                                   \
    if (g_gdn_tc != 3) {                                                                                 \
      e = cb_launch(gdn_prep_kernel<DK_, DV_>, dim3((unsigned)((Tp + kPrepTok - 1) / kPrepTok)), dim3(256), 0, st, pa);                \
      if (e != cudaSuccess) return (int)e;                                                               \
    }                                                                                                    \
    if (g_gdn_tc >= 2) {                                                                                 \
      /* the fused prepare kernel reads the ring (rows before the chunk), so the ring moves on after it */ \
      size_t s1 = sizeof(float) * PrepTcLayout<DK_, DV_>::floats;                                        \
      if (g_gdn_tc == 3) {                                                                               \
        if ((rc = set_smem(gdn_chunk_prepare_tc_kernel<DK_, DV_, true, true>, s1))) return rc;           \
        e = cb_launch(gdn_chunk_prepare_tc_kernel<DK_, DV_, true, true>, dim3((unsigned)nc, (unsigned)nv), dim3(256), s1, st, ca); \
      } else {                                                                                           \
        if ((rc = set_smem(gdn_chunk_prepare_tc_kernel<DK_, DV_, true>, s1))) return rc;                 \
        e = cb_launch(gdn_chunk_prepare_tc_kernel<DK_, DV_, true>, dim3((unsigned)nc, (unsigned)nv), dim3(256), s1, st, ca); \
      }                                                                                                  \
      if (e != cudaSuccess) return (int)e;                                                               \
      e = cb_launch(gdn_ring_update_kernel, dim3((unsigned)(T < kRing ? T : kRing)), dim3(256), 0, st,   \
                    (const bf16*)proj, ldp, (bf16*)ring_seq, (int)T, (int)pos0, conv_dim);               \
      if (e != cudaSuccess) return (int)e;                                                               \
      size_t s2 = ScanBfLayout<DK_, DVS_>::bytes;                                                        \
      if ((rc = set_smem(gdn_chunk_scan_bf_kernel<DK_, DV_, DVS_>, s2))) return rc;                      \
      e = cb_launch(gdn_chunk_scan_bf_kernel<DK_, DV_, DVS_>, dim3((unsigned)nv, (unsigned)(DV_ / DVS_)), \
                    dim3(256), s2, st, sa);                                                              \
      if (e != cudaSuccess) return (int)e;                                                               \
    } else if (g_gdn_tc) {                                                                               \
      e = cb_launch(gdn_ring_update_kernel, dim3((unsigned)(T < kRing ? T : kRing)), dim3(256), 0, st,   \
                    (const bf16*)proj, ldp, (bf16*)ring_seq, (int)T, (int)pos0, conv_dim);               \
      if (e != cudaSuccess) return (int)e;                                                               \
      size_t s1 = sizeof(float) * PrepTcLayout<DK_, DV_>::floats;                                        \
      if ((rc = set_smem(gdn_chunk_prepare_tc_kernel<DK_, DV_>, s1))) return rc;                         \
      e = cb_launch(gdn_chunk_prepare_tc_kernel<DK_, DV_>, dim3((unsigned)nc, (unsigned)nv), dim3(256), s1, st, ca); \
      if (e != cudaSuccess) return (int)e;                                                               \
      size_t s2 = sizeof(float) * ScanTcLayout<DK_, DVS_>::floats;                                       \
      if ((rc = set_smem(gdn_chunk_scan_tc_kernel<DK_, DV_, DVS_>, s2))) return rc;                      \
      e = cb_launch(gdn_chunk_scan_tc_kernel<DK_, DV_, DVS_>, dim3((unsigned)nv, (unsigned)(DV_ / DVS_)), \
                    dim3(256), s2, st, sa);                                                              \
      if (e != cudaSuccess) return (int)e;                                                               \
    } else {                                                                                             \
      e = cb_launch(gdn_ring_update_kernel, dim3((unsigned)(T < kRing ? T : kRing)), dim3(256), 0, st,   \
                    (const bf16*)proj, ldp, (bf16*)ring_seq, (int)T, (int)pos0, conv_dim);               \
      if (e != cudaSuccess) return (int)e;                                                               \
      size_t s1 = chunk_prepare_smem<DK_, DV_>();                                                        \
      if ((rc = set_smem(gdn_chunk_prepare_kernel<DK_, DV_>, s1))) return rc;                            \
      e = cb_launch(gdn_chunk_prepare_kernel<DK_, DV_>, dim3((unsigned)nc, (unsigned)nv), dim3(256), s1, st, ca); \
      if (e != cudaSuccess) return (int)e;                                                               \
      size_t s2 = chunk_scan_smem<DK_, DVS_>();                                                          \
      if ((rc = set_smem(gdn_chunk_scan_kernel<DK_, DV_, DVS_>, s2))) return rc;                         \
      e = cb_launch(gdn_chunk_scan_kernel<DK_, DV_, DVS_>, dim3((unsigned)nv, (unsigned)(DV_ / DVS_)),    \
                    dim3(256), s2, st, sa);                                                              \
      if (e != cudaSuccess) return (int)e;                                                               \
    }                                                                                                    \
    const int64_t tasks = T * nv;                                                                        \
    e = cb_launch(gdn_gated_norm_kernel<DV_>, dim3((unsigned)((tasks + 7) / 8)), dim3(256), 0, st,       \
                  (const float*)o, (const bf16*)proj + conv_dim, ldp, (const float*)norm_w, (bf16*)out,  \
                  ldo, (int)T, (int)nv, eps, (int)gate_sigmoid);                                         \
    return (int)e;                                                                                       \
  } while (0)
  if (dk == 128 && dv == 128) GDN_PREFILL(128, 128, 32);
  if (dk == 64 && dv == 64) GDN_PREFILL(64, 64, 32);
#undef GDN_PREFILL
  return CB_ERR_SHAPE;
}
