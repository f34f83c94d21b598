// Tensor-parallel all-reduce folded into the projections, over peer memory (NVLink / NVSwitch).
//
// A row-parallel projection leaves every rank with a partial sum of the hidden vector.  Instead of
// a collective call between kernels, the producing GEMV *pushes* its partial rows straight into an
// inbox on every rank (plain peer stores through IPC-mapped pointers), each value paired with the
// step's epoch; the consumer *pulls*: a one-CTA kernel per row (comm.cu) or the consumer phase of
// the persistent decode kernel (decode_mega.cu) polls (bounded) every rank's element until it
// carries this step's epoch and adds them in rank order to the residual.  The sum order is fixed,
// hence every rank computes bit-identical activations.  Replaces the reference's per-projection gloo all-reduce of
// RowParallelProjection (models/qwen35/parallel.py:1015-1061) and the idea of its p2p_combine kernel
// (backends/corex/kernels/p2p_reduce.cu:55-173: write to all peers, publish flag, bounded spin).
//
// The epoch is a device-side counter every rank advances once per step, so buffers
// are reused without resetting: a site's inbox can only be overwritten a full step later, and a rank
// cannot get there before all peers consumed the previous contents because it needs their partial
// sums of the sites in between.  Waits give up after the limit, set the status word and continue
// with whatever is in the inbox, so a dead peer costs an error, not a hung GPU; once the status word
// is set no later wait spins (the step finishes at once with garbage, and the host, which reads the
// word after every step, raises).
#pragma once
#include "common.cuh"

constexpr int kTpMaxWorld = 8;
constexpr unsigned long long kTpWaitNs = 2000000000ull;   // default limit of a device-side wait: 2 s

struct TpComm {
  int rank, world;
  int64_t slot_floats;      // floats per (site, rank) inbox slot  (= max rows * hidden)
  float* inbox[kTpMaxWorld];       // base of every rank's inbox: [sites][world][slot_floats] {value, epoch} pairs
  unsigned* flags[kTpMaxWorld];    // base of every rank's flags: [sites][world]
  const float* my_inbox;    // == inbox[rank]; a separate field so that no kernel indexes the arrays
  const unsigned* my_flags; // == flags[rank]  with a run-time value (that would copy the parameter
                            //    block to local memory in every thread)
  unsigned* arrive;         // local: [sites] CTA arrival counters of the producer
  const unsigned* epoch;    // local: current step number
  int* status;              // local status word (set to 16 + rank on a wait that ran out)
  unsigned long long wait_ns;   // limit of a device-side wait (0: kTpWaitNs)
};

__device__ __forceinline__ unsigned long long tp_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned tp_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void tp_st_release(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Data and flag travel together (the "low-latency" layout of collective libraries): an inbox element
// is an aligned 8-byte pair {fp32 value, epoch}, written with one 64-bit store.  The consumer polls
// the element itself until its epoch word equals the current step, so the producer needs no fence,
// no arrival counter and no separate flag, and the consumer sees a value the moment it lands.
__device__ __forceinline__ void tp_st_pair(float* slot_base, int64_t elem, float v, unsigned epoch) {
  const unsigned long long packed = ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
  asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(reinterpret_cast<unsigned long long*>(slot_base) + elem),
               "l"(packed) : "memory");
}
__device__ __forceinline__ unsigned long long tp_ld_pair(const float* slot_base, int64_t elem) {
  unsigned long long v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v)
               : "l"(reinterpret_cast<const unsigned long long*>(slot_base) + elem) : "memory");
  return v;
}
// Producer: store the fp32 partial value of element `off` of this rank's slot on every rank.
// Called by the thread that owns the value.
__device__ __forceinline__ void tp_push_value(const TpComm& c, int site, int64_t off, float v) {
  const int64_t elem = ((int64_t)site * c.world + c.rank) * c.slot_floats + off;
  const unsigned e = *c.epoch;
#pragma unroll
  for (int p = 0; p < kTpMaxWorld; ++p)
    if (p < c.world) tp_st_pair(c.inbox[p], elem, v, e);
}
__device__ __forceinline__ int tp_status_set(const int* status) {
  return *reinterpret_cast<const volatile int*>(status);
}
// Consumer: sum of the ranks' partial values at element `off` (fixed rank order).  Polls every
// rank's element until it carries this step's epoch; gives up after the wait limit, records
// 16 + rank in the status word and uses what is there.
__device__ __forceinline__ float tp_pull_value(const TpComm& c, int site, int64_t off) {
  const unsigned e = *c.epoch;
  float s = 0.f;
  for (int r = 0; r < c.world; ++r) {
    const int64_t elem = ((int64_t)site * c.world + r) * c.slot_floats + off;
    unsigned long long v = tp_ld_pair(c.my_inbox, elem);
    if ((unsigned)(v >> 32) != e) {
      const unsigned long long t0 = tp_now_ns(), limit = c.wait_ns ? c.wait_ns : kTpWaitNs;
      unsigned spins = 0;
      if (tp_status_set(c.status)) spins = ~0u;   // an earlier wait already ran out: do not spin again
      while ((unsigned)(v >> 32) != e && spins != ~0u) {
        if ((++spins & 255u) == 0) {
          if (tp_status_set(c.status)) break;
          if (tp_now_ns() - t0 > limit) {
            atomicCAS(c.status, 0, 16 + r);
            break;
          }
        }
        v = tp_ld_pair(c.my_inbox, elem);
      }
    }
    s += __uint_as_float((unsigned)v);
  }
  return s;
}

// Consumer, vector form: sums of 8 consecutive elements starting at `off` (a multiple of 8).  The 64
// bytes of a rank's 8 pairs are fetched with four independent 16-byte loads before any flag is
// looked at, so a thread pays one memory round trip per rank instead of eight; only pairs that have
// not landed yet are polled again.
__device__ __forceinline__ void tp_pull8(const TpComm& c, int site, int64_t off, float* out) {
  const unsigned e = *c.epoch;
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = 0.f;
  for (int r = 0; r < c.world; ++r) {
    const unsigned long long* base = reinterpret_cast<const unsigned long long*>(c.my_inbox) +
                                     ((int64_t)site * c.world + r) * c.slot_floats + off;
    uint4 q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(q[j].x), "=r"(q[j].y), "=r"(q[j].z), "=r"(q[j].w) : "l"(base + 2 * j) : "memory");
    bool ok = true;
#pragma unroll
    for (int j = 0; j < 4; ++j) ok = ok && q[j].y == e && q[j].w == e;
    if (!ok) {
      const unsigned long long t0 = tp_now_ns(), limit = c.wait_ns ? c.wait_ns : kTpWaitNs;
      unsigned spins = 0;
      if (tp_status_set(c.status)) ok = true;     // an earlier wait already ran out: do not spin again
      while (!ok) {
        if ((++spins & 63u) == 0) {
          if (tp_status_set(c.status)) break;
          if (tp_now_ns() - t0 > limit) {
            atomicCAS(c.status, 0, 16 + r);
            break;
          }
        }
        ok = true;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (q[j].y != e || q[j].w != e)
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(q[j].x), "=r"(q[j].y), "=r"(q[j].z), "=r"(q[j].w) : "l"(base + 2 * j) : "memory");
          ok = ok && q[j].y == e && q[j].w == e;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      out[2 * j] += __uint_as_float(q[j].x);
      out[2 * j + 1] += __uint_as_float(q[j].z);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Prefill: row-parallel GEMM -> all-reduce as reduce-scatter + all-gather over peer memory.
//
// The GEMM epilogue (gemm_tc.cu, gemm_tc2.cu) leaves every bf16 partial row in this rank's own
// peer-visible buffer ("inbox") at its row index and the last CTA publishes the sequence number to
// every rank; rows are cut into `world` equal slices, and a small kernel on each rank then PULLS the
// slice it owns from every rank's buffer (coalesced 16-byte peer loads), adds the partial rows in rank
// order (+ an optional residual) and stores the reduced rows into every rank's result buffer.  Two flag arrays carry a sequence number that the host advances once per use (all
// ranks run the same sequence of calls), so nothing is reset between uses; waits are bounded and
// set the status word.  This replaces the reference's per-projection gloo all-reduce in prefill
// (models/qwen35/parallel.py:1015-1061) and is what NCCL all-reduce would otherwise do between
// kernels.
// The descriptor lives in device memory (kernels index its pointer tables with run-time ranks).
struct TpPfDev {
  int rank, world;
  int rows_per_rank;          // rows of one slice = ceil(max chunk rows / world)
  int width;                  // row width in elements (hidden size)
  bf16* inbox[kTpMaxWorld];       // rank p's partial rows, all of them: [world * rows_per_rank][width]; row r is
                                  // pulled by its owner, rank r / rows_per_rank
  bf16* out[kTpMaxWorld];         // rank p's result: [world * rows_per_rank][width]
  unsigned* flags1[kTpMaxWorld];  // rank p's flags: [source rank] that rank's partial rows are complete
  unsigned* flags2[kTpMaxWorld];  // rank p's flags: [source rank] reduced rows have landed
  unsigned* arrive;               // local: [2] CTA arrival counters (scatter, gather)
  int* status;
  unsigned long long wait_ns;     // limit of a device-side wait (0: kTpWaitNs)
  unsigned* seq_dev;              // local: sequence number of the last completed all-reduce
  bf16* os_inbox[kTpMaxWorld];    // rank p's one-shot inbox: [2 halves][source rank][64 rows][width] (comm.cu)
};

// Sequence number of the all-reduce in progress.  The kernels are passed 0 and take "last completed
// + 1" from device memory (the wait kernel, last of the three, stores it back), so a captured CUDA
// graph advances the numbering on every replay; a non-zero argument is used as it is.
__device__ __forceinline__ unsigned tp_pf_seq(const TpPfDev* d, unsigned seq_arg) {
  return seq_arg ? seq_arg : *reinterpret_cast<const volatile unsigned*>(d->seq_dev) + 1u;
}

// Bounded wait for `flags[0..world)` (local) to reach `seq`. Thread 0 of the block waits.
__device__ __forceinline__ void tp_pf_wait(const unsigned* flags, int world, unsigned seq, int* status,
                                           unsigned long long wait_ns) {
  if (threadIdx.x == 0) {
    const unsigned long long t0 = tp_now_ns();
    const unsigned long long limit = wait_ns ? wait_ns : kTpWaitNs;
    for (int r = 0; r < world; ++r) {
      unsigned spins = 0;
      if (tp_status_set(status)) break;           // an earlier wait already ran out: do not spin again
      while ((int)(tp_ld_acquire(flags + r) - seq) < 0) {
        if ((++spins & 1023u) == 0) {
          if (tp_status_set(status)) break;
          if (tp_now_ns() - t0 > limit) {
            atomicCAS(status, 0, 32 + r);
            break;
          }
        }
      }
    }
  }
  __syncthreads();
}
// After a CTA's peer stores: the last CTA of the grid publishes `seq` in slot [my rank] of every
// rank's flag array `which` (1 or 2). `arrive_slot` is 0 for the scatter, 1 for the gather.
__device__ __forceinline__ void tp_pf_publish(const TpPfDev* d, int which, unsigned seq, unsigned nblocks) {
  // callers have done __threadfence_system() + a barrier over the storing threads
  const unsigned prev = atomicAdd(d->arrive + (which - 1), 1u);
  if (prev == nblocks - 1) {
    seq = tp_pf_seq(d, seq);
    d->arrive[which - 1] = 0;
    __threadfence_system();
    for (int p = 0; p < d->world; ++p)
      tp_st_release((which == 1 ? d->flags1[p] : d->flags2[p]) + d->rank, seq);
  }
}
