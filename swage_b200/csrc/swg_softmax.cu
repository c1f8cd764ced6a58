// Segmented softmax, fp32 in / fp32 out:
//   m = max(x), d = sum(exp(x - m)), out[i] = exp(x[i] - m) / d
// over each segment, written to the segment's own range of `out`; an empty
// segment writes nothing.  This is the reference's semantic form
// (test/Dialect/Swage/softmax.mlir:13-31, docs/adr/ADR-0008:24-32); the
// reference has no lowering for it (roadmap M5), so there is no kernel to
// compare mappings with -- the arithmetic contract is the three steps above.
//
// HBM-bound: 8 bytes per value (read once, written once) + 4 per offset.  The
// schedules here read a segment from HBM once; the second and third sweeps of
// a segment that does not fit in registers or shared memory are served by L2
// (loads keep the default caching policy on the first sweep for that reason,
// stores are streaming).
#include <mutex>

#include "swg_common.cuh"
#include "swg_launch.h"

namespace swg {

constexpr float kLog2e = 1.4426950408889634f;

// exp(x) for x <= 0 (and NaN / -inf pass through as NaN / 0): one multiply
// and one MUFU.EX2.  Relative error ~2^-22, far inside the stated tolerance.
__device__ __forceinline__ float exp_neg(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x * kLog2e));
  return r;
}

// One thread's share of sum(exp(v[begin,end) - m)).
__device__ __forceinline__ float strided_expsum(const float *__restrict__ v,
                                                int64_t begin, int64_t end,
                                                float m, int rank,
                                                int nthreads) {
  const float *p = v + begin;
  const int64_t len = end - begin;
  float acc = 0.0f;
  if (len <= 0) return acc;
  int head = head_elems(p);
  if (head > len) head = (int)len;
  if (rank < head) acc += exp_neg(p[rank] - m);
  const float4 *body = reinterpret_cast<const float4 *>(p + head);
  const int64_t nvec = (len - head) >> 2;
  float a1 = 0.0f;
  int64_t i = rank;
  for (; i + nthreads < nvec; i += 2 * (int64_t)nthreads) {
    const float4 q0 = body[i], q1 = body[i + nthreads];
    acc += (exp_neg(q0.x - m) + exp_neg(q0.y - m)) +
           (exp_neg(q0.z - m) + exp_neg(q0.w - m));
    a1 += (exp_neg(q1.x - m) + exp_neg(q1.y - m)) +
          (exp_neg(q1.z - m) + exp_neg(q1.w - m));
  }
  if (i < nvec) {
    const float4 q0 = body[i];
    acc += (exp_neg(q0.x - m) + exp_neg(q0.y - m)) +
           (exp_neg(q0.z - m) + exp_neg(q0.w - m));
  }
  acc += a1;
  const int64_t tail = head + (nvec << 2);
  if (rank < (int)(len - tail)) acc += exp_neg(p[tail + rank] - m);
  return acc;
}

// One thread's share of the normalise-and-store sweep.  `out` has the same
// 16-byte phase as `v` only when both base pointers agree; otherwise scalar.
__device__ __forceinline__ void strided_normalise(const float *__restrict__ v,
                                                  float *__restrict__ out,
                                                  int64_t begin, int64_t end,
                                                  float m, float inv, int rank,
                                                  int nthreads) {
  const float *p = v + begin;
  float *o = out + begin;
  const int64_t len = end - begin;
  if (len <= 0) return;
  const bool same_phase = (((uintptr_t)p ^ (uintptr_t)o) & 15u) == 0;
  if (!same_phase) {
    for (int64_t i = rank; i < len; i += nthreads)
      __stcs(o + i, exp_neg(p[i] - m) * inv);
    return;
  }
  int head = head_elems(p);
  if (head > len) head = (int)len;
  if (rank < head) __stcs(o + rank, exp_neg(p[rank] - m) * inv);
  const float4 *body = reinterpret_cast<const float4 *>(p + head);
  float4 *obody = reinterpret_cast<float4 *>(o + head);
  const int64_t nvec = (len - head) >> 2;
  for (int64_t i = rank; i < nvec; i += nthreads) {
    const float4 q = body[i];
    float4 r;
    r.x = exp_neg(q.x - m) * inv;
    r.y = exp_neg(q.y - m) * inv;
    r.z = exp_neg(q.z - m) * inv;
    r.w = exp_neg(q.w - m) * inv;
    __stcs(obody + i, r);
  }
  const int64_t tail = head + (nvec << 2);
  if (rank < (int)(len - tail))
    __stcs(o + tail + rank, exp_neg(p[tail + rank] - m) * inv);
}

// Max sweep that leaves the lines in L2 for the two sweeps that follow.
__device__ __forceinline__ float strided_max_keep(const float *__restrict__ v,
                                                  int64_t begin, int64_t end,
                                                  int rank, int nthreads) {
  const float *p = v + begin;
  const int64_t len = end - begin;
  float acc = MaxOp::identity();
  if (len <= 0) return acc;
  int head = head_elems(p);
  if (head > len) head = (int)len;
  if (rank < head) acc = MaxOp::apply(acc, p[rank]);
  const float4 *body = reinterpret_cast<const float4 *>(p + head);
  const int64_t nvec = (len - head) >> 2;
  float a1 = MaxOp::identity();
  int64_t i = rank;
  for (; i + nthreads < nvec; i += 2 * (int64_t)nthreads) {
    acc = fold4<MaxOp>(acc, body[i]);
    a1 = fold4<MaxOp>(a1, body[i + nthreads]);
  }
  if (i < nvec) acc = fold4<MaxOp>(acc, body[i]);
  acc = MaxOp::apply(acc, a1);
  const int64_t tail = head + (nvec << 2);
  if (rank < (int)(len - tail)) acc = MaxOp::apply(acc, p[tail + rank]);
  return acc;
}

__global__ void __launch_bounds__(256)
segsoftmax_cta_kernel(const float *__restrict__ values,
                      const int32_t *__restrict__ offsets,
                      float *__restrict__ out, int32_t segment_count) {
  __shared__ float scratch[32];
  for (int64_t seg = blockIdx.x; seg < segment_count; seg += gridDim.x) {
    const int64_t begin = __ldg(offsets + seg);
    const int64_t end = __ldg(offsets + seg + 1);
    if (end <= begin) continue;
    float m = strided_max_keep(values, begin, end, threadIdx.x, blockDim.x);
    m = cta_reduce<MaxOp>(m, scratch);
    float d = strided_expsum(values, begin, end, m, threadIdx.x, blockDim.x);
    d = cta_reduce<SumOp>(d, scratch);
    strided_normalise(values, out, begin, end, m, 1.0f / d, threadIdx.x,
                      blockDim.x);
  }
}

__global__ void __launch_bounds__(256)
segsoftmax_warp_kernel(const float *__restrict__ values,
                       const int32_t *__restrict__ offsets,
                       float *__restrict__ out, int32_t segment_count) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t seg = warp; seg < segment_count; seg += nwarps) {
    const int64_t begin = __ldg(offsets + seg);
    const int64_t end = __ldg(offsets + seg + 1);
    if (end <= begin) continue;
    float m = strided_max_keep(values, begin, end, lane, kWarp);
    m = warp_reduce<MaxOp>(m);
    float d = strided_expsum(values, begin, end, m, lane, kWarp);
    d = warp_reduce<SumOp>(d);
    strided_normalise(values, out, begin, end, m, 1.0f / d, lane, kWarp);
  }
}

// ---------------------------------------------------------------------------
// Planned schedule.
// ---------------------------------------------------------------------------

// Resident buckets: a segment of at most kThreads * kResidentRows values is
// held in the registers of kThreads threads (one warp, or a CTA of 128 or 512
// threads): every value is read from HBM exactly once and written exactly
// once, with coalesced 4-byte accesses, so no alignment case exists.
constexpr int kResidentRows = 16;

template <int kThreads>
__global__ void __launch_bounds__(kThreads == 32 ? 256 : kThreads,
                                  kThreads == 512 ? 3 : 1)
segsoftmax_resident_kernel(const float *__restrict__ values,
                           const int32_t *__restrict__ offsets,
                           float *__restrict__ out,
                           const int32_t *__restrict__ segments,
                           int32_t count) {
  __shared__ float scratch[32];
  const int t = kThreads == 32 ? (int)(threadIdx.x & 31) : (int)threadIdx.x;
  const int64_t which =
      kThreads == 32
          ? (((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5)
          : (int64_t)blockIdx.x;
  if (which >= count) return;
  const int32_t seg = __ldg(segments + which);
  const int64_t begin = __ldg(offsets + seg);
  const int length = (int)(__ldg(offsets + seg + 1) - begin);
  const float *p = values + begin + t;
  float x[kResidentRows];
#pragma unroll
  for (int r = 0; r < kResidentRows; ++r)
    x[r] = (r * kThreads + t < length) ? __ldcs(p + r * kThreads)
                                       : MaxOp::identity();
  float m = x[0];
#pragma unroll
  for (int r = 1; r < kResidentRows; ++r) m = MaxOp::apply(m, x[r]);
  m = kThreads == 32 ? warp_reduce<MaxOp>(m) : cta_reduce<MaxOp>(m, scratch);
  float d = 0.0f;
#pragma unroll
  for (int r = 0; r < kResidentRows; ++r) {
    // padding slots are masked: exp(-inf - m) is 0 only for an ordered m
    const float e = (r * kThreads + t < length) ? exp_neg(x[r] - m) : 0.0f;
    x[r] = e;
    d += e;
  }
  d = kThreads == 32 ? warp_reduce<SumOp>(d) : cta_reduce<SumOp>(d, scratch);
  const float inv = 1.0f / d;
  float *o = out + begin + t;
#pragma unroll
  for (int r = 0; r < kResidentRows; ++r)
    if (r * kThreads + t < length) __stcs(o + r * kThreads, x[r] * inv);
}

// Long bucket: one CTA per segment, two sweeps.  Sweep A reads the segment
// from HBM once (loads carry an L2 evict-last policy so the lines stay for
// sweep B) and keeps a running (maximum, sum of exp) pair per thread,
// rescaling the sum only when a batch of 16 values raises the maximum; sweep
// B re-reads the segment from L2 and writes the normalised values with
// streaming stores.  Both sweeps issue a batch of independent 128-bit loads
// before touching any of them.  Two 512-thread CTAs per SM keep the set of
// live segments (296 of them) far below the L2 capacity; the register cap
// (room for three CTAs) leaves space for the resident buckets' CTAs to run
// beside them.
#ifndef SWG_SOFTMAX_LONG_THREADS
#define SWG_SOFTMAX_LONG_THREADS 512
#endif
#ifndef SWG_SOFTMAX_LONG_CTAS
#define SWG_SOFTMAX_LONG_CTAS 2
#endif
constexpr int kLongThreads = SWG_SOFTMAX_LONG_THREADS;
constexpr int kLongCtasPerSm = SWG_SOFTMAX_LONG_CTAS;
#ifndef SWG_SOFTMAX_LONG_BATCH
#define SWG_SOFTMAX_LONG_BATCH 4
#endif
#ifndef SWG_SOFTMAX_LONG_MINBLOCKS
#define SWG_SOFTMAX_LONG_MINBLOCKS 3
#endif
constexpr int kLongBatch = SWG_SOFTMAX_LONG_BATCH;  // 128-bit loads in flight per thread, sweep A

struct MaxSum {
  float m, d;
};

__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t policy;
  asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

__device__ __forceinline__ float4 ld_keep4(const float4 *p, uint64_t policy) {
  float4 q;
  asm volatile("ld.global.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
               : "=f"(q.x), "=f"(q.y), "=f"(q.z), "=f"(q.w)
               : "l"(p), "l"(policy));
  return q;
}

__device__ __forceinline__ float max4(const float4 q) {
  return MaxOp::apply(MaxOp::apply(q.x, q.y), MaxOp::apply(q.z, q.w));
}

// s.m only ever takes ordered values: a NaN batch maximum fails `lm > s.m`.
// NaN is tracked by the caller's NaN-propagating maximum instead.
__device__ __forceinline__ void online_raise(MaxSum &s, const float lm) {
  if (lm > s.m) {
    s.d *= exp_neg(s.m - lm);
    s.m = lm;
  }
}

__device__ __forceinline__ float expsum4(const float4 q, const float m) {
  return (exp_neg(q.x - m) + exp_neg(q.y - m)) +
         (exp_neg(q.z - m) + exp_neg(q.w - m));
}

__device__ __forceinline__ void online_add1(MaxSum &s, const float v) {
  online_raise(s, v);
  // while only -inf has been seen every term is exp(-inf) = 0 against any
  // finite final maximum; adding exp(-inf - -inf) = NaN would poison the sum
  if (s.m > -CUDART_INF_F) s.d += exp_neg(v - s.m);
}

__device__ __forceinline__ float4 normalise4(const float4 q, const float m,
                                             const float inv) {
  float4 r;
  r.x = exp_neg(q.x - m) * inv;
  r.y = exp_neg(q.y - m) * inv;
  r.z = exp_neg(q.z - m) * inv;
  r.w = exp_neg(q.w - m) * inv;
  return r;
}

__global__ void __launch_bounds__(kLongThreads, SWG_SOFTMAX_LONG_MINBLOCKS)
segsoftmax_long_kernel(const float *__restrict__ values,
                       const int32_t *__restrict__ offsets,
                       float *__restrict__ out,
                       const int32_t *__restrict__ segments, int32_t count) {
  __shared__ float scratch[32];
  const int tid = threadIdx.x;
  const uint64_t keep = policy_evict_last();
  constexpr int64_t T = kLongThreads;
  for (int64_t j = blockIdx.x; j < count; j += gridDim.x) {
    const int32_t seg = __ldg(segments + j);
    const int64_t begin = __ldg(offsets + seg);
    const int64_t end = __ldg(offsets + seg + 1);
    const float *p = values + begin;
    float *o = out + begin;
    const int64_t len = end - begin;
    int head = head_elems(p);
    if (head > len) head = (int)len;
    const float4 *body = reinterpret_cast<const float4 *>(p + head);
    const int64_t nvec = (len - head) >> 2;
    const int64_t tail = head + (nvec << 2);
    const int tail_count = (int)(len - tail);

    // ---- sweep A ----
    MaxSum s{-CUDART_INF_F, 0.0f};
    float any = MaxOp::identity();  // NaN-propagating maximum
    if (tid < head) {
      online_add1(s, p[tid]);
      any = MaxOp::apply(any, p[tid]);
    }
    int64_t i = tid;
    for (; i + (kLongBatch - 1) * T < nvec; i += kLongBatch * T) {
      float4 q[kLongBatch];
#pragma unroll
      for (int k = 0; k < kLongBatch; ++k) q[k] = ld_keep4(body + i + k * T, keep);
      float lm = max4(q[0]);
#pragma unroll
      for (int k = 1; k < kLongBatch; ++k) lm = MaxOp::apply(lm, max4(q[k]));
      any = MaxOp::apply(any, lm);
      online_raise(s, lm);
      if (s.m > -CUDART_INF_F) {
        float d0 = 0.0f, d1 = 0.0f;
#pragma unroll
        for (int k = 0; k < kLongBatch; k += 2) {
          d0 += expsum4(q[k], s.m);
          d1 += expsum4(q[k + 1], s.m);
        }
        s.d += d0 + d1;
      }
    }
    for (; i < nvec; i += T) {
      const float4 q = ld_keep4(body + i, keep);
      const float lm = max4(q);
      any = MaxOp::apply(any, lm);
      online_raise(s, lm);
      if (s.m > -CUDART_INF_F) s.d += expsum4(q, s.m);
    }
    if (tid < tail_count) {
      online_add1(s, p[tail + tid]);
      any = MaxOp::apply(any, p[tail + tid]);
    }
    // combine: the segment maximum first (NaN-propagating), then the sums
    // rescaled to it
    const float m = cta_reduce<MaxOp>(any, scratch);
    const float mine = s.d == 0.0f ? 0.0f : s.d * exp_neg(s.m - m);
    const float d = cta_reduce<SumOp>(mine, scratch);
    const float inv = 1.0f / d;

    // ---- sweep B ----
    const bool same_phase = (((uintptr_t)p ^ (uintptr_t)o) & 15u) == 0;
    if (!same_phase) {
      for (int64_t e = tid; e < len; e += T)
        __stcs(o + e, exp_neg(p[e] - m) * inv);
      continue;
    }
    if (tid < head) __stcs(o + tid, exp_neg(p[tid] - m) * inv);
    float4 *obody = reinterpret_cast<float4 *>(o + head);
    i = tid;
    for (; i + 3 * T < nvec; i += 4 * T) {
      const float4 q0 = __ldcs(body + i), q1 = __ldcs(body + i + T),
                   q2 = __ldcs(body + i + 2 * T), q3 = __ldcs(body + i + 3 * T);
      __stcs(obody + i, normalise4(q0, m, inv));
      __stcs(obody + i + T, normalise4(q1, m, inv));
      __stcs(obody + i + 2 * T, normalise4(q2, m, inv));
      __stcs(obody + i + 3 * T, normalise4(q3, m, inv));
    }
    for (; i < nvec; i += T)
      __stcs(obody + i, normalise4(__ldcs(body + i), m, inv));
    if (tid < tail_count)
      __stcs(o + tail + tid, exp_neg(p[tail + tid] - m) * inv);
  }
}

// Ring kernel: one CTA per segment, two sweeps through a ring of kRingStages
// shared-memory stages of kRingChunk values, filled by bulk async copies that
// thread 0 issues up to a full ring ahead of the readers.
//
//   sweep A  chunks 0 .. n-1: running (maximum, sum of exp) per thread;
//   sweep B  chunks n-1 .. 0: normalise and store.
//
// Sweep B walks backwards, so the last kRingStages chunks of sweep A are still
// in the ring and are not loaded again: a segment of up to kRingStages chunks
// is read from HBM once and never again, a longer one re-reads all but its
// tail, most recent lines first, which L2 serves (sweep A loads of chunks
// that will come back carry an evict-last policy, everything else
// evict-first).  Chunk c lives in stage c % kRingStages in both sweeps.
//
// A chunk is a run of whole 16-byte lines of `values` counted from the line
// that holds the segment's first value, so every copy is aligned whatever
// the offsets are; the up-to-three values that share a line with the array's
// ends are fetched by plain loads.
//
// Every stage has a `full` barrier (one arrival + the copy's bytes per load)
// and an `empty` barrier (one arrival per warp, after the last read of what
// was loaded).  All waits are bounded; a wait that gives up raises the
// plan's timeout flag and the CTA walks to the end without touching the ring.
#ifndef SWG_RING_STAGES
#define SWG_RING_STAGES 8
#endif
constexpr int kRingStages = SWG_RING_STAGES;
constexpr int kRingChunk = 2048;
constexpr int kRingThreads = 256;
constexpr int kRingWarps = kRingThreads / 32;
constexpr int kRingVectors = kRingChunk / 4 / kRingThreads;  // per thread
static_assert(kRingStages >= 2 && kRingStages <= 27, "ring size");
constexpr int kRingBytes = kRingStages * kRingChunk * 4;
// CTAs that fit an SM's 227 KB of shared memory (1 KB reserved per CTA)
constexpr int kRingCtasPerSm =
    (227 * 1024) / (kRingBytes + 1024 + 256) < 2048 / kRingThreads
        ? (227 * 1024) / (kRingBytes + 1024 + 256)
        : 2048 / kRingThreads;
#ifndef SWG_SOFTMAX_RING
#define SWG_SOFTMAX_RING 1
#endif

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t policy;
  asm("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

__device__ __forceinline__ void bulk_g2s_hint(void *dst_smem,
                                              const void *src_gmem,
                                              uint32_t bytes, uint64_t *bar,
                                              uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

struct RingSegment {
  int64_t begin, end;  // the segment's values
  int64_t origin;      // index of slot 0: the aligned line holding `begin`
  int64_t last_line;   // first index past the last whole line of the array
  int64_t line_end;    // index past the line holding the segment's last value
  int mis;             // (values pointer / 4) mod 4
};

// Thread 0 only: waits until the stage's previous contents have been read by
// every warp, then starts the copy of chunk `c` into it.
__device__ __forceinline__ bool ring_issue(const RingSegment &g,
                                           const float *__restrict__ values,
                                           float *ring, uint64_t *full,
                                           uint64_t *empty, int64_t c,
                                           uint32_t &loaded,
                                           uint32_t &empty_parity,
                                           uint64_t policy) {
  const int stage = (int)(c % kRingStages);
  const uint32_t bit = 1u << stage;
  if (loaded & bit) {
    if (!mbar_wait(&empty[stage], (empty_parity & bit) ? 1u : 0u)) return false;
    empty_parity ^= bit;
  }
  loaded |= bit;
  float *slot = ring + stage * kRingChunk;
  const int64_t g0 = g.origin + c * kRingChunk;
  int64_t g1 = g0 + kRingChunk;
  if (g1 > g.line_end) g1 = g.line_end;
  int64_t lo = g0 < 0 ? g0 + 4 : g0;
  int64_t hi = g1 > g.last_line ? g.last_line : g1;
  if (hi < lo) hi = lo;
  const int64_t vb = g.begin > g0 ? g.begin : g0;
  const int64_t ve = g.end < g1 ? g.end : g1;
  for (int64_t i = vb; i < ve && i < lo; ++i) slot[i - g0] = values[i];
  for (int64_t i = hi > vb ? hi : vb; i < ve; ++i) slot[i - g0] = values[i];
  const uint32_t bytes = (uint32_t)(hi - lo) * 4u;
  mbar_arrive_expect_tx(&full[stage], bytes);
  if (bytes)
    bulk_g2s_hint(slot + (lo - g0), values + lo, bytes, &full[stage], policy);
  return true;
}

__global__ void __launch_bounds__(kRingThreads)
segsoftmax_ring_kernel(const float *__restrict__ values,
                       const int32_t *__restrict__ offsets,
                       float *__restrict__ out,
                       const int32_t *__restrict__ segments, int32_t count,
                       int32_t value_count, uint32_t *__restrict__ control) {
  extern __shared__ __align__(128) unsigned char smem[];
  float *ring = reinterpret_cast<float *>(smem);
  __shared__ uint64_t full[kRingStages], empty[kRingStages];
  __shared__ float scratch[32];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < kRingStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kRingWarps);
    }
    fence_mbar_init();
  }
  __syncthreads();
  const uint64_t keep = policy_evict_last();
  const uint64_t once = policy_evict_first();
  RingSegment g;
  g.mis = (int)(((uintptr_t)values >> 2) & 3);
  g.last_line = (int64_t)value_count - ((value_count + g.mis) & 3);
  const bool same_phase =
      (int)(((uintptr_t)out >> 2) & 3) == g.mis;  // lines of out = lines of values
  uint32_t full_parity = 0;                // every thread, one bit per stage
  uint32_t empty_parity = 0, loaded = 0;   // thread 0
  bool failed = false;

  for (int64_t j = blockIdx.x; j < count; j += gridDim.x) {
    const int32_t seg = __ldg(segments + j);
    g.begin = __ldg(offsets + seg);
    g.end = __ldg(offsets + seg + 1);
    const int shift = (int)((g.begin + g.mis) & 3);
    g.origin = g.begin - shift;
    g.line_end = g.end + ((4 - ((g.end + g.mis) & 3)) & 3);
    const int64_t slots = (int64_t)shift + (g.end - g.begin);  // valid: [shift, slots)
    const int64_t n = (slots + kRingChunk - 1) / kRingChunk;
    const int64_t resident_from = n > kRingStages ? n - kRingStages : 0;

    if (tid == 0 && !failed)
      for (int64_t c = 0; c < n && c < kRingStages && !failed; ++c)
        failed = !ring_issue(g, values, ring, full, empty, c, loaded,
                             empty_parity, c < resident_from ? keep : once);

    // ---- sweep A ----
    MaxSum s{-CUDART_INF_F, 0.0f};
    float any = MaxOp::identity();  // NaN-propagating maximum
    for (int64_t c = 0; c < n && !failed; ++c) {
      if (tid == 0 && c >= 1 && c + kRingStages - 1 < n) {
        const int64_t ahead = c + kRingStages - 1;
        if (!ring_issue(g, values, ring, full, empty, ahead, loaded,
                        empty_parity, ahead < resident_from ? keep : once)) {
          failed = true;
          break;
        }
      }
      const int stage = (int)(c % kRingStages);
      const uint32_t bit = 1u << stage;
      if (!mbar_wait(&full[stage], (full_parity & bit) ? 1u : 0u)) {
        failed = true;
        break;
      }
      full_parity ^= bit;
      const float4 *slot =
          reinterpret_cast<const float4 *>(ring + stage * kRingChunk);
      // valid local slots of this chunk: [l0, l1)
      const int l0 = c == 0 ? shift : 0;
      const int64_t left = slots - c * kRingChunk;
      const int l1 = left < kRingChunk ? (int)left : kRingChunk;
      float4 q[kRingVectors];
#pragma unroll
      for (int k = 0; k < kRingVectors; ++k) {
        const int i = tid + k * kRingThreads;
        q[k] = slot[i];
        if (4 * i < l0 || 4 * i + 4 > l1) {
          if (4 * i + 0 < l0 || 4 * i + 0 >= l1) q[k].x = MaxOp::identity();
          if (4 * i + 1 < l0 || 4 * i + 1 >= l1) q[k].y = MaxOp::identity();
          if (4 * i + 2 < l0 || 4 * i + 2 >= l1) q[k].z = MaxOp::identity();
          if (4 * i + 3 < l0 || 4 * i + 3 >= l1) q[k].w = MaxOp::identity();
        }
      }
      if (c < resident_from) {  // will be loaded again for sweep B
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);
      }
      float lm = max4(q[0]);
#pragma unroll
      for (int k = 1; k < kRingVectors; ++k) lm = MaxOp::apply(lm, max4(q[k]));
      any = MaxOp::apply(any, lm);
      online_raise(s, lm);
      if (s.m > -CUDART_INF_F) {
        float d0 = 0.0f;
#pragma unroll
        for (int k = 0; k < kRingVectors; ++k) d0 += expsum4(q[k], s.m);
        s.d += d0;
      }
    }
    if (failed) atomicCAS(control + 2, 0u, 1u);
    // the segment maximum first (NaN-propagating), then the sums rescaled to it
    const float m = cta_reduce<MaxOp>(any, scratch);
    const float mine = s.d == 0.0f ? 0.0f : s.d * exp_neg(s.m - m);
    const float d = cta_reduce<SumOp>(mine, scratch);
    const float inv = 1.0f / d;

    // ---- sweep B ----
    for (int64_t c = n - 1; c >= 0 && !failed; --c) {
      if (tid == 0 && c <= n - 2 && c + 1 - kRingStages >= 0) {
        if (!ring_issue(g, values, ring, full, empty, c + 1 - kRingStages,
                        loaded, empty_parity, once)) {
          failed = true;
          break;
        }
      }
      const int stage = (int)(c % kRingStages);
      const uint32_t bit = 1u << stage;
      if (c < resident_from) {
        if (!mbar_wait(&full[stage], (full_parity & bit) ? 1u : 0u)) {
          failed = true;
          break;
        }
        full_parity ^= bit;
      }
      const float4 *slot =
          reinterpret_cast<const float4 *>(ring + stage * kRingChunk);
      const int l0 = c == 0 ? shift : 0;
      const int64_t left = slots - c * kRingChunk;
      const int l1 = left < kRingChunk ? (int)left : kRingChunk;
      float *o = out + (g.origin + c * kRingChunk);  // local slot 0
      float4 q[kRingVectors];
#pragma unroll
      for (int k = 0; k < kRingVectors; ++k) q[k] = slot[tid + k * kRingThreads];
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);
#pragma unroll
      for (int k = 0; k < kRingVectors; ++k) {
        const int i = tid + k * kRingThreads;
        const float4 r = normalise4(q[k], m, inv);
        if (same_phase && 4 * i >= l0 && 4 * i + 4 <= l1) {
          __stcs(reinterpret_cast<float4 *>(o) + i, r);
        } else {
          if (4 * i + 0 >= l0 && 4 * i + 0 < l1) __stcs(o + 4 * i + 0, r.x);
          if (4 * i + 1 >= l0 && 4 * i + 1 < l1) __stcs(o + 4 * i + 1, r.y);
          if (4 * i + 2 >= l0 && 4 * i + 2 < l1) __stcs(o + 4 * i + 2, r.z);
          if (4 * i + 3 >= l0 && 4 * i + 3 < l1) __stcs(o + 4 * i + 3, r.w);
        }
      }
    }
    if (failed) atomicCAS(control + 2, 0u, 1u);
  }
}

// Side streams so the bucket kernels of one call run concurrently: created once
// per device, joined back into the caller's stream before the call returns
// control to it.
namespace {
struct Fork {
  bool ready = false;
  cudaStream_t side[3];
  cudaEvent_t begin;
  cudaEvent_t done[3];
};
std::mutex g_fork_lock;
Fork g_fork[64];

cudaError_t fork_for(int device, Fork **fork) {
  std::lock_guard<std::mutex> guard(g_fork_lock);
  Fork &f = g_fork[device];
  if (!f.ready) {
    cudaError_t e =
        cudaEventCreateWithFlags(&f.begin, cudaEventDisableTiming);
    for (int i = 0; i < 3 && e == cudaSuccess; ++i) {
      e = cudaStreamCreateWithFlags(&f.side[i], cudaStreamNonBlocking);
      if (e == cudaSuccess)
        e = cudaEventCreateWithFlags(&f.done[i], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) return e;
    f.ready = true;
  }
  *fork = &f;
  return cudaSuccess;
}
}  // namespace

cudaError_t configure_softmax_kernels() {
  return cudaFuncSetAttribute(segsoftmax_ring_kernel,
                              cudaFuncAttributeMaxDynamicSharedMemorySize,
                              kRingBytes);
}

cudaError_t launch_segsoftmax_planned(const float *values,
                                      const int32_t *offsets, float *out,
                                      int32_t value_count,
                                      const DevicePlan &plan,
                                      cudaStream_t stream,
                                      const Probe *probe) {
  Fork *fork = nullptr;
  cudaError_t e = fork_for(plan.device, &fork);
  if (e != cudaSuccess) return e;
  probe_begin(probe, stream);
  e = cudaEventRecord(fork->begin, stream);
  if (e != cudaSuccess) return e;
  const int32_t *list = plan.softmax_segments;
  const int32_t n_stream = plan.softmax_count[3];
  if (n_stream > 0) {
#if SWG_SOFTMAX_RING
    int grid = plan.sm_count * kRingCtasPerSm;
    if (grid > n_stream) grid = n_stream;
    segsoftmax_ring_kernel<<<grid, kRingThreads, kRingBytes, stream>>>(
        values, offsets, out, list + plan.softmax_begin[3], n_stream,
        value_count, plan.control);
#else
    int grid = plan.sm_count * kLongCtasPerSm;
    if (grid > n_stream) grid = n_stream;
    segsoftmax_long_kernel<<<grid, kLongThreads, 0, stream>>>(
        values, offsets, out, list + plan.softmax_begin[3], n_stream);
#endif
  }
  for (int b = 2; b >= 0; --b) {
    const int32_t n = plan.softmax_count[b];
    if (n == 0) continue;
    cudaStream_t side = fork->side[b];
    e = cudaStreamWaitEvent(side, fork->begin, 0);
    if (e != cudaSuccess) return e;
    const int32_t *bucket = list + plan.softmax_begin[b];
    if (b == 2)
      segsoftmax_resident_kernel<512>
          <<<(unsigned)n, 512, 0, side>>>(values, offsets, out, bucket, n);
    else if (b == 1)
      segsoftmax_resident_kernel<128>
          <<<(unsigned)n, 128, 0, side>>>(values, offsets, out, bucket, n);
    else
      segsoftmax_resident_kernel<32>
          <<<(unsigned)((n + 7) / 8), 256, 0, side>>>(values, offsets, out,
                                                      bucket, n);
    e = cudaEventRecord(fork->done[b], side);
    if (e != cudaSuccess) return e;
    e = cudaStreamWaitEvent(stream, fork->done[b], 0);
    if (e != cudaSuccess) return e;
  }
  probe_end(probe, stream);
  return cudaGetLastError();
}

cudaError_t launch_segsoftmax_cta(const float *values, const int32_t *offsets,
                                  float *out, int32_t segment_count,
                                  int sm_count, cudaStream_t stream,
                                  const Probe *probe) {
  int64_t grid = segment_count;
  const int64_t cap = (int64_t)sm_count * 8 * 4;
  if (grid > cap) grid = cap;
  probe_begin(probe, stream);
  segsoftmax_cta_kernel<<<(unsigned)grid, 256, 0, stream>>>(
      values, offsets, out, segment_count);
  probe_end(probe, stream);
  return cudaGetLastError();
}

cudaError_t launch_segsoftmax_warp(const float *values, const int32_t *offsets,
                                   float *out, int32_t segment_count,
                                   int sm_count, cudaStream_t stream,
                                   const Probe *probe) {
  int64_t grid = ((int64_t)segment_count + 7) / 8;
  const int64_t cap = (int64_t)sm_count * 8 * 4;
  if (grid > cap) grid = cap;
  probe_begin(probe, stream);
  segsoftmax_warp_kernel<<<(unsigned)grid, 256, 0, stream>>>(
      values, offsets, out, segment_count);
  probe_end(probe, stream);
  return cudaGetLastError();
}

}  // namespace swg
