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

// Resident buckets: a segment of at most kThreads * kRows values is held in
// the registers of kThreads threads (an eighth of a warp, a warp, or a CTA of
// 128 threads): every value is read from HBM exactly once and written exactly
// once, with coalesced 4-byte accesses, so no alignment case exists.  Groups
// narrower than a CTA share a 256-thread CTA.
template <int kThreads, int kRows>
__global__ void __launch_bounds__(kThreads <= 32 ? 256 : kThreads)
segsoftmax_resident_kernel(const float *__restrict__ values,
                           const int32_t *__restrict__ offsets,
                           float *__restrict__ out,
                           const int32_t *__restrict__ segments,
                           int32_t count) {
  __shared__ float scratch[32];
  constexpr bool kGroup = kThreads <= 32;
  const int t = kGroup ? (int)(threadIdx.x % kThreads) : (int)threadIdx.x;
  // Groups narrower than a CTA take one segment each; a CTA-wide group walks
  // the list with the grid's stride (the launcher sizes the grid to what is
  // resident at once), and fetches the bounds of its next segment while the
  // values of the current one are in flight: neither a CTA launch nor the two
  // dependent index loads sit between two segments of a CTA.
  const int64_t stride = kGroup ? (int64_t)count : (int64_t)gridDim.x;
  int64_t which =
      kGroup ? ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / kThreads
             : (int64_t)blockIdx.x;
  // a group past the end of the list keeps in step with the rest of its warp
  int64_t begin = 0;
  int length = 0;
  if (which < count) {
    const int32_t seg = __ldg(segments + which);
    begin = __ldg(offsets + seg);
    length = (int)(__ldg(offsets + seg + 1) - begin);
  }
  while (true) {
    const float *p = values + begin + t;
    float x[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r)
      x[r] = (r * kThreads + t < length) ? __ldcs(p + r * kThreads)
                                         : MaxOp::identity();
    const int64_t after = which + stride;
    int64_t next_begin = 0;
    int next_length = 0;
    if (!kGroup && after < count) {
      const int32_t seg = __ldg(segments + after);
      next_begin = __ldg(offsets + seg);
      next_length = (int)(__ldg(offsets + seg + 1) - next_begin);
    }
    float m = x[0];
#pragma unroll
    for (int r = 1; r < kRows; ++r) m = MaxOp::apply(m, x[r]);
    m = kGroup ? group_reduce<MaxOp>(m, kThreads)
               : cta_reduce<MaxOp>(m, scratch);
    float d = 0.0f;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      // padding slots are masked: exp(-inf - m) is 0 only for an ordered m
      const float e = (r * kThreads + t < length) ? exp_neg(x[r] - m) : 0.0f;
      x[r] = e;
      d += e;
    }
    d = kGroup ? group_reduce<SumOp>(d, kThreads)
               : cta_reduce<SumOp>(d, scratch);
    const float inv = 1.0f / d;
    float *o = out + begin + t;
#pragma unroll
    for (int r = 0; r < kRows; ++r)
      if (r * kThreads + t < length) __stcs(o + r * kThreads, x[r] * inv);
    if (kGroup || after >= count) break;
    which = after;
    begin = next_begin;
    length = next_length;
  }
}

// Pieces of the streamed (two-sweep) schedule.
struct MaxSum {
  float m, d;
};

__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t policy;
  asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
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

// Ring kernel: one CTA per segment, two sweeps.  The segment is cut into
// chunks of kRingChunk values dealt round-robin to the CTA's warps, and every
// warp streams its chunks through a private ring of kStages shared-memory
// stages filled by bulk async copies that its lane 0 issues:
//
//   sweep A  its chunks in ascending order: running (maximum, sum of exp) per
//            lane; a stage is refilled as soon as the warp has read it;
//   sweep B  its chunks in descending order: normalise and store.
//
// Sweep B walks backwards, so the last kStages chunks a warp saw in sweep A
// are still in its ring and are not loaded again: a segment of up to
// warps * kStages chunks is read from HBM once and never again, a longer one
// re-reads all but that tail, most recent lines first, which L2 serves (sweep
// A loads of chunks that will come back carry an evict-last policy,
// everything else evict-first).  A stage has a single reader -- the warp that
// owns it -- so handing it back to the copy engine needs no barrier, only a
// warp vote that depends on the loaded values; each stage has one mbarrier
// counting the copy's bytes.
//
// The stages that sweep B empties for good are refilled at once with the
// first chunks of the CTA's next segment, so the copy engine never idles
// between segments.  For the order in which sweep B frees stages (last chunk
// first) to be the order in which the next sweep A wants them (first chunk
// first), the chunk -> stage map runs upwards on even segments and downwards
// on odd ones.
//
// A chunk is a run of whole 16-byte lines of `values` counted from the line
// that holds the segment's first value, so every copy is aligned whatever
// the offsets are; the up-to-three values that share a line with the array's
// ends are fetched by plain loads.
//
// All waits are bounded; a wait that gives up raises the plan's timeout flag
// and the CTA walks to the end without touching the ring.
constexpr int kRingChunk = 512;
constexpr int kRingVectors = kRingChunk / 128;  // 128-bit loads per lane per chunk

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
  int64_t line_end;    // index past the line holding the segment's last value
  int64_t slots;       // valid slots: [shift, slots)
  int chunks;          // chunks of the segment (0: no such segment)
  int shift;           // begin - origin
};

// [begin, end) of the j-th segment of the list; {0, 0} past its end.
__device__ __forceinline__ int2
ring_bounds(const int32_t *__restrict__ offsets,
            const int32_t *__restrict__ segments, int64_t j, int32_t count) {
  if (j >= count) return make_int2(0, 0);
  const int32_t seg = __ldg(segments + j);
  return make_int2(__ldg(offsets + seg), __ldg(offsets + seg + 1));
}

__device__ __forceinline__ RingSegment ring_segment(const int2 bounds,
                                                    int mis) {
  RingSegment g;
  g.begin = bounds.x;
  g.end = bounds.y;
  g.shift = (int)((g.begin + mis) & 3);
  g.origin = g.begin - g.shift;
  g.line_end = g.end + ((4 - ((g.end + mis) & 3)) & 3);
  g.slots = (int64_t)g.shift + (g.end - g.begin);
  g.chunks =
      bounds.y > bounds.x ? (int)((g.slots + kRingChunk - 1) / kRingChunk) : 0;
  return g;
}

// One lane: starts the copy of the segment's chunk `c` into `slot`.  The
// caller has made sure that nobody reads the slot any more.
__device__ __forceinline__ void ring_issue(const RingSegment &g,
                                           const float *__restrict__ values,
                                           int64_t last_line, float *slot,
                                           uint64_t *full, int c,
                                           uint64_t policy) {
  const int64_t g0 = g.origin + (int64_t)c * kRingChunk;
  // the slot has just been read through the generic proxy; the copy writes it
  // through the async proxy
  fence_proxy_async();
  if (c > 0 && c < g.chunks - 1) {  // whole lines well inside the array
    mbar_arrive_expect_tx(full, kRingChunk * 4);
    bulk_g2s_hint(slot, values + g0, kRingChunk * 4, full, policy);
    return;
  }
  int64_t g1 = g0 + kRingChunk;
  if (g1 > g.line_end) g1 = g.line_end;
  int64_t lo = g0 < 0 ? g0 + 4 : g0;
  int64_t hi = g1 > last_line ? last_line : g1;
  if (hi < lo) hi = lo;
  const int64_t vb = g.begin > g0 ? g.begin : g0;
  const int64_t ve = g.end < g1 ? g.end : g1;
  for (int64_t i = vb; i < ve && i < lo; ++i) slot[i - g0] = values[i];
  for (int64_t i = hi > vb ? hi : vb; i < ve; ++i) slot[i - g0] = values[i];
  const uint32_t bytes = (uint32_t)(hi - lo) * 4u;
  mbar_arrive_expect_tx(full, bytes);
  if (bytes) bulk_g2s_hint(slot + (lo - g0), values + lo, bytes, full, policy);
}

// Returns once every lane of the warp HOLDS what it loaded from a stage.  A
// bulk copy into the stage may only be started after this: __syncwarp alone
// orders the issue of the loads, not their completion, and a copy served by
// L2 can land before a shared-memory load that is still queued behind the
// SM's global stores.  The vote consumes one word of every 128-bit load, so
// it cannot issue before the loads have returned.
__device__ __forceinline__ void ring_loads_landed(
    const float4 (&q)[kRingVectors]) {
  uint32_t word = 0;
#pragma unroll
  for (int v = 0; v < kRingVectors; ++v) word |= __float_as_uint(q[v].w);
  const unsigned seen = __ballot_sync(kFullMask, word != 0x7fedcba9u);
  asm volatile("" ::"r"(seen) : "memory");
}

// (The shape with one CTA per SM is compiled for 640 threads per block though
// it runs 512: that caps it at 96 registers, at no cost in speed, and leaves
// room on every SM for CTAs of the short classes' kernels to run beside it.)
template <int kWarps, int kStages, int kCtasPerSm>
__global__ void __launch_bounds__(kCtasPerSm == 1 ? kWarps * 40 : kWarps * 32,
                                  kCtasPerSm)
segsoftmax_ring_kernel(const float *__restrict__ values,
                       const int32_t *__restrict__ offsets,
                       float *__restrict__ out,
                       const int32_t *__restrict__ segments, int32_t count,
                       int32_t value_count, uint32_t *__restrict__ control,
                       uint32_t *__restrict__ ticket) {
  static_assert(kWarps <= 32 && kStages >= 1 && kStages <= 16, "ring shape");
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full_all[kWarps * kStages];
  __shared__ float scratch[32];
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  float *ring = reinterpret_cast<float *>(smem) + warp * kStages * kRingChunk;
  uint64_t *full = full_all + warp * kStages;
  if (lane == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();
  const uint64_t keep = policy_evict_last();
  const uint64_t once = policy_evict_first();
  const int mis = (int)(((uintptr_t)values >> 2) & 3);
  const int64_t last_line = (int64_t)value_count - ((value_count + mis) & 3);
  const bool same_phase =
      (int)(((uintptr_t)out >> 2) & 3) == mis;  // lines of out = lines of values
  uint32_t parity = 0;  // one bit per stage of this warp's ring
  bool failed = false;
  // this warp's chunks of a segment: warp, warp + kWarps, ...
  auto share = [&](const RingSegment &r) {
    return r.chunks > warp ? (r.chunks - warp + kWarps - 1) / kWarps : 0;
  };

  // Segments are handed out in list order to whichever CTA asks next (a
  // ticket counter per length class, zeroed by the launcher): the CTAs of a
  // class then work side by side on neighbouring segments whatever their
  // pace, and none is left with a long tail.  Tickets are drawn two segments
  // ahead of use -- thread 0 starts the atomic at the top of a segment and
  // publishes it through shared memory across the barriers of that segment's
  // reduction -- so neither the atomic nor the bounds of the next segment,
  // fetched one segment ahead, are ever waited for.
  __shared__ int ticket_box;
  auto draw = [&]() -> int64_t {
    if (tid == 0) ticket_box = (int)atomicAdd(ticket, 1u);
    __syncthreads();
    const int64_t drawn = ticket_box;
    __syncthreads();
    return drawn;
  };
  int64_t j = draw();
  int64_t j_next = draw();
  RingSegment g = ring_segment(ring_bounds(offsets, segments, j, count), mis);
  int mine = share(g);
  if (lane == 0)
    for (int k = 0; k < mine && k < kStages; ++k)
      ring_issue(g, values, last_line, ring + k * kRingChunk, &full[k],
                 k * kWarps + warp, k + kStages < mine ? keep : once);

  bool down = false;  // direction of the chunk -> stage map
  for (; j < count; down = !down) {
    // the next segment's bounds are fetched now and used after sweep A
    unsigned drawn = 0;
    if (tid == 0) drawn = atomicAdd(ticket, 1u);  // consumed after sweep A
    const int2 next_bounds = ring_bounds(offsets, segments, j_next, count);
    const int resident_from = mine > kStages ? mine - kStages : 0;
    auto stage_of = [&](int k, bool reversed) {
      return reversed ? kStages - 1 - k % kStages : k % kStages;
    };

    // ---- sweep A ----
    MaxSum s{-CUDART_INF_F, 0.0f};
    float any = MaxOp::identity();  // NaN-propagating maximum
    for (int k = 0; k < mine && !failed; ++k) {
      const int stage = stage_of(k, down);
      const uint32_t bit = 1u << stage;
      const bool ok = mbar_wait(&full[stage], (parity & bit) ? 1u : 0u);
      if (__any_sync(kFullMask, !ok)) {
        failed = true;
        break;
      }
      parity ^= bit;
      float *slot = ring + stage * kRingChunk;
      const int c = k * kWarps + warp;
      // valid local slots of this chunk: [l0, l1)
      const int l0 = c == 0 ? g.shift : 0;
      const int64_t left = g.slots - (int64_t)c * kRingChunk;
      const int l1 = left < kRingChunk ? (int)left : kRingChunk;
      float4 q[kRingVectors];
#pragma unroll
      for (int v = 0; v < kRingVectors; ++v)
        q[v] = reinterpret_cast<const float4 *>(slot)[lane + v * 32];
      if (k < resident_from) {  // comes back for sweep B: refill the stage now
        ring_loads_landed(q);
        if (lane == 0)
          ring_issue(g, values, last_line, slot, &full[stage],
                     (k + kStages) * kWarps + warp,
                     k + kStages < resident_from ? keep : once);
      }
      if (l0 > 0 || l1 < kRingChunk) {
#pragma unroll
        for (int v = 0; v < kRingVectors; ++v) {
          const int i = 4 * (lane + v * 32);
          if (i + 0 < l0 || i + 0 >= l1) q[v].x = MaxOp::identity();
          if (i + 1 < l0 || i + 1 >= l1) q[v].y = MaxOp::identity();
          if (i + 2 < l0 || i + 2 >= l1) q[v].z = MaxOp::identity();
          if (i + 3 < l0 || i + 3 >= l1) q[v].w = MaxOp::identity();
        }
      }
      float lm = max4(q[0]);
#pragma unroll
      for (int v = 1; v < kRingVectors; ++v) lm = MaxOp::apply(lm, max4(q[v]));
      any = MaxOp::apply(any, lm);
      online_raise(s, lm);
      if (s.m > -CUDART_INF_F) {
        float d0 = 0.0f;
#pragma unroll
        for (int v = 0; v < kRingVectors; ++v) d0 += expsum4(q[v], s.m);
        s.d += d0;
      }
    }
    if (failed) atomicCAS(control + 2, 0u, 1u);
    if (tid == 0) ticket_box = (int)drawn;
    // the segment maximum first (NaN-propagating), then the sums rescaled to it
    const float m = cta_reduce<MaxOp>(any, scratch);
    const int64_t j_after = ticket_box;  // written before the barriers above
    const float part = s.d == 0.0f ? 0.0f : s.d * exp_neg(s.m - m);
    const float d = cta_reduce<SumOp>(part, scratch);
    const float inv = 1.0f / d;

    // ---- the CTA's next segment: its first chunks go into the stages this
    // segment did not use, then into each stage sweep B is done with
    const RingSegment next = ring_segment(next_bounds, mis);
    const int next_mine = share(next);
    const int used = mine < kStages ? mine : kStages;
    __syncwarp();
    if (lane == 0 && !failed)
      for (int k = 0; k < kStages - used && k < next_mine; ++k) {
        const int stage = stage_of(k, !down);
        ring_issue(next, values, last_line, ring + stage * kRingChunk,
                   &full[stage], k * kWarps + warp,
                   k + kStages < next_mine ? keep : once);
      }

    // ---- sweep B ----
    for (int k = mine - 1; k >= 0 && !failed; --k) {
      const int stage = stage_of(k, down);
      const uint32_t bit = 1u << stage;
      if (k < resident_from) {  // loaded again
        const bool ok = mbar_wait(&full[stage], (parity & bit) ? 1u : 0u);
        if (__any_sync(kFullMask, !ok)) {
          failed = true;
          break;
        }
        parity ^= bit;
      }
      float *slot = ring + stage * kRingChunk;
      const int c = k * kWarps + warp;
      const int l0 = c == 0 ? g.shift : 0;
      const int64_t left = g.slots - (int64_t)c * kRingChunk;
      const int l1 = left < kRingChunk ? (int)left : kRingChunk;
      float *o = out + (g.origin + (int64_t)c * kRingChunk);  // local slot 0
      float4 q[kRingVectors];
#pragma unroll
      for (int v = 0; v < kRingVectors; ++v)
        q[v] = reinterpret_cast<const float4 *>(slot)[lane + v * 32];
      ring_loads_landed(q);
      if (lane == 0) {
        if (k >= kStages) {
          ring_issue(g, values, last_line, slot, &full[stage],
                     (k - kStages) * kWarps + warp, once);
        } else {
          const int k_next = kStages - 1 - k;  // same stage, opposite map
          if (k_next < next_mine)
            ring_issue(next, values, last_line, slot, &full[stage],
                       k_next * kWarps + warp,
                       k_next + kStages < next_mine ? keep : once);
        }
      }
      if (same_phase && l0 == 0 && l1 == kRingChunk) {
#pragma unroll
        for (int v = 0; v < kRingVectors; ++v)
          __stcs(reinterpret_cast<float4 *>(o) + lane + v * 32,
                 normalise4(q[v], m, inv));
      } else {
#pragma unroll
        for (int v = 0; v < kRingVectors; ++v) {
          const int i = 4 * (lane + v * 32);
          const float4 r = normalise4(q[v], m, inv);
          if (same_phase && i >= l0 && i + 4 <= l1) {
            __stcs(reinterpret_cast<float4 *>(o + i), r);
          } else {
            if (i + 0 >= l0 && i + 0 < l1) __stcs(o + i + 0, r.x);
            if (i + 1 >= l0 && i + 1 < l1) __stcs(o + i + 1, r.y);
            if (i + 2 >= l0 && i + 2 < l1) __stcs(o + i + 2, r.z);
            if (i + 3 >= l0 && i + 3 < l1) __stcs(o + i + 3, r.w);
          }
        }
      }
    }
    if (failed) atomicCAS(control + 2, 0u, 1u);
    g = next;
    mine = next_mine;
    j = j_next;
    j_next = j_after;
  }
}

// Ring shapes (warps, stages per warp, CTAs per SM), one per length class:
// the smallest ring that still holds a whole segment of the class, so that as
// many CTAs as possible share an SM while every value is read from HBM once.
//   bucket 3  (2048, 4096]    2 warps x 4 stages, 12 CTAs/SM  16 KB each
//   bucket 4  (4096, 8192]    4 warps x 4 stages,  6 CTAs/SM  32 KB each
//   bucket 5  (8192, 16384]   8 warps x 4 stages,  3 CTAs/SM  64 KB each
//   bucket 6  (16384, 24576] 12 warps x 4 stages,  2 CTAs/SM  96 KB each
//   bucket 7  longer         16 warps x 7 stages,  1 CTA/SM  224 KB: whole
//             up to 57344 values, above that all but the last 57344 values of
//             a segment are read a second time (from L2 when they are still
//             there)
// (A one-warp ring for (512, 2048] measured slower than the 128-thread
// register kernel, which keeps that class.)
constexpr int kFirstRingBucket = 3;

template <int kWarps, int kStages, int kCtasPerSm>
static cudaError_t ring_launch(const float *values, const int32_t *offsets,
                               float *out, const int32_t *segments,
                               int32_t count, int32_t value_count,
                               const DevicePlan &plan, cudaStream_t stream,
                               uint32_t *ticket, bool configure) {
  constexpr int kBytes = kWarps * kStages * kRingChunk * 4;
  static_assert((kBytes + 1024 + 8 * kWarps * kStages + 128) * kCtasPerSm <=
                    228 * 1024,
                "rings exceed shared memory");
  if (configure)
    return cudaFuncSetAttribute(
        segsoftmax_ring_kernel<kWarps, kStages, kCtasPerSm>,
        cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes);
  int grid = plan.sm_count * kCtasPerSm;
  if (grid > count) grid = count;
  segsoftmax_ring_kernel<kWarps, kStages, kCtasPerSm>
      <<<grid, kWarps * 32, kBytes, stream>>>(values, offsets, out, segments,
                                              count, value_count, plan.control,
                                              ticket);
  return cudaGetLastError();
}

// Side streams so the bucket kernels of one call run concurrently: created once
// per device, joined back into the caller's stream before the call returns
// control to it.
namespace {
struct Fork {
  bool ready = false;
  // held over the whole record / wait / launch sequence of one call: the
  // events are shared by every call on the device, so two host threads must
  // not interleave their sequences
  std::mutex sequence;
  cudaStream_t side[kSoftmaxBuckets - 1];
  cudaEvent_t begin;
  cudaEvent_t done[kSoftmaxBuckets - 1];
};
std::mutex g_fork_lock;
Fork g_fork[64];

cudaError_t fork_for(int device, Fork **fork) {
  std::lock_guard<std::mutex> guard(g_fork_lock);
  Fork &f = g_fork[device];
  if (!f.ready) {
    cudaError_t e =
        cudaEventCreateWithFlags(&f.begin, cudaEventDisableTiming);
    for (int i = 0; i < kSoftmaxBuckets - 1 && e == cudaSuccess; ++i) {
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

template <bool kConfigure>
static cudaError_t ring_bucket(int bucket, const float *values,
                               const int32_t *offsets, float *out,
                               const int32_t *segments, int32_t count,
                               int32_t value_count, const DevicePlan &plan,
                               cudaStream_t stream) {
  // one ticket counter per class, behind the plan's four control words
  uint32_t *ticket = plan.control ? plan.control + kTicketBase + bucket : nullptr;
  switch (bucket) {
    case 3:
      return ring_launch<2, 4, 12>(values, offsets, out, segments, count,
                                   value_count, plan, stream, ticket,
                                   kConfigure);
    case 4:
      return ring_launch<4, 4, 6>(values, offsets, out, segments, count,
                                  value_count, plan, stream, ticket,
                                   kConfigure);
    case 5:
      return ring_launch<8, 4, 3>(values, offsets, out, segments, count,
                                  value_count, plan, stream, ticket,
                                   kConfigure);
    case 6:
      return ring_launch<SWG_SOFTMAX_LIMIT6 / 2048, 4, 2>(
          values, offsets, out, segments, count, value_count, plan, stream,
          ticket, kConfigure);
    default:
      return ring_launch<16, 7, 1>(values, offsets, out, segments, count,
                                   value_count, plan, stream, ticket,
                                   kConfigure);
  }
}

cudaError_t configure_softmax_kernels() {
  DevicePlan none;
  for (int bucket = kFirstRingBucket; bucket < kSoftmaxBuckets; ++bucket) {
    cudaError_t e = ring_bucket<true>(bucket, nullptr, nullptr, nullptr,
                                      nullptr, 0, 0, none, nullptr);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// The launch sequence of one planned call: ticket counters cleared, the
// longest class on the caller's stream, every other class on its side stream
// behind `begin`, each joined back through its `done` event.
static cudaError_t launch_buckets(const float *values, const int32_t *offsets,
                                  float *out, int32_t value_count,
                                  const DevicePlan &plan, cudaStream_t stream,
                                  Fork *fork) {
  cudaError_t e;
  e = cudaMemsetAsync(plan.control + kTicketBase, 0,
                      kSoftmaxBuckets * sizeof(uint32_t), stream);
  if (e != cudaSuccess) return e;
  e = cudaEventRecord(fork->begin, stream);
  if (e != cudaSuccess) return e;
  const int32_t *list = plan.softmax_segments;
  // the longest class on the caller's stream; beside it first the three
  // register kernels of the short classes (their CTAs fit next to the long
  // class's and fill its bubbles), then the other rings, longest first
  constexpr int kLast = kSoftmaxBuckets - 1;
  if (plan.softmax_count[kLast] > 0) {
    e = ring_bucket<false>(kLast, values, offsets, out,
                           list + plan.softmax_begin[kLast],
                           plan.softmax_count[kLast], value_count, plan,
                           stream);
    if (e != cudaSuccess) return e;
  }
  static const int kOrder[kLast] = {2, 1, 0, 6, 5, 4, 3};
  for (int at = 0; at < kLast; ++at) {
    const int b = kOrder[at];
    const int32_t n = plan.softmax_count[b];
    if (n == 0) continue;
    cudaStream_t side = fork->side[b];
    e = cudaStreamWaitEvent(side, fork->begin, 0);
    if (e != cudaSuccess) return e;
    const int32_t *bucket = list + plan.softmax_begin[b];
    if (b >= kFirstRingBucket) {
      e = ring_bucket<false>(b, values, offsets, out, bucket, n, value_count,
                             plan, side);
      if (e != cudaSuccess) return e;
    } else if (b == 2) {
      // persistent over the class's list: what is resident at once
      // (registers allow twelve 128-thread CTAs per SM), never more CTAs
      // than segments
      const int resident = plan.sm_count * 12;
      segsoftmax_resident_kernel<128, 16>
          <<<(unsigned)(n < resident ? n : resident), 128, 0, side>>>(
              values, offsets, out, bucket, n);
    } else if (b == 1) {
      segsoftmax_resident_kernel<32, 16>
          <<<(unsigned)((n + 7) / 8), 256, 0, side>>>(values, offsets, out,
                                                      bucket, n);
    } else {
      segsoftmax_resident_kernel<8, 8>
          <<<(unsigned)((n + 31) / 32), 256, 0, side>>>(values, offsets, out,
                                                        bucket, n);
    }
    e = cudaEventRecord(fork->done[b], side);
    if (e != cudaSuccess) return e;
    e = cudaStreamWaitEvent(stream, fork->done[b], 0);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

cudaError_t launch_segsoftmax_planned(const float *values,
                                      const int32_t *offsets, float *out,
                                      int32_t value_count,
                                      const DevicePlan &plan,
                                      cudaStream_t stream,
                                      const Probe *probe) {
  static_assert(kSoftmaxBuckets == 8 && kSoftmaxLimit[0] == 8 * 8 &&
                    kSoftmaxLimit[1] == 32 * 16 && kSoftmaxLimit[2] == 128 * 16,
                "bucket limits are the capacities of the resident kernels");
  Fork *fork = nullptr;
  cudaError_t e = fork_for(plan.device, &fork);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> in_sequence(fork->sequence);
  probe_begin(probe, stream);
  e = launch_buckets(values, offsets, out, value_count, plan, stream, fork);
  probe_end(probe, stream);
  return e != cudaSuccess ? e : cudaGetLastError();
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
