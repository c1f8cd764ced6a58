// Shared device helpers for the sm_100a kernels: reduction operators with the
// reference's semantics, warp/CTA reductions with a fixed combine order, and
// thin wrappers over the PTX this library relies on (NaN-propagating max,
// mbarrier, bulk async copy).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "swage_b200.h"

namespace swg {

constexpr int kWarp = 32;
constexpr unsigned kFullMask = 0xffffffffu;

// ---------------------------------------------------------------------------
// Operators.  Sum: fp32 add from +0.0f.  Max: arith.maximumf of the reference
// (SegmentedReduction.cpp:173-175, 256-258): NaN if either side is NaN and
// -0.0 ordered below +0.0; identity -inf.  max.NaN.f32 has exactly these rules.
// ---------------------------------------------------------------------------
struct SumOp {
  using Acc = float;
  static __device__ __forceinline__ float identity() { return 0.0f; }
  static __device__ __forceinline__ float apply(float a, float b) {
    return __fadd_rn(a, b);  // never contracted into an fma
  }
};

struct MaxOp {
  using Acc = float;
  static __device__ __forceinline__ float identity() {
    return -CUDART_INF_F;
  }
  static __device__ __forceinline__ float apply(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
  }
};

// Min: arith.minimumf, the mirror image (NaN-propagating, -0 below +0,
// identity +inf).  The reference's dialect admits kind<min> (ADR-0008) but its
// lowering rejects it (SegmentedReduction.cpp:106-108).
struct MinOp {
  using Acc = float;
  static __device__ __forceinline__ float identity() { return CUDART_INF_F; }
  static __device__ __forceinline__ float apply(float a, float b) {
    float r;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
  }
};

// Integer segments (the dialect's element types include i32; the reference's
// lowering accepts f32 only, SegmentedReduction.cpp:106-119): two's-complement
// wrap-around sum from 0, signed max from INT32_MIN, signed min from INT32_MAX.
// Integer addition is associative, so every summation order gives the same
// bits as the sequential one.
struct ISumOp {
  using Acc = int32_t;
  static __device__ __forceinline__ int32_t identity() { return 0; }
  static __device__ __forceinline__ int32_t apply(int32_t a, int32_t b) {
    return (int32_t)((uint32_t)a + (uint32_t)b);
  }
};
struct IMaxOp {
  using Acc = int32_t;
  static __device__ __forceinline__ int32_t identity() { return INT32_MIN; }
  static __device__ __forceinline__ int32_t apply(int32_t a, int32_t b) {
    return a > b ? a : b;
  }
};
struct IMinOp {
  using Acc = int32_t;
  static __device__ __forceinline__ int32_t identity() { return INT32_MAX; }
  static __device__ __forceinline__ int32_t apply(int32_t a, int32_t b) {
    return a < b ? a : b;
  }
};

// Element types a tile may hold, and what they accumulate in: f16 / bf16
// values are widened to fp32 (exactly) and reduced in fp32.
template <class T>
struct Elem;
template <>
struct Elem<float> {
  using Acc = float;
  static __device__ __forceinline__ float get(float v) { return v; }
};
template <>
struct Elem<int32_t> {
  using Acc = int32_t;
  static __device__ __forceinline__ int32_t get(int32_t v) { return v; }
};
template <>
struct Elem<__half> {
  using Acc = float;
  static __device__ __forceinline__ float get(__half v) {
    return __half2float(v);
  }
};
template <>
struct Elem<__nv_bfloat16> {
  using Acc = float;
  static __device__ __forceinline__ float get(__nv_bfloat16 v) {
    return __bfloat162float(v);
  }
};

// ---------------------------------------------------------------------------
// Element maps: what is applied to a value (already widened to its
// accumulator type) before it enters the reduction -- the dialect's swage.map
// region in front of a swage.reduce (test/Dialect/Swage/roundtrip.mlir:43-52,
// softmax.mlir:17-24), which the reference's lowering rejects
// (SegmentedReduction.cpp:106-119).  NoMap is the identity region every
// reference kernel has and costs nothing.  ScalarMap is fn(scale * x + shift)
// with scale and shift captured at launch; the product and the sum are
// rounded separately (arith.mulf, arith.addf), the exponential is one
// multiply and one ex2.approx like the softmax kernels'.
// ---------------------------------------------------------------------------
struct NoMap {
  template <class A>
  __device__ __forceinline__ A operator()(A v) const {
    return v;
  }
};

struct ScalarMap {
  int32_t fn;  // SWG_MAP_*
  float scale, shift;
};

// ScalarMap with the function fixed at compile time: what the kernels' inner
// loops are instantiated for (see with_fixed_map), so that no loop carries a
// test of `fn`.
template <int kFn>
struct FixedMap {
  float scale, shift;
  __device__ __forceinline__ float operator()(float x) const {
    float y = __fadd_rn(__fmul_rn(x, scale), shift);
    if constexpr (kFn == SWG_MAP_ABS) {
      y = fabsf(y);
    } else if constexpr (kFn == SWG_MAP_SQUARE) {
      y = __fmul_rn(y, y);
    } else if constexpr (kFn == SWG_MAP_EXP) {
      float r;
      asm("ex2.approx.ftz.f32 %0, %1;"
          : "=f"(r)
          : "f"(__fmul_rn(y, 1.4426950408889634f)));
      y = r;
    }
    return y;
  }
};

// Calls f with the map to apply: NoMap as it is, a ScalarMap as the FixedMap
// of its function (one warp-uniform switch per call).
template <class F>
__device__ __forceinline__ void with_fixed_map(const NoMap &map, F &&f) {
  f(map);
}
template <class F>
__device__ __forceinline__ void with_fixed_map(const ScalarMap &map, F &&f) {
  switch (map.fn) {
    case SWG_MAP_ABS:
      f(FixedMap<SWG_MAP_ABS>{map.scale, map.shift});
      break;
    case SWG_MAP_SQUARE:
      f(FixedMap<SWG_MAP_SQUARE>{map.scale, map.shift});
      break;
    case SWG_MAP_EXP:
      f(FixedMap<SWG_MAP_EXP>{map.scale, map.shift});
      break;
    default:
      f(FixedMap<SWG_MAP_IDENTITY>{map.scale, map.shift});
      break;
  }
}

// ---------------------------------------------------------------------------
// Where a segment's result goes.  NoPeers: out[seg], the caller's array.
// PeerOut: element offset + seg of EVERY GPU's copy of the full result array
// of a sharded reduction -- this GPU's own copy and its peers', mapped into
// this process -- written by the reducing warp itself with plain stores, so
// that the exchange of the results rides along with the reduction instead of
// following it as a collective or a copy kernel.  No multicast, no load from
// peer memory, nothing waits on another GPU.
// ---------------------------------------------------------------------------
constexpr int kMaxPeers = SWG_MAX_PEERS;

struct NoPeers {
  template <class A>
  __device__ __forceinline__ void store(A *out, int seg, A v) const {
    out[seg] = v;
  }
};

struct PeerOut {
  float *base[kMaxPeers];
  int32_t count;
  int64_t offset;
  __device__ __forceinline__ void store(float *, int seg, float v) const {
    for (int p = 0; p < count; ++p) base[p][offset + seg] = v;
  }
};

template <class Op>
__device__ __forceinline__ float fold4(float acc, float4 q) {
  return Op::apply(Op::apply(acc, Op::apply(q.x, q.y)), Op::apply(q.z, q.w));
}

// One 16-byte line of elements of type T folded into acc: four 32-bit
// elements as fold4 does, or eight 16-bit ones as two such groups.
template <class Op, class T, class M = NoMap>
__device__ __forceinline__ typename Op::Acc fold_line(typename Op::Acc acc,
                                                      uint4 raw,
                                                      const M &map = M{}) {
  using A = typename Op::Acc;
  if constexpr (sizeof(T) == 4) {
    T v[4];
    memcpy(v, &raw, 16);
    const A x = map(Elem<T>::get(v[0])), y = map(Elem<T>::get(v[1])),
            z = map(Elem<T>::get(v[2])), w = map(Elem<T>::get(v[3]));
    return Op::apply(Op::apply(acc, Op::apply(x, y)), Op::apply(z, w));
  } else {
    T v[8];
    memcpy(v, &raw, 16);
    A e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = map(Elem<T>::get(v[i]));
    const A lo = Op::apply(Op::apply(e[0], e[1]), Op::apply(e[2], e[3]));
    const A hi = Op::apply(Op::apply(e[4], e[5]), Op::apply(e[6], e[7]));
    return Op::apply(Op::apply(acc, lo), hi);
  }
}

// Butterfly over the 32 lanes; every lane ends with the same value and the
// combine order is fixed, so results do not depend on timing.
template <class Op>
__device__ __forceinline__ typename Op::Acc warp_reduce(typename Op::Acc v) {
#pragma unroll
  for (int delta = 16; delta > 0; delta >>= 1)
    v = Op::apply(v, __shfl_xor_sync(kFullMask, v, delta));
  return v;
}

// Reduce over a sub-group of `width` adjacent lanes (width a power of two).
template <class Op>
__device__ __forceinline__ typename Op::Acc group_reduce(typename Op::Acc v,
                                                         int width) {
  for (int delta = width >> 1; delta > 0; delta >>= 1)
    v = Op::apply(v, __shfl_xor_sync(kFullMask, v, delta));
  return v;
}

// CTA-wide reduce through `scratch` (>= 32 words of shared memory).  All
// threads of the CTA must call it; the value is returned to every thread.
template <class Op>
__device__ __forceinline__ typename Op::Acc cta_reduce(typename Op::Acc v,
                                                       float *scratch) {
  using A = typename Op::Acc;
  static_assert(sizeof(A) == 4, "accumulators are 32-bit");
  A *words = reinterpret_cast<A *>(scratch);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_reduce<Op>(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) words[warp] = v;
  __syncthreads();
  A r = lane < nwarps ? words[lane] : Op::identity();
  return warp_reduce<Op>(r);
}

// ---------------------------------------------------------------------------
// Global loads.  Values are read exactly once, so they bypass L1 and are
// marked evict-first in L2.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float4 ld_stream4(const float4 *p) {
  return __ldcs(p);
}
__device__ __forceinline__ float ld_stream(const float *p) { return __ldcs(p); }

// Elements before the first 16-byte boundary at or after p (0..3).
__device__ __forceinline__ int head_elems(const float *p) {
  return (int)(((16u - (unsigned)((uintptr_t)p & 15u)) & 15u) >> 2);
}

// One thread's share of reduce(v[begin, end)) when `nthreads` threads with
// ranks 0..nthreads-1 stride over the range: scalar head up to the first
// 16-byte boundary, float4 body with kInFlight independent 128-bit loads
// issued before any of them is used (four accumulators), scalar tail.
template <class Op, int kInFlight = 4>
__device__ __forceinline__ float strided_partial(const float *__restrict__ v,
                                                 int64_t begin, int64_t end,
                                                 int rank, int nthreads) {
  static_assert(kInFlight % 4 == 0, "loads in flight: a multiple of four");
  float acc[4] = {Op::identity(), Op::identity(), Op::identity(),
                  Op::identity()};
  const float *p = v + begin;
  const int len = (int)(end - begin);  // one segment: < 2^31
  if (len <= 0) return acc[0];
  int head = head_elems(p);
  if (head > len) head = len;
  if (rank < head) acc[0] = Op::apply(acc[0], ld_stream(p + rank));
  const float4 *body = reinterpret_cast<const float4 *>(p + head);
  const int nvec = (len - head) >> 2;
  int i = rank;
  for (; i < nvec; i += kInFlight * nthreads) {
    // (the loads of a last, partial batch are predicated off)
    float4 q[kInFlight];
#pragma unroll
    for (int k = 0; k < kInFlight; ++k)
      if (i + k * nthreads < nvec)
        q[k] = ld_stream4(body + i + k * nthreads);
#pragma unroll
    for (int k = 0; k < kInFlight; ++k)
      if (i + k * nthreads < nvec)
        acc[k & 3] = fold4<Op>(acc[k & 3], q[k]);
  }
  float r = Op::apply(Op::apply(acc[0], acc[1]), Op::apply(acc[2], acc[3]));
  const int tail = head + (nvec << 2);
  const int rem = len - tail;
  if (rank < rem) r = Op::apply(r, ld_stream(p + tail + rank));
  return r;
}

// Sum and maximum of the same range in one pass over it: every value is
// loaded once and folded into both accumulators.
struct SumMax {
  float sum, max;
};

template <int kInFlight>
__device__ __forceinline__ SumMax strided_sum_max(const float *__restrict__ v,
                                                  int64_t begin, int64_t end,
                                                  int rank, int nthreads) {
  static_assert(kInFlight % 4 == 0, "loads in flight: a multiple of four");
  float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  float m[4] = {MaxOp::identity(), MaxOp::identity(), MaxOp::identity(),
                MaxOp::identity()};
  const float *p = v + begin;
  const int len = (int)(end - begin);  // one segment: < 2^31
  if (len <= 0) return SumMax{s[0], m[0]};
  int head = head_elems(p);
  if (head > len) head = len;
  if (rank < head) {
    const float x = ld_stream(p + rank);
    s[0] = SumOp::apply(s[0], x);
    m[0] = MaxOp::apply(m[0], x);
  }
  const float4 *body = reinterpret_cast<const float4 *>(p + head);
  const int nvec = (len - head) >> 2;
  int i = rank;
  for (; i < nvec; i += kInFlight * nthreads) {
    float4 q[kInFlight];
#pragma unroll
    for (int k = 0; k < kInFlight; ++k)
      if (i + k * nthreads < nvec)
        q[k] = ld_stream4(body + i + k * nthreads);
#pragma unroll
    for (int k = 0; k < kInFlight; ++k)
      if (i + k * nthreads < nvec) {
        s[k & 3] = fold4<SumOp>(s[k & 3], q[k]);
        m[k & 3] = fold4<MaxOp>(m[k & 3], q[k]);
      }
  }
  SumMax r;
  r.sum = SumOp::apply(SumOp::apply(s[0], s[1]), SumOp::apply(s[2], s[3]));
  r.max = MaxOp::apply(MaxOp::apply(m[0], m[1]), MaxOp::apply(m[2], m[3]));
  const int tail = head + (nvec << 2);
  const int rem = len - tail;
  if (rank < rem) {
    const float x = ld_stream(p + tail + rank);
    r.sum = SumOp::apply(r.sum, x);
    r.max = MaxOp::apply(r.max, x);
  }
  return r;
}

// ---------------------------------------------------------------------------
// mbarrier + bulk async copy (TMA, untiled form).  Every wait is bounded: after
// kWaitLimitNs without success the caller gets `false` and is expected to raise the
// error flag and leave.
// ---------------------------------------------------------------------------
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // two seconds

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(count)
               : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar,
                                                      uint32_t bytes) {
  asm volatile(
      "mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
          smem_u32(bar)),
      "r"(bytes)
      : "memory");
}

// One probe.  The hardware parks the thread for a system-chosen time while
// the phase is incomplete.  (An explicit 20 us suspend-time hint and a
// __nanosleep between probes both measured no different: the waiting warps do
// not take issue slots from the working ones.)
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait; false = gave up after `limit_ns`.  The clock is only read
// once the first few probes have failed, so the common case costs one probe.
__device__ __forceinline__ bool mbar_wait_for(uint64_t *bar, uint32_t parity,
                                              uint64_t limit_ns) {
  for (int probe = 0; probe < 16; ++probe)
    if (mbar_try_wait(bar, parity)) return true;
  const uint64_t deadline = global_timer_ns() + limit_ns;
  for (;;) {
    for (int probe = 0; probe < 32; ++probe)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() > deadline) return false;
  }
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  return mbar_wait_for(bar, parity, kWaitLimitNs);
}

// Orders this thread's earlier generic-proxy accesses to shared memory (and
// those of other threads it has synchronised with) before the async-proxy
// writes of the bulk copies it issues next: the architected fence for handing
// a stage that has just been read back to the copy engine.
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Asks L2 to fetch [src, src + bytes) (16-byte aligned, a multiple of 16
// bytes); nothing is delivered to the SM.  L2 is the point of coherence for
// global memory, so a line prefetched before its last writer has finished
// still holds that writer's data when it is read later.
__device__ __forceinline__ void bulk_prefetch_l2(const void *src_gmem,
                                                 uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_gmem),
               "r"(bytes)
               : "memory");
}

// global -> shared bulk copy, completion counted in bytes on `bar`.  Both
// addresses 16-byte aligned, `bytes` a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem,
                                         uint32_t bytes, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// ---------------------------------------------------------------------------
// Error words of a plan's control block: control[2] = code (first one wins),
// control[3] = detail.  control[12..13] may hold the address of a host-visible
// copy {code, detail} (pinned memory), which the host can read without a CUDA
// call once the kernel has finished.
// ---------------------------------------------------------------------------
constexpr uint32_t kErrTimeout = 1u, kErrBadTask = 2u, kErrBadSegment = 3u;

__device__ __forceinline__ void report(uint32_t *control, uint32_t code,
                                       uint32_t detail) {
  if (atomicCAS(control + 2, 0u, code) != 0u) return;
  atomicExch(control + 3, detail);
  volatile uint32_t *host = reinterpret_cast<volatile uint32_t *>(
      *reinterpret_cast<unsigned long long *>(control + 12));
  if (host != nullptr) {
    host[1] = detail;
    __threadfence_system();
    host[0] = code;
    __threadfence_system();
  }
}

}  // namespace swg
