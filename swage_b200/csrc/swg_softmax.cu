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
