// Fixed-block fp32 vector add, out[i] = x[i] + y[i] for i < n.
//
// Replaces the kernel the reference generates in
// lib/Conversion/FixedBlockToGPU/FixedBlockToGPU.cpp:177-226 (one element per
// thread, scalar ld/st, grid = ceil(n / BLOCK)).  The logical BLOCK does not
// change any result bit (one fp32 add per element), so the physical mapping is
// chosen for HBM throughput instead: each thread moves kVecPerThread 128-bit
// vectors of x and of y, all loads issued before the first add, streaming
// cache hints on both sides (each byte is touched once).
//
// HBM-bound: 12 bytes per element (two loads, one store).
#include "swg_common.cuh"
#include "swg_launch.h"

namespace swg {

constexpr int kVaddThreads = 256;
constexpr int kVecPerThread = 4;  // 4 x 16 B of x and of y in flight per thread

// All three pointers share the same offset from a 16-byte boundary: `head`
// scalar elements, then float4 body, then a scalar tail.
__global__ void __launch_bounds__(kVaddThreads)
vadd_aligned_kernel(const float *__restrict__ x, const float *__restrict__ y,
                    float *__restrict__ out, int n, int head) {
  const int64_t nvec = (int64_t)(n - head) >> 2;
  const float4 *x4 = reinterpret_cast<const float4 *>(x + head);
  const float4 *y4 = reinterpret_cast<const float4 *>(y + head);
  float4 *o4 = reinterpret_cast<float4 *>(out + head);
  const int64_t base =
      (int64_t)blockIdx.x * (kVaddThreads * kVecPerThread) + threadIdx.x;

  if (base + (int64_t)(kVecPerThread - 1) * kVaddThreads < nvec) {
    float4 a[kVecPerThread], b[kVecPerThread];
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) a[k] = __ldcs(x4 + base + k * kVaddThreads);
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) b[k] = __ldcs(y4 + base + k * kVaddThreads);
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) {
      float4 r;
      r.x = __fadd_rn(a[k].x, b[k].x);
      r.y = __fadd_rn(a[k].y, b[k].y);
      r.z = __fadd_rn(a[k].z, b[k].z);
      r.w = __fadd_rn(a[k].w, b[k].w);
      __stcs(o4 + base + k * kVaddThreads, r);
    }
  } else {
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) {
      const int64_t i = base + k * kVaddThreads;
      if (i < nvec) {
        float4 a = __ldcs(x4 + i), b = __ldcs(y4 + i), r;
        r.x = __fadd_rn(a.x, b.x);
        r.y = __fadd_rn(a.y, b.y);
        r.z = __fadd_rn(a.z, b.z);
        r.w = __fadd_rn(a.w, b.w);
        __stcs(o4 + i, r);
      }
    }
  }
  // The ragged ends (at most 3 + 3 elements) ride on the first CTA.
  if (blockIdx.x == 0) {
    const int t = threadIdx.x;
    if (t < head) out[t] = __fadd_rn(x[t], y[t]);
    const int64_t tail = head + (nvec << 2);
    if (tail + t < n) out[tail + t] = __fadd_rn(x[tail + t], y[tail + t]);
  }
}

// 256-bit variant: all three pointers share the same offset from a 32-byte
// boundary.  sm_100 has 256-bit global loads and stores (ld/st.global.v8.f32):
// half the memory instructions of the 128-bit path for the same bytes in
// flight.
struct alignas(32) Float8 {
  float v[8];
};

__device__ __forceinline__ Float8 ld_stream8(const Float8 *p) {
  Float8 r;
  asm volatile(
      "ld.global.cs.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]),
        "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
      : "l"(p));
  return r;
}

__device__ __forceinline__ void st_stream8(Float8 *p, const Float8 &r) {
  asm volatile(
      "st.global.cs.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p),
      "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]), "f"(r.v[3]), "f"(r.v[4]),
      "f"(r.v[5]), "f"(r.v[6]), "f"(r.v[7])
      : "memory");
}

#ifndef SWG_VADD_V8_PER_THREAD
#define SWG_VADD_V8_PER_THREAD 1
#endif
constexpr int kVec8PerThread = SWG_VADD_V8_PER_THREAD;

__global__ void __launch_bounds__(kVaddThreads)
vadd_aligned32_kernel(const float *__restrict__ x, const float *__restrict__ y,
                      float *__restrict__ out, int n, int head) {
  const int64_t nvec = (int64_t)(n - head) >> 3;
  const Float8 *x8 = reinterpret_cast<const Float8 *>(x + head);
  const Float8 *y8 = reinterpret_cast<const Float8 *>(y + head);
  Float8 *o8 = reinterpret_cast<Float8 *>(out + head);
  const int64_t base =
      (int64_t)blockIdx.x * (kVaddThreads * kVec8PerThread) + threadIdx.x;
  Float8 a[kVec8PerThread], b[kVec8PerThread];
  if (base + (int64_t)(kVec8PerThread - 1) * kVaddThreads < nvec) {
#pragma unroll
    for (int k = 0; k < kVec8PerThread; ++k)
      a[k] = ld_stream8(x8 + base + k * kVaddThreads);
#pragma unroll
    for (int k = 0; k < kVec8PerThread; ++k)
      b[k] = ld_stream8(y8 + base + k * kVaddThreads);
#pragma unroll
    for (int k = 0; k < kVec8PerThread; ++k) {
#pragma unroll
      for (int e = 0; e < 8; ++e) a[k].v[e] = __fadd_rn(a[k].v[e], b[k].v[e]);
      st_stream8(o8 + base + k * kVaddThreads, a[k]);
    }
  } else {
#pragma unroll
    for (int k = 0; k < kVec8PerThread; ++k) {
      const int64_t i = base + k * kVaddThreads;
      if (i < nvec) {
        Float8 p = ld_stream8(x8 + i);
        const Float8 q = ld_stream8(y8 + i);
#pragma unroll
        for (int e = 0; e < 8; ++e) p.v[e] = __fadd_rn(p.v[e], q.v[e]);
        st_stream8(o8 + i, p);
      }
    }
  }
  // The ragged ends (at most 7 + 7 elements) ride on the first CTA.
  if (blockIdx.x == 0) {
    const int t = threadIdx.x;
    if (t < head) out[t] = __fadd_rn(x[t], y[t]);
    const int64_t tail = head + (nvec << 3);
    if (tail + t < n) out[tail + t] = __fadd_rn(x[tail + t], y[tail + t]);
  }
}

// Pointers disagree about their 16-byte phase: coalesced scalar accesses (the
// same bytes per sector, just more instructions).
__global__ void __launch_bounds__(kVaddThreads)
vadd_scalar_kernel(const float *__restrict__ x, const float *__restrict__ y,
                   float *__restrict__ out, int n) {
  const int64_t base =
      (int64_t)blockIdx.x * (kVaddThreads * 8) + threadIdx.x;
  float a[8], b[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int64_t i = base + k * kVaddThreads;
    a[k] = i < n ? __ldcs(x + i) : 0.0f;
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int64_t i = base + k * kVaddThreads;
    b[k] = i < n ? __ldcs(y + i) : 0.0f;
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int64_t i = base + k * kVaddThreads;
    if (i < n) __stcs(out + i, __fadd_rn(a[k], b[k]));
  }
}

cudaError_t launch_vadd(const float *x, const float *y, float *out, int32_t n,
                        cudaStream_t stream, const Probe *probe) {
  const unsigned px = (unsigned)((uintptr_t)x & 15u);
  const unsigned py = (unsigned)((uintptr_t)y & 15u);
  const unsigned po = (unsigned)((uintptr_t)out & 15u);
  probe_begin(probe, stream);
  const unsigned qx = (unsigned)((uintptr_t)x & 31u);
  const unsigned qy = (unsigned)((uintptr_t)y & 31u);
  const unsigned qo = (unsigned)((uintptr_t)out & 31u);
  if (qx == qy && qy == qo && (qx & 3u) == 0) {
    int head = (int)(((32u - qx) & 31u) >> 2);
    if (head > n) head = n;
    const int64_t nvec = (int64_t)(n - head) >> 3;
    const int64_t per_cta = (int64_t)kVaddThreads * kVec8PerThread;
    int64_t grid = (nvec + per_cta - 1) / per_cta;
    if (grid < 1) grid = 1;
    vadd_aligned32_kernel<<<(unsigned)grid, kVaddThreads, 0, stream>>>(
        x, y, out, n, head);
  } else if (px == py && py == po && (px & 3u) == 0) {
    int head = (int)(((16u - px) & 15u) >> 2);
    if (head > n) head = n;
    const int64_t nvec = (int64_t)(n - head) >> 2;
    const int64_t per_cta = (int64_t)kVaddThreads * kVecPerThread;
    int64_t grid = (nvec + per_cta - 1) / per_cta;
    if (grid < 1) grid = 1;
    vadd_aligned_kernel<<<(unsigned)grid, kVaddThreads, 0, stream>>>(
        x, y, out, n, head);
  } else {
    const int64_t per_cta = (int64_t)kVaddThreads * 8;
    const int64_t grid = ((int64_t)n + per_cta - 1) / per_cta;
    vadd_scalar_kernel<<<(unsigned)grid, kVaddThreads, 0, stream>>>(x, y, out,
                                                                    n);
  }
  probe_end(probe, stream);
  return cudaGetLastError();
}

}  // namespace swg
