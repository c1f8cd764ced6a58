/*
 * CPU oracle for the segmented sum / max / softmax and fixed-block vector add
 * path.  TEST INFRASTRUCTURE ONLY: the shipped library never links, loads or
 * calls anything in this file; it exists so the CUDA kernels can be checked
 * against the reference's arithmetic and so a CPU baseline can be timed.
 *
 * Parity status: PINNED against the reference's own known answers
 *   - test/Conversion/SwageToCPU/segmented-sum-runner.mlir:37-53,67-68
 *       values [2,3,4,5], offsets [0,0,1,4,4]  ->  sum [0,2,12,0]
 *   - python/tests/mlir/test_segmented_runtime.py:151-181
 *       values [1,NaN,3,4,5], offsets [0,3,3,5] -> max [NaN,-inf,5]
 *   - python/tests/mlir/test_segmented_runtime.py:15-36,100-131
 *       eight length cases with values ((i % 17) - 8) / 4 (exactly
 *       representable, so every summation order gives the same bits)
 * The reference's executable CPU path (swage-opt | mlir-opt | mlir-runner,
 * python/swage/_segmented_qualification.py:288-329) needs the pinned LLVM/MLIR
 * llvmorg-22.1.8 toolchain, which is not part of the reference tree, so this
 * file restates the loop nest that path executes instead of running it.
 *
 * What is restated, line by line:
 *   lib/Conversion/SegmentedReduction/SegmentedReduction.cpp:131-183
 *   (buildSequentialReduction): for sid in [0, segment_count): start =
 *   offsets[sid], end = offsets[sid+1] (i32 widened to index), acc = identity
 *   (+0.0f for sum :157-158, -inf for max :159), for i in [start, end) step 1:
 *   acc = acc + v (arith.addf, one fp32 rounding) or acc = maximumf(acc, v)
 *   (NaN if either operand is NaN, -0 orders below +0), then out[sid] = acc.
 *
 * Build with -O2 -ffp-contract=off and without -ffast-math so the compiler
 * keeps the strict left-to-right fp32 order.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define SWG_ORACLE_SUM 0
#define SWG_ORACLE_MAX 1
/* kind<min> exists in the reference's dialect only (ADR-0008; its lowering
 * rejects it, SegmentedReduction.cpp:106-108): the mirror image of max --
 * arith.minimumf from +inf -- is restated here by symmetry; no reference test
 * pins it. */
#define SWG_ORACLE_MIN 2

/* arith.maximumf: NaN-propagating, -0.0 < +0.0.
 * SegmentedReduction.cpp:173-175 creates arith::MaximumFOp for kind == Max. */
static inline float oracle_maximumf(float a, float b) {
  if (isnan(a) || isnan(b)) return NAN;
  if (a > b) return a;
  if (b > a) return b;
  /* equal magnitudes: only +0 / -0 differ in bits; +0 wins */
  return signbit(a) ? b : a;
}

/* arith.minimumf: NaN-propagating, -0.0 < +0.0. */
static inline float oracle_minimumf(float a, float b) {
  if (isnan(a) || isnan(b)) return NAN;
  if (a < b) return a;
  if (b < a) return b;
  return signbit(a) ? a : b;
}

static inline float oracle_segment_f32(int kind, const float *values,
                                       int64_t start, int64_t end) {
  if (kind == SWG_ORACLE_SUM) {
    float acc = 0.0f; /* identity, SegmentedReduction.cpp:157-158 */
    for (int64_t i = start; i < end; ++i) acc = acc + values[i];
    return acc;
  }
  if (kind == SWG_ORACLE_MIN) {
    float acc = INFINITY;
    for (int64_t i = start; i < end; ++i) acc = oracle_minimumf(acc, values[i]);
    return acc;
  }
  float acc = -INFINITY; /* identity, SegmentedReduction.cpp:159 */
  for (int64_t i = start; i < end; ++i) acc = oracle_maximumf(acc, values[i]);
  return acc;
}

/* The reference's CPU path: one thread, segments in order.
 * threads <= 1 is the faithful single-thread form; threads > 1 runs the same
 * per-segment arithmetic with OpenMP over segments (identical bits because no
 * segment is ever split). Returns the number of threads actually used. */
int swg_oracle_segreduce_f32(int kind, const float *values,
                             const int32_t *offsets, float *out,
                             int64_t segment_count, int threads) {
  if (kind != SWG_ORACLE_SUM && kind != SWG_ORACLE_MAX &&
      kind != SWG_ORACLE_MIN)
    return -1;
  int used = 1;
#ifdef _OPENMP
  if (threads > 1) {
    used = threads;
#pragma omp parallel for schedule(dynamic, 64) num_threads(threads)
    for (int64_t sid = 0; sid < segment_count; ++sid)
      out[sid] = oracle_segment_f32(kind, values, (int64_t)offsets[sid],
                                    (int64_t)offsets[sid + 1]);
    return used;
  }
#else
  (void)threads;
#endif
  for (int64_t sid = 0; sid < segment_count; ++sid)
    out[sid] = oracle_segment_f32(kind, values, (int64_t)offsets[sid],
                                  (int64_t)offsets[sid + 1]);
  return used;
}

/* Integer segments (the dialect's kind<...> over i32 elements; the reference's
 * lowering accepts f32 only, SegmentedReduction.cpp:110-119, so this is the
 * sequential loop of :131-183 with the integer identities of ADR-0008 :34-39:
 * sum from 0 with two's-complement wrap-around, signed max from INT32_MIN,
 * signed min from INT32_MAX).  Unpinned: the reference holds no test for it. */
int swg_oracle_segreduce_i32(int kind, const int32_t *values,
                             const int32_t *offsets, int32_t *out,
                             int64_t segment_count) {
  if (kind != SWG_ORACLE_SUM && kind != SWG_ORACLE_MAX &&
      kind != SWG_ORACLE_MIN)
    return -1;
  for (int64_t sid = 0; sid < segment_count; ++sid) {
    uint32_t sum = 0;
    int32_t top = INT32_MIN, bottom = INT32_MAX;
    for (int64_t i = offsets[sid]; i < offsets[sid + 1]; ++i) {
      sum += (uint32_t)values[i];
      if (values[i] > top) top = values[i];
      if (values[i] < bottom) bottom = values[i];
    }
    out[sid] = kind == SWG_ORACLE_SUM   ? (int32_t)sum
               : kind == SWG_ORACLE_MAX ? top
                                        : bottom;
  }
  return 1;
}

/* Element map in front of a reduction: out[i] = fn(scale * x[i] + shift) in
 * fp32, product and sum rounded separately (arith.mulf, arith.addf; this file
 * is built with -ffp-contract=off), fn = 0 identity, 1 |y|, 2 y * y,
 * 3 exp(y) evaluated in double and rounded once.  The form of a swage.map
 * region (test/Dialect/Swage/roundtrip.mlir:43-52, softmax.mlir:17-24).
 * Unpinned: the reference lowers no map in front of a reduce
 * (SegmentedReduction.cpp:106-119), so it holds no result for one.  The
 * mapped values are then reduced by the pinned functions of this file. */
int swg_oracle_map_f32(int fn, float scale, float shift, const float *values,
                       float *out, int64_t count) {
  if (fn < 0 || fn > 3) return -1;
  for (int64_t i = 0; i < count; ++i) {
    const float product = values[i] * scale;
    float y = product + shift;
    if (fn == 1) y = fabsf(y);
    if (fn == 2) y = y * y;
    if (fn == 3) y = (float)exp((double)y);
    out[i] = y;
  }
  return 1;
}

/* fp64 accumulation of the same sum: the quantity the fp32 tolerance
 * |err| <= 1e-5 * sqrt(len) * max|x| is stated against. */
int swg_oracle_segsum_f64(const float *values, const int32_t *offsets,
                          double *out, int64_t segment_count, int threads) {
  int used = threads > 1 ? threads : 1;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 64) num_threads(used)
#else
  used = 1;
#endif
  for (int64_t sid = 0; sid < segment_count; ++sid) {
    double acc = 0.0;
    for (int64_t i = offsets[sid]; i < offsets[sid + 1]; ++i)
      acc += (double)values[i];
    out[sid] = acc;
  }
  return used;
}

/* max|x| per segment (0 for an empty one): scale of the sum tolerance. */
int swg_oracle_segabsmax_f64(const float *values, const int32_t *offsets,
                             double *out, int64_t segment_count, int threads) {
  int used = threads > 1 ? threads : 1;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 64) num_threads(used)
#else
  used = 1;
#endif
  for (int64_t sid = 0; sid < segment_count; ++sid) {
    double acc = 0.0;
    for (int64_t i = offsets[sid]; i < offsets[sid + 1]; ++i) {
      double a = fabs((double)values[i]);
      if (a > acc) acc = a;
    }
    out[sid] = acc;
  }
  return used;
}

/* Segmented softmax composed exactly as the reference's semantic form
 * (test/Dialect/Swage/softmax.mlir:13-31): m = reduce max, d = reduce sum of
 * exp(x - m), out[i] = exp(x[i] - m) / d, written to the segment's own range
 * of out; an empty segment writes nothing. fp64 variant = the stated oracle
 * for config "segmented softmax"; the fp32 variant follows the same three
 * steps in fp32 with sequential order and is what a CPU run of the
 * reference's composition would compute (timed as the CPU baseline). */
int swg_oracle_segsoftmax_f64(const float *values, const int32_t *offsets,
                              double *out, int64_t segment_count, int threads) {
  int used = threads > 1 ? threads : 1;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 16) num_threads(used)
#else
  used = 1;
#endif
  for (int64_t sid = 0; sid < segment_count; ++sid) {
    int64_t start = offsets[sid], end = offsets[sid + 1];
    if (start >= end) continue;
    float m32 = -INFINITY;
    for (int64_t i = start; i < end; ++i) m32 = oracle_maximumf(m32, values[i]);
    double m = (double)m32, d = 0.0;
    for (int64_t i = start; i < end; ++i) d += exp((double)values[i] - m);
    for (int64_t i = start; i < end; ++i)
      out[i] = exp((double)values[i] - m) / d;
  }
  return used;
}

int swg_oracle_segsoftmax_f32(const float *values, const int32_t *offsets,
                              float *out, int64_t segment_count, int threads) {
  int used = threads > 1 ? threads : 1;
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 16) num_threads(used)
#else
  used = 1;
#endif
  for (int64_t sid = 0; sid < segment_count; ++sid) {
    int64_t start = offsets[sid], end = offsets[sid + 1];
    if (start >= end) continue;
    float m = -INFINITY;
    for (int64_t i = start; i < end; ++i) m = oracle_maximumf(m, values[i]);
    float d = 0.0f;
    for (int64_t i = start; i < end; ++i) d = d + expf(values[i] - m);
    for (int64_t i = start; i < end; ++i) out[i] = expf(values[i] - m) / d;
  }
  return used;
}

/* Fixed-block vector add, lib/Conversion/FixedBlockToGPU/FixedBlockToGPU.cpp
 * :198-221: out[i] = x[i] + y[i] for i = bid*BLOCK + tid, guarded i < n.  One
 * arith.addf per element, so the block size does not change any bit; the
 * block loop is kept so the restatement follows the reference's indexing. */
int swg_oracle_vadd_f32(const float *x, const float *y, float *out, int64_t n,
                        int64_t block, int threads) {
  if (block <= 0) return -1;
  int64_t grid = (n + block - 1) / block;
  int used = threads > 1 ? threads : 1;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(used)
#else
  used = 1;
#endif
  for (int64_t bid = 0; bid < grid; ++bid) {
    for (int64_t tid = 0; tid < block; ++tid) {
      int64_t i = bid * block + tid;
      if (i < n) out[i] = x[i] + y[i];
    }
  }
  return used;
}

int swg_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
