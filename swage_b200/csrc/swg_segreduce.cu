// Segmented sum / max / min over dense fp32 values addressed by CSR int32
// offsets.
//
// Replaces the kernels the reference generates in
// lib/Conversion/SegmentedReduction/SegmentedReduction.cpp:185-283 (one
// 128-thread CTA per segment, block-stride scalar loads, gpu.all_reduce).
// Schedules:
//
//   warp        one warp per segment, 128-bit loads straight from global
//   cta         one CTA per segment (the reference's own mapping, vectorised)
//   split       the plan's tile tasks, one per warp, two per CTA
//   persistent  the same tile tasks, drawn from a ticket counter by the
//               warps of one resident CTA per SM; every warp keeps three
//               tiles in flight in its own shared-memory ring
//   resident    the same tile tasks at a fixed stride per SM, one stage per
//               warp of one resident CTA per SM
//
// The three tile schedules stage tiles with bulk async copies (TMA); segments
// that cross a tile boundary leave partials that a small merge pass, launched
// right behind the tile kernel, combines.
//
// All of them are HBM-bound: 4 bytes per value + 4 per offset + 4 per output.
// No floating-point atomics anywhere: every result is produced by a fixed
// combine tree, so launches are bit-reproducible.
#include <mutex>

#include "swg_common.cuh"
#include "swg_launch.h"

namespace swg {

// ---------------------------------------------------------------------------
// warp per segment
// ---------------------------------------------------------------------------
#ifndef SWG_WARP_THREADS
#define SWG_WARP_THREADS 256
#endif
#ifndef SWG_WARP_INFLIGHT
#define SWG_WARP_INFLIGHT 8
#endif
#ifndef SWG_WARP_MINBLOCKS
#define SWG_WARP_MINBLOCKS 4
#endif
constexpr int kWarpKernelThreads = SWG_WARP_THREADS;

template <class Op>
__global__ void __launch_bounds__(kWarpKernelThreads, SWG_WARP_MINBLOCKS)
segreduce_warp_kernel(const float *__restrict__ values,
                      const int32_t *__restrict__ offsets,
                      float *__restrict__ out, int32_t segment_count) {
  // Launched with programmatic stream serialisation: when the kernel before
  // this one in the stream is one of this library's, the CTAs are placed
  // while it drains; nothing of the caller's is touched before the wait.
  asm volatile("griddepcontrol.launch_dependents;");
  const int lane = threadIdx.x & 31;
  const int64_t warp =
      ((int64_t)blockIdx.x * kWarpKernelThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kWarpKernelThreads) >> 5;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int64_t seg = warp; seg < segment_count; seg += nwarps) {
    const int64_t begin = __ldg(offsets + seg);
    const int64_t end = __ldg(offsets + seg + 1);
    // eight 128-bit loads per lane are issued before the first is used: a
    // segment of up to 1024 values is one round trip to memory
    float acc = strided_partial<Op, SWG_WARP_INFLIGHT>(values, begin, end, lane, kWarp);
    acc = warp_reduce<Op>(acc);
    if (lane == 0) out[seg] = acc;
  }
}

// Sum AND max of every segment in one pass over the values (one launch, each
// value read once, two outputs per segment): the canonical configuration asks
// for both reductions of the same input.  Identities and combiners are those
// of the two single kernels (SegmentedReduction.cpp:156-161, 236-241,
// 256-258).  kCta = false: one warp per segment; true: one CTA per segment.
template <bool kCta>
__global__ void __launch_bounds__(kWarpKernelThreads, SWG_WARP_MINBLOCKS)
segreduce_sum_max_kernel(const float *__restrict__ values,
                         const int32_t *__restrict__ offsets,
                         float *__restrict__ out_sum,
                         float *__restrict__ out_max, int32_t segment_count) {
  __shared__ float scratch[32];
  // (programmatic stream serialisation: see segreduce_warp_kernel)
  asm volatile("griddepcontrol.launch_dependents;");
  const int lane = threadIdx.x & 31;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (kCta) {
    for (int64_t seg = blockIdx.x; seg < segment_count; seg += gridDim.x) {
      const int64_t begin = __ldg(offsets + seg);
      const int64_t end = __ldg(offsets + seg + 1);
      const SumMax r = strided_sum_max<SWG_WARP_INFLIGHT>(
          values, begin, end, threadIdx.x, kWarpKernelThreads);
      const float sum = cta_reduce<SumOp>(r.sum, scratch);
      const float max = cta_reduce<MaxOp>(r.max, scratch);
      if (threadIdx.x == 0) {
        out_sum[seg] = sum;
        out_max[seg] = max;
      }
    }
    return;
  }
  const int64_t warp =
      ((int64_t)blockIdx.x * kWarpKernelThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kWarpKernelThreads) >> 5;
  for (int64_t seg = warp; seg < segment_count; seg += nwarps) {
    const int64_t begin = __ldg(offsets + seg);
    const int64_t end = __ldg(offsets + seg + 1);
    const SumMax r =
        strided_sum_max<SWG_WARP_INFLIGHT>(values, begin, end, lane, kWarp);
    const float sum = warp_reduce<SumOp>(r.sum);
    const float max = warp_reduce<MaxOp>(r.max);
    if (lane == 0) {
      out_sum[seg] = sum;
      out_max[seg] = max;
    }
  }
}

// ---------------------------------------------------------------------------
// warp or CTA per segment for f16 / bf16 / i32 values: the plan-free mapping
// of small inputs.  Coalesced element loads, four accumulators per thread.
// ---------------------------------------------------------------------------
template <class Op, class T, bool kCta, class M = NoMap>
__global__ void __launch_bounds__(kWarpKernelThreads)
segreduce_typed_kernel(const T *__restrict__ values,
                       const int32_t *__restrict__ offsets,
                       typename Op::Acc *__restrict__ out,
                       int32_t segment_count, M map) {
  using A = typename Op::Acc;
  __shared__ float scratch[32];
  const int lane = threadIdx.x & 31;
  const int rank = kCta ? (int)threadIdx.x : lane;
  const int width = kCta ? kWarpKernelThreads : kWarp;
  const int64_t first =
      kCta ? (int64_t)blockIdx.x
           : ((int64_t)blockIdx.x * kWarpKernelThreads + threadIdx.x) >> 5;
  const int64_t stride =
      kCta ? (int64_t)gridDim.x
           : ((int64_t)gridDim.x * kWarpKernelThreads) >> 5;
  with_fixed_map(map, [&](auto apply) {
    for (int64_t seg = first; seg < segment_count; seg += stride) {
      const int64_t begin = __ldg(offsets + seg);
      const int64_t end = __ldg(offsets + seg + 1);
      A a0 = Op::identity(), a1 = Op::identity(), a2 = Op::identity(),
        a3 = Op::identity();
      int64_t i = begin + rank;
      for (; i + 3 * width < end; i += 4 * width) {
        const T q0 = values[i], q1 = values[i + width],
                q2 = values[i + 2 * width], q3 = values[i + 3 * width];
        a0 = Op::apply(a0, apply(Elem<T>::get(q0)));
        a1 = Op::apply(a1, apply(Elem<T>::get(q1)));
        a2 = Op::apply(a2, apply(Elem<T>::get(q2)));
        a3 = Op::apply(a3, apply(Elem<T>::get(q3)));
      }
      for (; i < end; i += width)
        a0 = Op::apply(a0, apply(Elem<T>::get(values[i])));
      A r = Op::apply(Op::apply(a0, a1), Op::apply(a2, a3));
      r = kCta ? cta_reduce<Op>(r, scratch) : warp_reduce<Op>(r);
      if (rank == 0) out[seg] = r;
    }
  });
}

// ---------------------------------------------------------------------------
// CTA per segment
// ---------------------------------------------------------------------------
template <class Op>
__global__ void segreduce_cta_kernel(const float *__restrict__ values,
                                     const int32_t *__restrict__ offsets,
                                     float *__restrict__ out,
                                     int32_t segment_count) {
  __shared__ float scratch[32];
  for (int64_t seg = blockIdx.x; seg < segment_count; seg += gridDim.x) {
    const int64_t begin = __ldg(offsets + seg);
    const int64_t end = __ldg(offsets + seg + 1);
    float acc =
        strided_partial<Op>(values, begin, end, threadIdx.x, blockDim.x);
    acc = cta_reduce<Op>(acc, scratch);
    if (threadIdx.x == 0) out[seg] = acc;
  }
}

// ---------------------------------------------------------------------------
// Tile tasks (split, persistent and resident schedules)
//
// A task is small enough (kTileValues values, kTileMaxSegments segments) for
// ONE WARP to own it from the bulk copy to the output store, so no CTA-wide
// barrier appears anywhere: every warp runs its own copy -> wait -> reduce
// pipeline on its own shared-memory stages and its own mbarriers, and the SM
// overlaps the phases of its resident warps.
//
// A segment that crosses a tile boundary is cut into pieces that different
// warps reduce; each piece leaves its partial in the plan's scratch and a
// merge pass -- a second, small kernel launched right behind the tile kernel
// -- combines the partials of every cut segment in slot order.  (Merging
// inside the tile kernel, by whichever warp delivers a segment's last partial,
// was built and measured: the device-wide fence each piece then needs before
// it counts itself in costs 20 - 50 % of the kernel's throughput, far more
// than the second launch.)
// ---------------------------------------------------------------------------
#ifndef SWG_WIDE_VECTOR
#define SWG_WIDE_VECTOR 0  // 1: whole-warp segments of a packed tile by 128-bit loads
#endif
constexpr int kLaneSegment = 16;    // reduced by a single lane inside a tile
constexpr int kGroupSegment = 256;  // up to here by a group of eight lanes
// One stage holds the task's values and, for a packed task, its offsets right
// behind them (the planner bounds values + segments by kTileItems so both
// fit): element i sits at tile[i - origin], offset j of the aligned offsets
// range at ((int*)tile)[offsets_base + j].
constexpr int kTileFloats = kTileValues + 8;
constexpr int kStageBytes = ((kTileFloats * 4 + 127) / 128) * 128;
static_assert(kTileItems + 3 + 3 + 8 <= kTileFloats,
              "values, padding and offsets of a packed task fit one stage");
static_assert(kStatusWord == 12, "report() reads control[12..13]");

// Elements of type T per 16-byte line, and the first 32-bit word of the
// offsets of a packed task in its stage: the 16-byte line after its values.
template <class T>
constexpr int kPerLine = 16 / (int)sizeof(T);
// Phase of the values pointer inside a 16-byte line, in elements.
template <class T>
__device__ __forceinline__ int value_phase(const T *values) {
  return (int)(((uintptr_t)values / sizeof(T)) & (kPerLine<T> - 1));
}
template <class T>
__device__ __forceinline__ int offsets_word(int shift, int vcount) {
  return (((shift + vcount) * (int)sizeof(T) + 15) >> 4) << 2;
}
constexpr uint32_t kTaskStop = 15u;  // sentinel kind: no more tasks

#ifndef SWG_SPLIT_WARPS
#define SWG_SPLIT_WARPS 2
#endif

constexpr int kSplitWarps = SWG_SPLIT_WARPS;  // split: tasks per CTA, one stage each
constexpr int kTaskLookahead = 2048;  // CTAs ahead whose descriptors are prefetched

struct Stage {
  unsigned char *tile;  // element i of the task at ((T *)tile)[i - origin]
};

// Per-warp lists of the segments (of the current 32) that more than one lane
// works on, and their results.
struct WarpScratch {
  int begin[32];
  int end[32];
  uint32_t result[32];  // accumulator words (fp32 or int32)
};

__device__ __forceinline__ Stage stage_at(unsigned char *base, int index) {
  unsigned char *p = base + (size_t)index * kStageBytes;
  Stage s;
  s.tile = p;
  return s;
}

__device__ __forceinline__ Task stop_task() {
  Task t;
  t.seg = 0;
  t.count = 0;
  t.vbegin = 0;
  t.vcount_kind = kTaskStop << 28;
  t.head_slot = t.tail_slot = -1;
  t.link_first = -1;
  t.link_pieces = 0;
  return t;
}

__device__ __forceinline__ bool is_stop(const Task &t) {
  return (t.vcount_kind >> 28) == kTaskStop;
}

// Broadcast lane `src`'s task to the whole warp.
__device__ __forceinline__ Task shuffle_task(const Task &mine, int src) {
  Task t;
  t.seg = __shfl_sync(kFullMask, mine.seg, src);
  t.count = __shfl_sync(kFullMask, mine.count, src);
  t.vbegin = __shfl_sync(kFullMask, mine.vbegin, src);
  t.vcount_kind = __shfl_sync(kFullMask, mine.vcount_kind, src);
  t.head_slot = __shfl_sync(kFullMask, mine.head_slot, src);
  t.tail_slot = __shfl_sync(kFullMask, mine.tail_slot, src);
  t.link_first = __shfl_sync(kFullMask, mine.link_first, src);
  t.link_pieces = __shfl_sync(kFullMask, mine.link_pieces, src);
  return t;
}

// What a task may touch; every task is checked against it before use, so a
// plan that does not belong to the launch's arrays (or a corrupted one) is
// reported through the error word instead of being dereferenced.
struct Limits {
  int32_t value_count;
  int32_t segment_count;
  int32_t partial_slots;
  int32_t slot_step;
};

// Slot of piece k of a segment whose piece 0 has slot `first` (see Task).
__device__ __forceinline__ int piece_slot(int first, int k, int step) {
  return first + k * step - (k > 0 ? step - 1 : 0);
}
__device__ __forceinline__ int piece_index(int first, int slot, int step) {
  return slot == first ? 0 : (slot - first + step - 1) / step;
}

// Slots first .. piece_slot(pieces - 1) lie inside the scratch.
__device__ __forceinline__ bool slots_ok(int first, int pieces,
                                         const Limits &limits) {
  return first >= 0 && pieces >= 2 &&
         (int64_t)first + (int64_t)(pieces - 1) * limits.slot_step <
             (int64_t)limits.partial_slots + (limits.slot_step - 1);
}

// (A task's link_first / link_pieces are not used by the tile kernels: the
// merge pass checks its own records.)
__device__ __forceinline__ bool task_ok(const Task &t, const Limits &limits) {
  const uint32_t kind = t.vcount_kind >> 28;
  const int64_t vcount = (int64_t)(t.vcount_kind & kTaskCountMask);
  if (t.seg < 0 || t.seg >= limits.segment_count) return false;
  if (t.vbegin < 0 || vcount > kTileValues ||
      (int64_t)t.vbegin + vcount > limits.value_count)
    return false;
  if (kind == kTaskPack)
    return t.count >= 1 && t.count <= kTileMaxSegments &&
           vcount + t.count <= kTileItems &&
           (int64_t)t.seg + t.count <= limits.segment_count &&
           t.head_slot >= -1 && t.head_slot < limits.partial_slots &&
           t.tail_slot >= -1 && t.tail_slot < limits.partial_slots &&
           !(t.count == 1 && t.head_slot >= 0 && t.tail_slot >= 0);
  if (kind == kTaskChunk)
    return t.count >= -1 && t.count < limits.partial_slots;
  return false;
}

// The lines of `values` a task's bulk copy takes: every 16-byte line that
// intersects the task's value range and lies wholly inside the values array
// (neighbouring elements that ride along are never read).  Element i lands at
// tile[i - origin] with origin = vbegin - ((vbegin + mis) mod P), P the
// elements per line; `mis` is the phase of the values pointer inside a 16-byte
// line, in elements.
struct CopyRange {
  int64_t origin, lo, hi;  // copy [lo, hi); hi <= lo: nothing to copy
};

template <class T>
__device__ __forceinline__ CopyRange copy_range(const Task &task, int mis,
                                                int32_t value_count) {
  constexpr int P = kPerLine<T>;
  const int64_t vb = task.vbegin;
  const int64_t ve = vb + (int64_t)(task.vcount_kind & kTaskCountMask);
  CopyRange r;
  r.origin = vb - ((vb + mis) & (P - 1));
  r.lo = r.origin < 0 ? r.origin + P : r.origin;
  r.hi = ve + ((P - ((ve + mis) & (P - 1))) & (P - 1));
  const int64_t last_line =
      (int64_t)value_count - ((value_count + mis) & (P - 1));
  if (r.hi > last_line) r.hi = last_line;
  if (r.hi < r.lo) r.hi = r.lo;
  return r;
}

// Stage one task; runs entirely in the calling thread.  The at most three
// elements at either end of the array that no whole line covers are fetched
// with plain loads.
template <class T>
__device__ __forceinline__ void issue_task(const Task &task,
                                           const T *__restrict__ values,
                                           int mis, int32_t value_count,
                                           const int32_t *__restrict__ d_off,
                                           Stage stage, uint64_t *full) {
  const uint32_t kind = task.vcount_kind >> 28;
  const int64_t vb = task.vbegin;
  const int64_t ve = vb + (int64_t)(task.vcount_kind & kTaskCountMask);
  const CopyRange r = copy_range<T>(task, mis, value_count);
  const int64_t origin = r.origin, lo = r.lo, hi = r.hi;
  T *tile = reinterpret_cast<T *>(stage.tile);
  if (lo > vb || hi < ve) {
    // only the first and the last task of an array can get here
    for (int64_t idx = vb; idx < ve && idx < lo; ++idx)
      tile[idx - origin] = values[idx];
    for (int64_t idx = hi > vb ? hi : vb; idx < ve; ++idx)
      if (idx >= hi || idx < lo) tile[idx - origin] = values[idx];
  }
  const uint32_t bytes_v = (uint32_t)(hi - lo) * (uint32_t)sizeof(T);
  uint32_t bytes_o = 0;
  int32_t o_lo = 0;
  if (kind == kTaskPack) {
    o_lo = task.seg & ~3;
    const int32_t o_hi = (task.seg + task.count + 1 + 3) & ~3;
    bytes_o = (uint32_t)(o_hi - o_lo) * 4u;
  }
  // the stage may have been read a moment ago (generic proxy); the copies
  // below write it through the async proxy
  fence_proxy_async();
  mbar_arrive_expect_tx(full, bytes_v + bytes_o);
  if (bytes_v) bulk_g2s(tile + (lo - origin), values + lo, bytes_v, full);
  if (bytes_o)
    bulk_g2s(reinterpret_cast<int32_t *>(stage.tile) +
                 offsets_word<T>((int)(vb - origin), (int)(ve - vb)),
             d_off + o_lo, bytes_o, full);
}

// 128-bit load from a stage, explicitly in the shared window.
__device__ __forceinline__ uint4 lds_line(const void *p) {
  uint4 q;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w)
               : "r"(smem_u32(p)));
  return q;
}

// Warp-collective: reduces tile[lo, hi) (element indices) -- scalar ends,
// 128-bit body, four independent accumulators per lane -- and returns the
// result to every lane.
template <class Op, class T, class M>
__device__ __forceinline__ typename Op::Acc warp_range(const T *tile, int lo,
                                                       int hi, int lane,
                                                       const M &map) {
  using A = typename Op::Acc;
  constexpr int P = kPerLine<T>;
  int blo = (lo + P - 1) & ~(P - 1), bhi = hi & ~(P - 1);
  if (blo > bhi) blo = bhi = hi;  // too short for an aligned body
  const int head_end = blo < hi ? blo : hi;
  A a0 = Op::identity(), a1 = Op::identity(), a2 = Op::identity(),
    a3 = Op::identity();
  if (lo + lane < head_end)
    a0 = Op::apply(a0, map(Elem<T>::get(tile[lo + lane])));
  const uint4 *body = reinterpret_cast<const uint4 *>(tile);
  const int vlo = blo / P, vhi = bhi / P;
  int v = vlo + lane;
  for (; v + 96 < vhi; v += 128) {
    const uint4 q0 = lds_line(body + v), q1 = lds_line(body + v + 32),
                q2 = lds_line(body + v + 64), q3 = lds_line(body + v + 96);
    a0 = fold_line<Op, T, M>(a0, q0, map);
    a1 = fold_line<Op, T, M>(a1, q1, map);
    a2 = fold_line<Op, T, M>(a2, q2, map);
    a3 = fold_line<Op, T, M>(a3, q3, map);
  }
  for (; v < vhi; v += 32)
    a0 = fold_line<Op, T, M>(a0, lds_line(body + v), map);
  const int tail = bhi > head_end ? bhi : head_end;
  if (tail + lane < hi)
    a1 = Op::apply(a1, map(Elem<T>::get(tile[tail + lane])));
  return warp_reduce<Op>(Op::apply(Op::apply(a0, a1), Op::apply(a2, a3)));
}

// Warp-collective: reduce one staged task.
template <class Op, class T, class M, class R = NoPeers>
__device__ __forceinline__ void process_task(
    const Task &task, const Stage &stage, int mis,
    typename Op::Acc *__restrict__ out,
    typename Op::Acc *__restrict__ partials, WarpScratch *scratch,
    const Limits &limits, uint32_t *control, int lane, const M &map,
    const R &peers = R{}) {
  using A = typename Op::Acc;
  constexpr int P = kPerLine<T>;
  if (!task_ok(task, limits)) {
    if (lane == 0) report(control, kErrBadTask, (uint32_t)task.seg);
    return;
  }
  const uint32_t kind = task.vcount_kind >> 28;
  const int vcount = (int)(task.vcount_kind & kTaskCountMask);
  const int shift = (int)(((int64_t)task.vbegin + mis) & (P - 1));
  const T *tile = reinterpret_cast<const T *>(stage.tile);
  A *results = reinterpret_cast<A *>(scratch->result);

  if (kind == kTaskChunk) {
    // One piece of a long segment occupies tile[shift, shift + vcount).
    const A r = warp_range<Op, T, M>(tile, shift, shift + vcount, lane, map);
    if (lane == 0) {
      if (task.count < 0) peers.store(out, task.seg, r);
      else partials[task.count] = r;
    }
    return;
  }

  // Packed whole segments, 32 at a time: lane k owns segment base + k.
  //   length <= kLaneSegment   summed by the owning lane alone
  //   length <= kGroupSegment  listed, then reduced four at a time by the
  //                            warp's four groups of eight lanes
  //   longer                   listed, then reduced by the whole warp
  // Listed results come back through the warp's scratch to their owning
  // lanes, so the 32 results leave in one coalesced store.  Tile-relative
  // bounds of segment k are soff[k] - origin and soff[k + 1] - origin.
  const int32_t *soff = reinterpret_cast<const int32_t *>(stage.tile) +
                        offsets_word<T>(shift, vcount) + (task.seg & 3);
  const int origin = task.vbegin - shift;
  const unsigned below = (1u << lane) - 1u;
  const int group = lane >> 3, sub = lane & 7;
  const unsigned group_mask = 0xffu << (group * 8);
  for (int base = 0; base < task.count; base += 32) {
    const int k = base + lane;
    const bool valid = k < task.count;
    int a = valid ? soff[k] - origin : 0;
    int b = valid ? soff[k + 1] - origin : 0;
    // the first segment may have begun in an earlier task and the last may
    // continue in a later one: only the part inside this tile is reduced
    // here, and the result is a partial
    const bool head_piece = valid && k == 0 && task.head_slot >= 0;
    const bool tail_piece =
        valid && k == task.count - 1 && task.tail_slot >= 0;
    if (head_piece && a <= shift) a = shift;
    if (tail_piece && b >= shift + vcount) b = shift + vcount;
    if (valid && (a < shift || b < a || b > shift + vcount)) {
      // offsets that do not match the plan: report, treat as empty
      report(control, kErrBadSegment, (uint32_t)(task.seg + k));
      a = b = shift;
    }
    const int length = b - a;
    A acc = Op::identity();
    const bool medium =
        valid && length > kLaneSegment && length <= kGroupSegment;
    const bool wide = valid && length > kGroupSegment;
    // tiny segments: the loads are issued eight at a time under a predicate
    // (independent of one another) and folded left to right; slots past the
    // segment's end hold the identity, which leaves the result unchanged
    const bool tiny = valid && length <= kLaneSegment;
    if (tiny) {
      A x[8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
        x[i] = a + i < b ? map(Elem<T>::get(tile[a + i])) : Op::identity();
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = Op::apply(acc, x[i]);
    }
    if (__any_sync(kFullMask, tiny && length > 8)) {
      if (tiny) {
        A x[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          x[i] = a + 8 + i < b ? map(Elem<T>::get(tile[a + 8 + i]))
                               : Op::identity();
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = Op::apply(acc, x[i]);
      }
    }
    const unsigned medium_mask = __ballot_sync(kFullMask, medium);
    const unsigned wide_mask = __ballot_sync(kFullMask, wide);
    // a piece of a cut segment leaves a partial; a whole segment its result
    A *piece = nullptr;
    if (head_piece) piece = partials + task.head_slot;
    if (tail_piece) piece = partials + task.tail_slot;
    if ((medium_mask | wide_mask) == 0) {
      if (valid) {
        if (piece) *piece = acc;
        else peers.store(out, task.seg + k, acc);
      }
      continue;
    }
    const int medium_count = __popc(medium_mask);
    const int listed = medium_count + __popc(wide_mask);
    int slot = -1;
    if (medium) slot = __popc(medium_mask & below);
    if (wide) slot = medium_count + __popc(wide_mask & below);
    if (slot >= 0) {
      scratch->begin[slot] = a;
      scratch->end[slot] = b;
    }
    __syncwarp();
    for (int e = group; e < medium_count; e += 4) {
      const int ea = scratch->begin[e], eb = scratch->end[e];
      A p0 = Op::identity(), p1 = Op::identity(), p2 = Op::identity(),
        p3 = Op::identity();
      int i = ea + sub;
      for (; i + 24 < eb; i += 32) {
        p0 = Op::apply(p0, map(Elem<T>::get(tile[i])));
        p1 = Op::apply(p1, map(Elem<T>::get(tile[i + 8])));
        p2 = Op::apply(p2, map(Elem<T>::get(tile[i + 16])));
        p3 = Op::apply(p3, map(Elem<T>::get(tile[i + 24])));
      }
      for (; i < eb; i += 8) p0 = Op::apply(p0, map(Elem<T>::get(tile[i])));
      A r = Op::apply(Op::apply(p0, p1), Op::apply(p2, p3));
      r = Op::apply(r, __shfl_xor_sync(group_mask, r, 4));
      r = Op::apply(r, __shfl_xor_sync(group_mask, r, 2));
      r = Op::apply(r, __shfl_xor_sync(group_mask, r, 1));
      if (sub == 0) results[e] = r;
    }
    __syncwarp();
    for (int e = medium_count; e < listed; ++e) {
      // (the 128-bit range reduce of the chunk path was tried here: same
      // speed on the lognormal workload, eight more registers everywhere)
#if SWG_WIDE_VECTOR
      const A r = warp_range<Op, T, M>(tile, scratch->begin[e],
                                       scratch->end[e], lane, map);
#else
      const int ea = scratch->begin[e], eb = scratch->end[e];
      A p0 = Op::identity(), p1 = Op::identity(), p2 = Op::identity(),
        p3 = Op::identity();
      int i = ea + lane;
      for (; i + 96 < eb; i += 128) {
        p0 = Op::apply(p0, map(Elem<T>::get(tile[i])));
        p1 = Op::apply(p1, map(Elem<T>::get(tile[i + 32])));
        p2 = Op::apply(p2, map(Elem<T>::get(tile[i + 64])));
        p3 = Op::apply(p3, map(Elem<T>::get(tile[i + 96])));
      }
      for (; i < eb; i += 32) p0 = Op::apply(p0, map(Elem<T>::get(tile[i])));
      const A r =
          warp_reduce<Op>(Op::apply(Op::apply(p0, p1), Op::apply(p2, p3)));
#endif
      if (lane == 0) results[e] = r;
    }
    __syncwarp();
    if (slot >= 0) acc = results[slot];
    if (valid) {
      if (piece) *piece = acc;
      else peers.store(out, task.seg + k, acc);
    }
    __syncwarp();  // the lists are rewritten by the next 32 segments
  }
}

// split schedule: CTA b, warp w reduces task b * kSplitWarps + w.
//
// Launched with programmatic stream serialisation.  Everything before
// griddepcontrol.wait (CTA placement, barrier set-up, the descriptor round
// trip) touches only memory the plan owns and may overlap the tail of the
// kernel before; the CTAs of the first wave (blockIdx < prefetch_ctas) also
// ask L2 to fetch their tile there, so that the first copies of the launch
// find their lines on the way instead of starting a cold DRAM round trip
// after the wait.  The caller's arrays are read into the SM and written only
// after the kernel before has finished.
template <class Op, class T, class M = NoMap, class R = NoPeers>
__global__ void __launch_bounds__(kSplitWarps * 32)
segreduce_split_kernel(const T *__restrict__ values,
                       typename Op::Acc *__restrict__ out, int32_t value_count,
                       const Task *__restrict__ tasks, int32_t task_count,
                       const int32_t *__restrict__ d_off,
                       typename Op::Acc *__restrict__ partials,
                       uint32_t *__restrict__ control, Limits limits,
                       uint32_t prefetch_ctas, M map, R peers) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[kSplitWarps];
  __shared__ WarpScratch scratch[kSplitWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int mis = value_phase(values);
  // let the kernel that follows in the stream be placed as soon as slots free
  // up; it waits for this grid to finish before it touches anything of the
  // caller's
  asm volatile("griddepcontrol.launch_dependents;");
  const int64_t index = (int64_t)blockIdx.x * kSplitWarps + warp;
  if (index >= task_count) return;
  if (lane == 0) {
    mbar_init(&full[warp], 1);
    fence_mbar_init();
  }
  __syncwarp();
  // the descriptors of the CTAs that will take this CTA's place a wave or so
  // from now: L2 starts fetching their line, so that their first instruction
  // -- the descriptor load every CTA's life begins with -- is an L2 hit
  // (1 % on the extreme-skew sum, 2 - 3 % on a 2^27-value share of it)
  if (lane == 1) {
    const int64_t ahead = index + (int64_t)kTaskLookahead * kSplitWarps;
    if (ahead < task_count)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(tasks + ahead));
  }
  const Task task = tasks[index];
  const Stage stage = stage_at(smem, warp);
  const bool ok = task_ok(task, limits);
  if (ok && lane == 0 && blockIdx.x < prefetch_ctas) {
    const CopyRange r = copy_range<T>(task, mis, value_count);
    if (r.hi > r.lo)
      bulk_prefetch_l2(values + r.lo,
                       (uint32_t)(r.hi - r.lo) * (uint32_t)sizeof(T));
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (!ok) {
    if (lane == 0) report(control, kErrBadTask, (uint32_t)index);
    return;
  }
  if (lane == 0)
    issue_task(task, values, mis, value_count, d_off, stage, &full[warp]);
  if (!mbar_wait(&full[warp], 0)) {
    if (lane == 0) report(control, kErrTimeout, (uint32_t)index);
    return;
  }
  with_fixed_map(map, [&](auto apply) {
    process_task<Op, T, decltype(apply), R>(task, stage, mis, out, partials,
                                            &scratch[warp], limits, control,
                                            lane, apply, peers);
  });
}

// persistent schedule: one resident CTA per SM, every warp an independent
// worker with its own ring of kStages shared-memory stages and its own
// mbarriers; no warp ever waits on another.  A worker draws tickets kStages
// at a time from control[0], two rounds ahead of their use, and loads the
// task descriptors one round ahead, so neither the atomic nor the descriptor
// load sits on its critical path; it refills a stage with the next task's
// bulk async copy as soon as it has reduced the previous one.
// control[1] counts workers that have stopped drawing; the last one resets
// control[0] and control[1] so the next launch needs no memset.
// control[2] is the error code, control[3] its detail.
template <class Op, int kWarps, int kStages>
__global__ void __launch_bounds__(kWarps * 32, 1)
segreduce_persistent_kernel(const float *__restrict__ values,
                            float *__restrict__ out, int32_t value_count,
                            const Task *__restrict__ tasks, int32_t task_count,
                            const int32_t *__restrict__ d_off,
                            float *__restrict__ partials,
                            uint32_t *__restrict__ control, Limits limits) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[kWarps * kStages];
  __shared__ WarpScratch scratch[kWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int mis = value_phase(values);
  uint64_t *bars = full + warp * kStages;
  unsigned char *ring = smem + (size_t)warp * kStages * kStageBytes;
  if (lane == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&bars[s], 1);
    fence_mbar_init();
  }
  __syncwarp();

  // draw() leaves the ticket in lane 0 only; it is broadcast where it is
  // used, a round later, so the atomic's latency is off the critical path.
  auto draw = [&]() -> uint32_t {
    uint32_t t = 0;
    if (lane == 0) t = atomicAdd(control, (uint32_t)kStages);
    return t;
  };
  auto fetch = [&](uint32_t lane0_base) -> Task {
    const uint32_t base = __shfl_sync(kFullMask, lane0_base, 0);
    Task t = stop_task();
    const uint32_t mine = base + (uint32_t)lane;
    if (lane < kStages && mine < (uint32_t)task_count) t = tasks[mine];
    return t;
  };
  // Stage `t` into stage s; a task that fails its check is staged as an
  // immediate arrival and reported by process_task.
  auto stage_in = [&](const Task &t, int s) {
    if (lane == 0) {
      if (task_ok(t, limits))
        issue_task(t, values, mis, value_count, d_off, stage_at(ring, s),
                   &bars[s]);
      else
        mbar_arrive(&bars[s]);
    }
  };

  // lane s holds the task now staged in stage s (cur) and the one that will
  // replace it (nxt)
  Task cur = fetch(draw());
  Task nxt = fetch(draw());
  uint32_t base_after = draw();
#pragma unroll
  for (int s = 0; s < kStages; ++s) {
    const Task t = shuffle_task(cur, s);
    if (!is_stop(t)) stage_in(t, s);
  }
  uint32_t parity = 0;
  bool running = true, ok = true;
  while (running) {
    const Task after = fetch(base_after);  // descriptors two rounds ahead
    base_after = draw();                   // tickets three rounds ahead
#pragma unroll
    for (int s = 0; s < kStages; ++s) {
      const Task t = shuffle_task(cur, s);
      if (is_stop(t)) {
        running = false;
        break;
      }
      if (!mbar_wait(&bars[s], parity)) {
        if (lane == 0) report(control, kErrTimeout, (uint32_t)t.seg);
        ok = false;
        running = false;
        break;
      }
      process_task<Op, float, NoMap>(t, stage_at(ring, s), mis, out, partials,
                                     &scratch[warp], limits, control, lane,
                                     NoMap{});
      __syncwarp();  // every lane is done with the stage before it is refilled
      const Task n = shuffle_task(nxt, s);
      if (!is_stop(n)) stage_in(n, s);
    }
    cur = nxt;
    nxt = after;
    parity ^= 1u;
  }
  if (!ok) {
    // A wait gave up: let this warp's copies in flight land (bounded) before
    // its shared memory can be handed on.
    for (int s = 0; s < kStages; ++s) mbar_wait(&bars[s], parity);
  }
  if (lane == 0) {
    __threadfence();
    const uint32_t finished = atomicAdd(control + 1, 1u);
    if (finished == gridDim.x * kWarps - 1) {
      atomicExch(control, 0u);
      atomicExch(control + 1, 0u);
    }
  }
}

// resident schedule: one CTA per SM, every warp owns one stage for the whole
// launch.  The SM's tiles are those of its own stride (tile = round * CTAs +
// CTA, so neighbouring tiles run on neighbouring SMs at the same time, as in
// the split schedule), and the rounds are handed out inside the CTA in the
// order warps ask for them (a shared-memory counter): whatever the pace of
// single warps, the tiles an SM has in flight are always the next ones of its
// stride, which keeps the whole machine reading one narrow window of the
// input -- with a fixed round per warp the window smears and the same kernel
// is 6 % slower.  What the schedule removes against split is the part of a
// tile's life in which its stage holds nothing: no CTA is launched per pair
// of tiles, and the next task's descriptor is fetched while the current
// tile's copy is in flight.  Measured: 7 - 9 % faster than split where tiles
// hold many segments (their reduction keeps a stage busy longest), 7 % slower
// where nearly every tile is a chunk of a long segment -- the planner picks by
// the share of values in long segments.
template <class Op, class T, int kWarps, class M = NoMap, class R = NoPeers>
__global__ void __launch_bounds__(kWarps * 32, 1)
segreduce_resident_kernel(const T *__restrict__ values,
                          typename Op::Acc *__restrict__ out,
                          int32_t value_count,
                          const Task *__restrict__ tasks, int32_t task_count,
                          const int32_t *__restrict__ d_off,
                          typename Op::Acc *__restrict__ partials,
                          uint32_t *__restrict__ control, Limits limits,
                          M map, R peers) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[kWarps];
  __shared__ WarpScratch scratch[kWarps];
  __shared__ int next_round;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int mis = value_phase(values);
  asm volatile("griddepcontrol.launch_dependents;");
  if (lane == 0) {
    mbar_init(&full[warp], 1);
    fence_mbar_init();
  }
  if (threadIdx.x == 0) next_round = 0;
  __syncthreads();
  const Stage stage = stage_at(smem, warp);
  auto draw = [&]() -> int64_t {
    int round = 0;
    if (lane == 0) round = atomicAdd(&next_round, 1);
    round = __shfl_sync(kFullMask, round, 0);
    return (int64_t)round * gridDim.x + blockIdx.x;
  };
  int64_t index = draw();
  if (index >= task_count) return;
  Task task = tasks[index];
  // the first tile of every warp: L2 starts fetching it while the kernel
  // before this one drains (see segreduce_split_kernel)
  if (lane == 0 && task_ok(task, limits)) {
    const CopyRange r = copy_range<T>(task, mis, value_count);
    if (r.hi > r.lo)
      bulk_prefetch_l2(values + r.lo,
                       (uint32_t)(r.hi - r.lo) * (uint32_t)sizeof(T));
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  uint32_t parity = 0;
  auto start = [&](const Task &t) {
    if (lane == 0) {
      if (task_ok(t, limits))
        issue_task(t, values, mis, value_count, d_off, stage, &full[warp]);
      else
        mbar_arrive(&full[warp]);  // reported by process_task
    }
  };
  start(task);
  while (true) {
    const int64_t next_index = draw();
    const bool more = next_index < task_count;
    Task next = task;
    if (more) next = tasks[next_index];  // in flight during the wait below
    if (!mbar_wait(&full[warp], parity)) {
      if (lane == 0) report(control, kErrTimeout, (uint32_t)index);
      return;
    }
    parity ^= 1u;
    with_fixed_map(map, [&](auto apply) {
      process_task<Op, T, decltype(apply), R>(task, stage, mis, out, partials,
                                              &scratch[warp], limits, control,
                                              lane, apply, peers);
    });
    if (!more) return;
    __syncwarp();  // every lane is done with the stage before it is refilled
    task = next;
    index = next_index;
    start(task);
  }
}

// Merge pass of the tile schedules: combines the partials of every cut
// segment in slot order and writes out[seg].
//
// CTAs [0, record_ctas): one thread per record (the host planner lists the
// cut segments; the device planner writes one record per tile, empty where no
// segment begins a cut there).  A segment of up to kLaneMerge pieces is merged
// by its thread, up to kWarpMerge by its warp.
// CTAs [record_ctas, gridDim): the segments with more pieces than that, which
// the planners list apart (`bigs`, *big_count of them, a number only the
// device needs to know): a CTA each, every thread with up to sixteen
// partials in flight.
// Thread- or lane-strided partial results, then a butterfly, so the result
// does not depend on timing.  Launched with programmatic stream
// serialisation: its CTAs are placed and read their records (plan-owned
// memory) while the tile kernel drains, and wait for that kernel's partials
// to be visible before they read one.
constexpr int kMergeThreads = 512;

template <class Op, class R = NoPeers>
__global__ void __launch_bounds__(kMergeThreads)
segreduce_merge_kernel(const MergeRecord *__restrict__ records, int32_t count,
                       uint32_t record_ctas,
                       const MergeRecord *__restrict__ bigs,
                       const int32_t *__restrict__ big_count,
                       const typename Op::Acc *__restrict__ partials,
                       typename Op::Acc *__restrict__ out, Limits limits,
                       R peers) {
  using A = typename Op::Acc;
  __shared__ float scratch[32];
  // the next launch in the stream, if it is one of the tile kernels, may
  // place its CTAs and fetch its descriptors while this grid runs
  asm volatile("griddepcontrol.launch_dependents;");
  const int tid = threadIdx.x, lane = tid & 31;
  const int step = limits.slot_step;
  // a record that does not fit the launch's arrays is skipped, not followed
  auto fits = [&](const MergeRecord &r) {
    return r.pieces >= 2 && r.seg >= 0 && r.seg < limits.segment_count &&
           slots_ok(r.first, r.pieces, limits);
  };
  if (blockIdx.x < record_ctas) {
    const int64_t index = (int64_t)blockIdx.x * kMergeThreads + tid;
    MergeRecord r{0, 0, 0, 0};
    if (index < count) r = records[index];
    const bool valid = fits(r) && r.pieces <= kWarpMerge;
    const bool small = valid && r.pieces <= kLaneMerge;
    const bool medium = valid && !small;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // (all the loads of a segment are issued before the first is used: one
    // round trip to L2, where the partials were just written, per segment)
    if (small) {
      A q[kLaneMerge];
#pragma unroll
      for (int k = 0; k < kLaneMerge; ++k)
        if (k < r.pieces) q[k] = partials[piece_slot(r.first, k, step)];
      A acc = Op::identity();
#pragma unroll
      for (int k = 0; k < kLaneMerge; ++k)
        if (k < r.pieces) acc = Op::apply(acc, q[k]);
      peers.store(out, r.seg, acc);
    }
    unsigned waiting = __ballot_sync(kFullMask, medium);
    while (waiting) {
      const int src = __ffs(waiting) - 1;
      waiting &= waiting - 1;
      const int seg = __shfl_sync(kFullMask, r.seg, src);
      const int first = __shfl_sync(kFullMask, r.first, src);
      const int pieces = __shfl_sync(kFullMask, r.pieces, src);
      A q[kWarpMerge / 32];
#pragma unroll
      for (int u = 0; u < kWarpMerge / 32; ++u)
        if (lane + 32 * u < pieces)
          q[u] = partials[piece_slot(first, lane + 32 * u, step)];
      A acc = Op::identity();
#pragma unroll
      for (int u = 0; u < kWarpMerge / 32; ++u)
        if (lane + 32 * u < pieces) acc = Op::apply(acc, q[u]);
      acc = warp_reduce<Op>(acc);
      if (lane == 0) peers.store(out, seg, acc);
    }
  } else {
    const int total = bigs != nullptr ? *big_count : 0;
    const int stride = (int)(gridDim.x - record_ctas);
    int i = (int)(blockIdx.x - record_ctas);
    MergeRecord r{0, 0, 0, 0};
    if (i < total) r = bigs[i];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    while (i < total) {
      const bool valid = fits(r);  // uniform over the CTA
      const int first = r.first, pieces = valid ? r.pieces : 0;
      // sixteen partials per thread are requested before the first is
      // used: a segment of up to 16 * kMergeThreads pieces costs one round
      // trip to L2
      A a[4] = {Op::identity(), Op::identity(), Op::identity(),
                Op::identity()};
      for (int k = tid; k < pieces; k += 16 * kMergeThreads) {
        A q[16];
#pragma unroll
        for (int u = 0; u < 16; ++u)
          if (k + u * kMergeThreads < pieces)
            q[u] = partials[piece_slot(first, k + u * kMergeThreads, step)];
#pragma unroll
        for (int u = 0; u < 16; ++u)
          if (k + u * kMergeThreads < pieces)
            a[u & 3] = Op::apply(a[u & 3], q[u]);
      }
      const A mine =
          Op::apply(Op::apply(a[0], a[1]), Op::apply(a[2], a[3]));
      const A v = cta_reduce<Op>(mine, scratch);
      if (tid == 0 && valid) peers.store(out, r.seg, v);
      i += stride;
      if (i < total) r = bigs[i];
    }
  }
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
constexpr int kSplitBytes = kSplitWarps * kStageBytes;
#ifndef SWG_SPLIT_CTAS_PER_SM
#define SWG_SPLIT_CTAS_PER_SM 12  // residency of the split kernel (shared memory)
#endif

static Limits limits_of(const DevicePlan &plan, int32_t value_count) {
  return Limits{value_count, plan.segment_count, plan.partial_slots,
                plan.slot_step};
}

template <class Op, int kWarps, int kStages>
static cudaError_t persistent_launch(const float *values, float *out,
                                     int32_t value_count,
                                     const DevicePlan &plan,
                                     cudaStream_t stream, bool configure) {
  constexpr int kBytes = kWarps * kStages * kStageBytes;
  static_assert(kBytes + 8 * kWarps * kStages +
                        (int)sizeof(WarpScratch) * kWarps <= 227 * 1024,
                "rings exceed shared memory");
  if (configure)
    return cudaFuncSetAttribute(
        segreduce_persistent_kernel<Op, kWarps, kStages>,
        cudaFuncAttributeMaxDynamicSharedMemorySize, kBytes);
  int grid = plan.sm_count;
  const int needed = (plan.task_count + kWarps - 1) / kWarps;
  if (grid > needed) grid = needed;
  segreduce_persistent_kernel<Op, kWarps, kStages>
      <<<grid, kWarps * 32, kBytes, stream>>>(
          values, out, value_count, plan.tasks, plan.task_count, plan.offsets,
          plan.partials, plan.control, limits_of(plan, value_count));
  return cudaGetLastError();
}

template <class Op>
static cudaError_t persistent_dispatch(const float *values, float *out,
                                       int32_t value_count,
                                       const DevicePlan &plan,
                                       cudaStream_t stream, bool configure) {
  return persistent_launch<Op, 9, 3>(values, out, value_count, plan, stream,
                                     configure);
}

#ifndef SWG_RESIDENT_WARPS
#define SWG_RESIDENT_WARPS 26
#endif
constexpr int kResidentWarps = SWG_RESIDENT_WARPS;
static_assert(kResidentWarps * (kStageBytes + (int)sizeof(WarpScratch) + 8) <=
                  227 * 1024,
              "stages of the resident kernel exceed shared memory");

// Calls f with the operator type of `kind` (f is a generic lambda).
template <class F>
static cudaError_t with_op(int kind, F &&f) {
  switch (kind) {
    case SWG_KIND_SUM: return f(SumOp{});
    case SWG_KIND_MAX: return f(MaxOp{});
    default: return f(MinOp{});
  }
}

// Calls f with the operator and element types of (kind, dtype).
template <class F>
static cudaError_t with_types(int kind, int dtype, F &&f) {
  switch (dtype) {
    case SWG_DTYPE_F16:
      return with_op(kind, [&](auto op) { return f(op, __half{}); });
    case SWG_DTYPE_BF16:
      return with_op(kind, [&](auto op) { return f(op, __nv_bfloat16{}); });
    case SWG_DTYPE_I32:
      switch (kind) {
        case SWG_KIND_SUM: return f(ISumOp{}, int32_t{});
        case SWG_KIND_MAX: return f(IMaxOp{}, int32_t{});
        default: return f(IMinOp{}, int32_t{});
      }
    default:
      return with_op(kind, [&](auto op) { return f(op, float{}); });
  }
}

// Calls f with the operator, element and map types of (kind, dtype, map).
// Maps exist for the floating element types only.
template <class F>
static cudaError_t with_map(int kind, int dtype, const swg_map *map, F &&f) {
  if (!map || dtype == SWG_DTYPE_I32)
    return with_types(kind, dtype, [&](auto op, auto element) {
      return f(op, element, NoMap{});
    });
  const ScalarMap m{map->fn, map->scale, map->shift};
  switch (dtype) {
    case SWG_DTYPE_F16:
      return with_op(kind, [&](auto op) { return f(op, __half{}, m); });
    case SWG_DTYPE_BF16:
      return with_op(kind, [&](auto op) { return f(op, __nv_bfloat16{}, m); });
    default:
      return with_op(kind, [&](auto op) { return f(op, float{}, m); });
  }
}

cudaError_t configure_segreduce_kernels() {
  DevicePlan none;
  for (int kind : {SWG_KIND_SUM, SWG_KIND_MAX, SWG_KIND_MIN}) {
    cudaError_t e = with_op(kind, [&](auto op) {
      return persistent_dispatch<decltype(op)>(nullptr, nullptr, 0, none,
                                               nullptr, true);
    });
    if (e != cudaSuccess) return e;
    const swg_map some_map{SWG_MAP_IDENTITY, 1.0f, 0.0f};
    for (int dtype : {SWG_DTYPE_F32, SWG_DTYPE_F16, SWG_DTYPE_BF16,
                      SWG_DTYPE_I32}) {
      for (const swg_map *map : {(const swg_map *)nullptr, &some_map}) {
        if (map && dtype == SWG_DTYPE_I32) continue;
        e = with_map(kind, dtype, map, [&](auto op, auto element, auto m) {
          using Op = decltype(op);
          using T = decltype(element);
          using M = decltype(m);
          const cudaError_t inner = cudaFuncSetAttribute(
              segreduce_resident_kernel<Op, T, kResidentWarps, M>,
              cudaFuncAttributeMaxDynamicSharedMemorySize,
              kResidentWarps * kStageBytes);
          if (inner != cudaSuccess) return inner;
          return cudaFuncSetAttribute(
              segreduce_split_kernel<Op, T, M>,
              cudaFuncAttributeMaxDynamicSharedMemorySize, kSplitBytes);
        });
        if (e != cudaSuccess) return e;
      }
    }
    e = with_op(kind, [&](auto op) {
      using Op = decltype(op);
      const cudaError_t inner = cudaFuncSetAttribute(
          segreduce_resident_kernel<Op, float, kResidentWarps, NoMap, PeerOut>,
          cudaFuncAttributeMaxDynamicSharedMemorySize,
          kResidentWarps * kStageBytes);
      if (inner != cudaSuccess) return inner;
      return cudaFuncSetAttribute(
          segreduce_split_kernel<Op, float, NoMap, PeerOut>,
          cudaFuncAttributeMaxDynamicSharedMemorySize, kSplitBytes);
    });
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// A tile kernel launched with programmatic stream serialisation: it may be
// placed while the kernel before it in the stream drains (see the kernels).
template <class Kernel, class... Args>
static cudaError_t launch_serialised(Kernel kernel, unsigned grid,
                                     unsigned block, size_t shared,
                                     cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(block);
  config.dynamicSmemBytes = shared;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, args...);
}

// Plan-free launch for the element types other than f32.
cudaError_t launch_segreduce_typed(int kind, int dtype, const void *values,
                                   const int32_t *offsets, void *out,
                                   int32_t value_count, int32_t segment_count,
                                   bool cta, int sm_count, cudaStream_t stream,
                                   const Probe *probe, const swg_map *map) {
  const int per_cta = cta ? 1 : kWarpKernelThreads / 32;
  int64_t grid = ((int64_t)segment_count + per_cta - 1) / per_cta;
  const int64_t cap = (int64_t)sm_count * 8 * 4;
  if (grid > cap) grid = cap;
  probe_begin(probe, stream);
  const cudaError_t e =
      with_map(kind, dtype, map, [&](auto op, auto element, auto m) {
        using Op = decltype(op);
        using T = decltype(element);
        using M = decltype(m);
        using A = typename Op::Acc;
        if (cta)
          segreduce_typed_kernel<Op, T, true, M>
              <<<(unsigned)grid, kWarpKernelThreads, 0, stream>>>(
                  static_cast<const T *>(values), offsets,
                  static_cast<A *>(out), segment_count, m);
        else
          segreduce_typed_kernel<Op, T, false, M>
              <<<(unsigned)grid, kWarpKernelThreads, 0, stream>>>(
                  static_cast<const T *>(values), offsets,
                  static_cast<A *>(out), segment_count, m);
        return cudaGetLastError();
      });
  probe_end(probe, stream);
  (void)value_count;
  return e;
}

cudaError_t launch_segreduce_warp(int kind, const float *values,
                                  const int32_t *offsets, float *out,
                                  int32_t segment_count, int sm_count,
                                  cudaStream_t stream, const Probe *probe) {
  const int warps_per_cta = kWarpKernelThreads / 32;
  int64_t grid = ((int64_t)segment_count + warps_per_cta - 1) / warps_per_cta;
  const int64_t cap = (int64_t)sm_count * 8 * 4;
  if (grid > cap) grid = cap;
  probe_begin(probe, stream);
  const cudaError_t e = with_op(kind, [&](auto op) {
    return launch_serialised(segreduce_warp_kernel<decltype(op)>,
                             (unsigned)grid, kWarpKernelThreads, 0, stream,
                             values, offsets, out, segment_count);
  });
  probe_end(probe, stream);
  return e;
}

cudaError_t launch_segreduce_sum_max(const float *values,
                                     const int32_t *offsets, float *out_sum,
                                     float *out_max, int32_t value_count,
                                     int32_t segment_count, int sm_count,
                                     cudaStream_t stream, const Probe *probe) {
  // long segments on average: a CTA each; else a warp each
  const bool cta = (int64_t)value_count >= (int64_t)segment_count * 2048;
  const int per_cta = cta ? 1 : kWarpKernelThreads / 32;
  int64_t grid = ((int64_t)segment_count + per_cta - 1) / per_cta;
  const int64_t cap = (int64_t)sm_count * 8 * 4;
  if (grid > cap) grid = cap;
  probe_begin(probe, stream);
  const cudaError_t e =
      cta ? launch_serialised(segreduce_sum_max_kernel<true>, (unsigned)grid,
                              kWarpKernelThreads, 0, stream, values, offsets,
                              out_sum, out_max, segment_count)
          : launch_serialised(segreduce_sum_max_kernel<false>, (unsigned)grid,
                              kWarpKernelThreads, 0, stream, values, offsets,
                              out_sum, out_max, segment_count);
  probe_end(probe, stream);
  return e;
}

cudaError_t launch_segreduce_cta(int kind, const float *values,
                                 const int32_t *offsets, float *out,
                                 int32_t segment_count, int32_t block,
                                 int sm_count, cudaStream_t stream,
                                 const Probe *probe) {
  if (block <= 0) block = 256;
  block = ((block + 31) / 32) * 32;
  if (block > 1024) block = 1024;
  int64_t grid = segment_count;
  const int64_t cap = (int64_t)sm_count * (2048 / block) * 4;
  if (grid > cap) grid = cap;
  probe_begin(probe, stream);
  const cudaError_t e = with_op(kind, [&](auto op) {
    segreduce_cta_kernel<decltype(op)><<<(unsigned)grid, block, 0, stream>>>(
        values, offsets, out, segment_count);
    return cudaGetLastError();
  });
  probe_end(probe, stream);
  return e;
}

static cudaError_t launch_merge(int kind, int dtype, const DevicePlan &plan,
                                void *out, int32_t value_count,
                                cudaStream_t stream,
                                const PeerOut *peers = nullptr) {
  if (plan.merge_count == 0 && plan.big_capacity == 0) return cudaSuccess;
  const unsigned record_ctas =
      (unsigned)(((int64_t)plan.merge_count + kMergeThreads - 1) /
                 kMergeThreads);
  // a CTA per listed long segment, as many as the list can hold but no more
  // than two rounds of the machine (they loop over the list)
  int big_ctas = plan.big_capacity;
  if (big_ctas > 2 * plan.sm_count) big_ctas = 2 * plan.sm_count;
  // (the accumulator type decides: f16 / bf16 values merge as fp32)
  const int acc_dtype = dtype == SWG_DTYPE_I32 ? SWG_DTYPE_I32 : SWG_DTYPE_F32;
  if (peers)  // fp32 results stored into every GPU's copy
    return with_op(kind, [&](auto op) {
      using Op = decltype(op);
      return launch_serialised(
          segreduce_merge_kernel<Op, PeerOut>, record_ctas + (unsigned)big_ctas,
          kMergeThreads, 0, stream, (const MergeRecord *)plan.merges,
          plan.merge_count, record_ctas, (const MergeRecord *)plan.bigs,
          (const int32_t *)plan.big_count, (const float *)plan.partials,
          static_cast<float *>(out), limits_of(plan, value_count), *peers);
    });
  return with_types(kind, acc_dtype, [&](auto op, auto) {
    using Op = decltype(op);
    using A = typename Op::Acc;
    return launch_serialised(
        segreduce_merge_kernel<Op>, record_ctas + (unsigned)big_ctas,
        kMergeThreads, 0, stream, (const MergeRecord *)plan.merges,
        plan.merge_count, record_ctas, (const MergeRecord *)plan.bigs,
        (const int32_t *)plan.big_count,
        reinterpret_cast<const A *>(plan.partials), static_cast<A *>(out),
        limits_of(plan, value_count), NoPeers{});
  });
}

cudaError_t launch_segreduce_split(int kind, int dtype, const void *values,
                                   void *out, int32_t value_count,
                                   const DevicePlan &plan, cudaStream_t stream,
                                   const Probe *probe, const swg_map *map,
                                   const PeerOut *peers) {
  if (plan.task_count == 0) return cudaSuccess;
  const unsigned grid =
      (unsigned)((plan.task_count + kSplitWarps - 1) / kSplitWarps);
  const uint32_t first_wave =
      (uint32_t)plan.sm_count * SWG_SPLIT_CTAS_PER_SM;
  probe_begin(probe, stream);
  cudaError_t e;
  if (peers)  // f32, unmapped (checked by the caller)
    e = with_op(kind, [&](auto op) {
      using Op = decltype(op);
      return launch_serialised(
          segreduce_split_kernel<Op, float, NoMap, PeerOut>, grid,
          kSplitWarps * 32, kSplitBytes, stream,
          static_cast<const float *>(values), static_cast<float *>(out),
          value_count, (const Task *)plan.tasks, plan.task_count,
          (const int32_t *)plan.offsets, plan.partials, plan.control,
          limits_of(plan, value_count), first_wave, NoMap{}, *peers);
    });
  else
    e = with_map(kind, dtype, map, [&](auto op, auto element, auto m) {
      using Op = decltype(op);
      using T = decltype(element);
      using M = decltype(m);
      using A = typename Op::Acc;
      return launch_serialised(
          segreduce_split_kernel<Op, T, M>, grid, kSplitWarps * 32,
          kSplitBytes, stream, static_cast<const T *>(values),
          static_cast<A *>(out), value_count, (const Task *)plan.tasks,
          plan.task_count, (const int32_t *)plan.offsets,
          reinterpret_cast<A *>(plan.partials), plan.control,
          limits_of(plan, value_count), first_wave, m, NoPeers{});
    });
  probe_end(probe, stream);
  if (e != cudaSuccess) return e;
  return launch_merge(kind, dtype, plan, out, value_count, stream, peers);
}

cudaError_t launch_segreduce_persistent(int kind, const float *values,
                                        float *out, int32_t value_count,
                                        const DevicePlan &plan,
                                        cudaStream_t stream,
                                        const Probe *probe) {
  if (plan.task_count == 0) return cudaSuccess;
  probe_begin(probe, stream);
  const cudaError_t e = with_op(kind, [&](auto op) {
    return persistent_dispatch<decltype(op)>(values, out, value_count, plan,
                                             stream, false);
  });
  probe_end(probe, stream);
  if (e != cudaSuccess) return e;
  return launch_merge(kind, SWG_DTYPE_F32, plan, out, value_count, stream);
}

cudaError_t launch_segreduce_resident(int kind, int dtype, const void *values,
                                      void *out, int32_t value_count,
                                      const DevicePlan &plan,
                                      cudaStream_t stream, const Probe *probe,
                                      const swg_map *map,
                                      const PeerOut *peers) {
  if (plan.task_count == 0) return cudaSuccess;
  int grid = plan.sm_count;
  const int needed = (plan.task_count + kResidentWarps - 1) / kResidentWarps;
  if (grid > needed) grid = needed;
  probe_begin(probe, stream);
  cudaError_t e;
  if (peers)  // f32, unmapped (checked by the caller)
    e = with_op(kind, [&](auto op) {
      using Op = decltype(op);
      return launch_serialised(
          segreduce_resident_kernel<Op, float, kResidentWarps, NoMap, PeerOut>,
          (unsigned)grid, kResidentWarps * 32,
          (size_t)kResidentWarps * kStageBytes, stream,
          static_cast<const float *>(values), static_cast<float *>(out),
          value_count, (const Task *)plan.tasks, plan.task_count,
          (const int32_t *)plan.offsets, plan.partials, plan.control,
          limits_of(plan, value_count), NoMap{}, *peers);
    });
  else
    e = with_map(kind, dtype, map, [&](auto op, auto element, auto m) {
      using Op = decltype(op);
      using T = decltype(element);
      using M = decltype(m);
      using A = typename Op::Acc;
      return launch_serialised(
          segreduce_resident_kernel<Op, T, kResidentWarps, M>, (unsigned)grid,
          kResidentWarps * 32, (size_t)kResidentWarps * kStageBytes, stream,
          static_cast<const T *>(values), static_cast<A *>(out), value_count,
          (const Task *)plan.tasks, plan.task_count,
          (const int32_t *)plan.offsets,
          reinterpret_cast<A *>(plan.partials), plan.control,
          limits_of(plan, value_count), m, NoPeers{});
    });
  probe_end(probe, stream);
  if (e != cudaSuccess) return e;
  return launch_merge(kind, dtype, plan, out, value_count, stream, peers);
}

// ---------------------------------------------------------------------------
// Self-test of the bounded wait: one warp arms an mbarrier for sixteen bytes
// that no copy will ever deliver, waits for at most `limit_ns`, and -- the
// wait having run out -- reports kErrTimeout through the plan's error words
// exactly as the tile kernels do, then returns.  Touches no caller memory.
// ---------------------------------------------------------------------------
__global__ void wait_selftest_kernel(uint32_t *control,
                                     unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  const int lane = threadIdx.x & 31;
  if (lane == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncwarp();
  if (lane == 0) mbar_arrive_expect_tx(&bar, 16);
  __syncwarp();
  if (!mbar_wait_for(&bar, 0, limit_ns) && lane == 0)
    report(control, kErrTimeout, 0xfeedu);
}

cudaError_t launch_wait_selftest(const DevicePlan &plan, uint64_t limit_ns,
                                 cudaStream_t stream) {
  wait_selftest_kernel<<<1, 32, 0, stream>>>(plan.control, limit_ns);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the split schedule.
//
// Everything the split schedule normally keeps in plan-owned device memory
// (task list, aligned offsets copy, the list of cut segments, their partials,
// control words) lives instead in one file-scope device array of fixed size,
// so the call path contains no cudaMalloc / cudaFree.  Every GPU that loads
// this library holds the array (kStaticBytes = 2,490,880 bytes, about 2.5 MB)
// until the process exits.
//
// The array's name is only a host-side handle: the address kernels can use is
// obtained once per device with cudaGetSymbolAddress, with that device
// current, the first time the entry point runs there.
// ---------------------------------------------------------------------------
constexpr size_t round256(size_t bytes) { return (bytes + 255) / 256 * 256; }
constexpr size_t kStaticOffsetBytes =
    round256(((size_t)kStaticMaxSegments + 8) * 4);
constexpr size_t kStaticTaskBytes = (size_t)kStaticMaxTasks * sizeof(Task);
// a cut segment has at least two partials; the long ones (more than
// kWarpMerge) are listed behind the others, the count of them last
constexpr size_t kStaticMergeBytes =
    (size_t)(kStaticMaxSlots / 2) * sizeof(MergeRecord);
constexpr int kStaticMaxBigs = kStaticMaxSlots / kWarpMerge;
constexpr size_t kStaticPartialBytes = (size_t)kStaticMaxSlots * 4;
constexpr size_t kStaticControlBytes = 256;
static_assert(kStaticControlBytes >= kControlWords * 4 + 4,
              "the count of long cut segments sits behind the control words");
constexpr size_t kStaticOffsetAt = 0;
constexpr size_t kStaticTaskAt = kStaticOffsetAt + kStaticOffsetBytes;
constexpr size_t kStaticMergeAt = kStaticTaskAt + kStaticTaskBytes;
constexpr size_t kStaticPartialAt = kStaticMergeAt + kStaticMergeBytes;
constexpr size_t kStaticControlAt = kStaticPartialAt + kStaticPartialBytes;
constexpr size_t kStaticBytes = kStaticControlAt + kStaticControlBytes;
static_assert(kStaticTaskAt % 256 == 0 && kStaticMergeAt % 256 == 0 &&
                  kStaticPartialAt % 256 == 0 && kStaticControlAt % 256 == 0,
              "regions of the static scratch keep 256-byte alignment");
static_assert(kStaticBytes == 2490880, "size quoted in the documentation");

static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

namespace {
std::mutex g_static_lock;
unsigned char *g_static_address[64] = {nullptr};
}  // namespace

// Device address of the static scratch on the current device (set up on the
// first call per device).
static cudaError_t static_scratch_address(int device, unsigned char **address) {
  std::lock_guard<std::mutex> guard(g_static_lock);
  if (g_static_address[device] == nullptr) {
    void *found = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&found, g_static_scratch);
    if (e != cudaSuccess) return e;
    g_static_address[device] = static_cast<unsigned char *>(found);
  }
  *address = g_static_address[device];
  return cudaSuccess;
}

cudaError_t launch_segreduce_static(int kind, const float *values, float *out,
                                    int32_t value_count,
                                    const int32_t *host_offsets,
                                    int32_t segment_count,
                                    const HostPlan &plan, int device,
                                    int sm_count, cudaStream_t stream) {
  unsigned char *base = nullptr;
  cudaError_t e = static_scratch_address(device, &base);
  if (e != cudaSuccess) return e;
  int32_t *d_off = reinterpret_cast<int32_t *>(base + kStaticOffsetAt);
  Task *d_tasks = reinterpret_cast<Task *>(base + kStaticTaskAt);
  MergeRecord *d_merges =
      reinterpret_cast<MergeRecord *>(base + kStaticMergeAt);
  uint32_t *d_control = reinterpret_cast<uint32_t *>(base + kStaticControlAt);

  const size_t noffsets = (size_t)segment_count + 1;
  const size_t padded = ((noffsets + 3) / 4) * 4 + 4;
  // The array keeps the previous call's contents: the padding after the
  // offsets and the control words are the parts that must start at zero.
  e = cudaMemsetAsync(d_off + noffsets, 0, (padded - noffsets) * 4, stream);
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(d_control, 0, kStaticControlBytes, stream);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyAsync(d_off, host_offsets, noffsets * 4,
                      cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyAsync(d_tasks, plan.tasks.data(),
                      plan.tasks.size() * sizeof(Task), cudaMemcpyHostToDevice,
                      stream);
  if (e != cudaSuccess) return e;
  // short and long cut segments share the region: the long ones fill it
  // from the end
  MergeRecord *d_bigs = d_merges + (kStaticMaxSlots / 2 - kStaticMaxBigs);
  int32_t *d_big_count = reinterpret_cast<int32_t *>(d_control + kControlWords);
  if (!plan.merges.empty()) {
    e = cudaMemcpyAsync(d_merges, plan.merges.data(),
                        plan.merges.size() * sizeof(MergeRecord),
                        cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return e;
  }
  if (!plan.big_merges.empty()) {
    e = cudaMemcpyAsync(d_bigs, plan.big_merges.data(),
                        plan.big_merges.size() * sizeof(MergeRecord),
                        cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return e;
  }
  const int32_t big_total = (int32_t)plan.big_merges.size();
  e = cudaMemcpyAsync(d_big_count, &big_total, sizeof(big_total),
                      cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return e;
  DevicePlan dev;
  dev.device = device;
  dev.sm_count = sm_count;
  dev.tasks = d_tasks;
  dev.task_count = (int32_t)plan.tasks.size();
  dev.segment_count = segment_count;
  dev.offsets = d_off;
  dev.partials = reinterpret_cast<float *>(base + kStaticPartialAt);
  dev.partial_slots = plan.partial_slots;
  dev.slot_step = plan.slot_step;
  dev.merges = d_merges;
  dev.merge_count = (int32_t)plan.merges.size();
  dev.bigs = d_bigs;
  dev.big_count = d_big_count;
  dev.big_capacity = big_total;
  dev.control = d_control;
  return launch_segreduce_split(kind, SWG_DTYPE_F32, values, out, value_count,
                                dev, stream, nullptr);
}

}  // namespace swg
