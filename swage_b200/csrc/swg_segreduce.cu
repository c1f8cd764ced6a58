// Segmented sum / max over dense fp32 values addressed by CSR int32 offsets.
//
// Replaces the kernels the reference generates in
// lib/Conversion/SegmentedReduction/SegmentedReduction.cpp:185-283 (one
// 128-thread CTA per segment, block-stride scalar loads, gpu.all_reduce).
// Four schedules:
//
//   warp        one warp per segment, 128-bit loads straight from global
//   cta         one CTA per segment (the reference's own mapping, vectorised)
//   split       the plan's tile tasks, one per CTA; segments longer than a
//               tile are chunked into partials and merged by a second pass
//   persistent  the same tile tasks, drawn from a ticket counter by one
//               resident CTA per SM; a producer warp stages tiles into a
//               shared-memory ring with bulk async copies (TMA) while eight
//               consumer warps reduce the previous ones
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
constexpr int kWarpKernelThreads = 256;

template <class Op>
__global__ void __launch_bounds__(kWarpKernelThreads)
segreduce_warp_kernel(const float *__restrict__ values,
                      const int32_t *__restrict__ offsets,
                      float *__restrict__ out, int32_t segment_count) {
  const int lane = threadIdx.x & 31;
  const int64_t warp =
      ((int64_t)blockIdx.x * kWarpKernelThreads + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * kWarpKernelThreads) >> 5;
  for (int64_t seg = warp; seg < segment_count; seg += nwarps) {
    const int64_t begin = __ldg(offsets + seg);
    const int64_t end = __ldg(offsets + seg + 1);
    float acc = strided_partial<Op>(values, begin, end, lane, kWarp);
    acc = warp_reduce<Op>(acc);
    if (lane == 0) out[seg] = acc;
  }
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
// Tile tasks (split and persistent schedules)
// ---------------------------------------------------------------------------
constexpr int kConsumerThreads = 256;
constexpr int kConsumerWarps = kConsumerThreads / 32;
constexpr int kShortSegment = 32;  // reduced by a single thread inside a tile
constexpr int kLongListCap = 256;  // > kTileValues / (kShortSegment + 1)
constexpr int kTileFloats = kTileValues + 8;
constexpr int kTileOffsets = kTileMaxSegments + 8;
constexpr int kStageTileBytes = kTileFloats * 4;
constexpr int kStageOffsetBytes = kTileOffsets * 4;
constexpr int kStageBytes =
    ((kStageTileBytes + kStageOffsetBytes + 16 + 127) / 128) * 128;
constexpr uint32_t kTaskStop = 15u;  // sentinel kind: no more tasks
constexpr int kRingStages = 4;
constexpr int kTicketBatch = 4;

struct Stage {
  float *tile;
  int32_t *soff;
  Task *desc;
};

__device__ __forceinline__ Stage stage_at(unsigned char *base, int index) {
  unsigned char *p = base + (size_t)index * kStageBytes;
  Stage s;
  s.tile = reinterpret_cast<float *>(p);
  s.soff = reinterpret_cast<int32_t *>(p + kStageTileBytes);
  s.desc = reinterpret_cast<Task *>(p + kStageTileBytes + kStageOffsetBytes);
  return s;
}

struct Scratch {
  float red[32];
  int long_list[kLongListCap];
  int long_count;
};

__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

// Warp-collective: stage one task.  `mis` is the phase of the values pointer
// inside a 16-byte line, in elements.  The bulk copy takes every 16-byte line
// that intersects the task's value range and lies wholly inside the values
// array (neighbouring elements that ride along are never read); the at most
// three elements at either end of the array that no such line covers are
// fetched with plain loads.  Element i lands at tile[i - origin] with
// origin = vbegin - ((vbegin + mis) & 3).
__device__ __forceinline__ void issue_task(const Task &task,
                                           const float *__restrict__ values,
                                           int mis, int32_t value_count,
                                           const int32_t *__restrict__ d_off,
                                           Stage stage, uint64_t *full,
                                           int lane) {
  const uint32_t kind = task.vcount_kind >> 28;
  const int64_t vb = task.vbegin;
  const int64_t ve = vb + (int64_t)(task.vcount_kind & kTaskCountMask);
  const int64_t origin = vb - ((vb + mis) & 3);
  int64_t lo = origin < 0 ? origin + 4 : origin;
  int64_t hi = ve + ((4 - ((ve + mis) & 3)) & 3);
  const int64_t last_line = (int64_t)value_count - ((value_count + mis) & 3);
  if (hi > last_line) hi = last_line;
  if (hi < lo) hi = lo;

  int64_t idx = -1;
  if (lane < 8) idx = vb + lane;
  else if (lane < 16) idx = ve - 1 - (lane - 8);
  if (idx >= vb && idx < ve && (idx < lo || idx >= hi))
    stage.tile[idx - origin] = values[idx];

  uint32_t bytes_v = (uint32_t)(hi - lo) * 4u;
  uint32_t bytes_o = 0;
  int32_t o_lo = 0;
  if (kind == kTaskPack) {
    o_lo = task.seg & ~3;
    const int32_t o_hi = (task.seg + task.count + 1 + 3) & ~3;
    bytes_o = (uint32_t)(o_hi - o_lo) * 4u;
  }
  __syncwarp();
  if (lane == 0) {
    *stage.desc = task;
    mbar_arrive_expect_tx(full, bytes_v + bytes_o);
    if (bytes_v) bulk_g2s(stage.tile + (lo - origin), values + lo, bytes_v, full);
    if (bytes_o) bulk_g2s(stage.soff, d_off + o_lo, bytes_o, full);
  }
}

// Reduce one staged task with the kConsumerThreads consumer threads.
template <class Op>
__device__ __forceinline__ void process_task(const Stage &stage, int mis,
                                             float *__restrict__ out,
                                             float *__restrict__ partials,
                                             Scratch *scratch, int tid) {
  const Task task = *stage.desc;
  const uint32_t kind = task.vcount_kind >> 28;
  const int vcount = (int)(task.vcount_kind & kTaskCountMask);
  const int shift = (int)(((int64_t)task.vbegin + mis) & 3);
  const float *tile = stage.tile;
  const int lane = tid & 31, warp = tid >> 5;

  if (kind == kTaskChunk) {
    // One piece of a long segment: every consumer thread strides over it.
    const float *p = tile + shift;
    float a0 = Op::identity(), a1 = Op::identity(), a2 = Op::identity(),
          a3 = Op::identity();
    int i = tid;
    for (; i + 3 * kConsumerThreads < vcount; i += 4 * kConsumerThreads) {
      a0 = Op::apply(a0, p[i]);
      a1 = Op::apply(a1, p[i + kConsumerThreads]);
      a2 = Op::apply(a2, p[i + 2 * kConsumerThreads]);
      a3 = Op::apply(a3, p[i + 3 * kConsumerThreads]);
    }
    for (; i < vcount; i += kConsumerThreads) a0 = Op::apply(a0, p[i]);
    float acc = Op::apply(Op::apply(a0, a1), Op::apply(a2, a3));
    acc = warp_reduce<Op>(acc);
    if (lane == 0) scratch->red[warp] = acc;
    consumer_sync();
    if (warp == 0) {
      float r = lane < kConsumerWarps ? scratch->red[lane] : Op::identity();
      r = warp_reduce<Op>(r);
      if (lane == 0) {
        if (task.count < 0) out[task.seg] = r;
        else partials[task.count] = r;
      }
    }
    consumer_sync();  // red[] and the tile are free again
    return;
  }

  // Packed whole segments.  Tile-relative bounds of segment k are
  // soff[ob + k] - origin and soff[ob + k + 1] - origin.
  const int32_t *soff = stage.soff + (task.seg & 3);
  const int origin = task.vbegin - shift;
  if (tid == 0) scratch->long_count = 0;
  consumer_sync();
  for (int k = tid; k < task.count; k += kConsumerThreads) {
    const int a = soff[k] - origin, b = soff[k + 1] - origin;
    if (b - a <= kShortSegment) {
      float acc = Op::identity();
      for (int i = a; i < b; ++i) acc = Op::apply(acc, tile[i]);
      out[task.seg + k] = acc;
    } else {
      const int slot = atomicAdd(&scratch->long_count, 1);
      scratch->long_list[slot] = k;
    }
  }
  consumer_sync();
  const int nlong = scratch->long_count;
  for (int j = warp; j < nlong; j += kConsumerWarps) {
    const int k = scratch->long_list[j];
    const int a = soff[k] - origin, b = soff[k + 1] - origin;
    float a0 = Op::identity(), a1 = Op::identity();
    int i = a + lane;
    for (; i + 32 < b; i += 64) {
      a0 = Op::apply(a0, tile[i]);
      a1 = Op::apply(a1, tile[i + 32]);
    }
    if (i < b) a0 = Op::apply(a0, tile[i]);
    const float r = warp_reduce<Op>(Op::apply(a0, a1));
    if (lane == 0) out[task.seg + k] = r;
  }
  consumer_sync();  // long_list and the tile are free again
}

// split schedule: one task per CTA, single stage.
template <class Op>
__global__ void __launch_bounds__(kConsumerThreads)
segreduce_split_kernel(const float *__restrict__ values,
                       float *__restrict__ out, int32_t value_count,
                       const Task *__restrict__ tasks,
                       const int32_t *__restrict__ d_off,
                       float *__restrict__ partials,
                       uint32_t *__restrict__ control) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full;
  __shared__ Scratch scratch;
  const int tid = threadIdx.x;
  const int mis = (int)(((uintptr_t)values >> 2) & 3);
  Stage stage = stage_at(smem, 0);
  if (tid == 0) {
    mbar_init(&full, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (tid < 32) {
    const Task task = tasks[blockIdx.x];
    issue_task(task, values, mis, value_count, d_off, stage, &full, tid);
  }
  if (!mbar_wait(&full, 0)) {
    if (tid == 0) atomicExch(control + 2, 1u);
    return;
  }
  process_task<Op>(stage, mis, out, partials, &scratch, tid);
}

// persistent schedule.
//   warp kConsumerWarps (the last one) = producer: draws tickets in batches,
//   loads the task descriptors one batch ahead, and keeps the ring full.
//   warps 0..kConsumerWarps-1 = consumers.
// control[0] = next ticket, control[1] = CTAs that stopped drawing,
// control[2] = error flag.  The last CTA to stop resets [0] and [1] so the
// next launch starts from zero without a memset.
template <class Op>
__global__ void __launch_bounds__(kConsumerThreads + 32, 1)
segreduce_persistent_kernel(const float *__restrict__ values,
                            float *__restrict__ out, int32_t value_count,
                            const Task *__restrict__ tasks, int32_t task_count,
                            const int32_t *__restrict__ d_off,
                            float *__restrict__ partials,
                            uint32_t *__restrict__ control) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[kRingStages], empty[kRingStages];
  __shared__ Scratch scratch;
  const int tid = threadIdx.x;
  const int mis = (int)(((uintptr_t)values >> 2) & 3);
  if (tid == 0) {
    for (int s = 0; s < kRingStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    fence_mbar_init();
  }
  __syncthreads();

  if (tid >= kConsumerThreads) {
    // ---------------- producer warp ----------------
    const int lane = tid - kConsumerThreads;
    int stage = 0;
    uint32_t phase = 0;
    int armed = 0;  // stages armed and possibly not yet consumed
    bool ok = true;
    Task stop;
    stop.seg = 0;
    stop.count = 0;
    stop.vbegin = 0;
    stop.vcount_kind = kTaskStop << 28;

    auto draw = [&]() -> uint32_t {
      uint32_t t = 0;
      if (lane == 0) t = atomicAdd(control, (uint32_t)kTicketBatch);
      return __shfl_sync(kFullMask, t, 0);
    };
    auto fetch = [&](uint32_t base) -> Task {
      Task t = stop;
      const uint32_t mine = base + (uint32_t)lane;
      if (lane < kTicketBatch && mine < (uint32_t)task_count)
        t = tasks[mine];
      return t;
    };

    uint32_t base_next = draw();
    Task cur = fetch(base_next);
    base_next = draw();
    bool done = false;
    while (!done && ok) {
      const uint32_t base_after = draw();   // in flight during this batch
      const Task nxt = fetch(base_next);    // descriptors one batch ahead
      for (int j = 0; j < kTicketBatch; ++j) {
        Task task;
        task.seg = __shfl_sync(kFullMask, cur.seg, j);
        task.count = __shfl_sync(kFullMask, cur.count, j);
        task.vbegin = __shfl_sync(kFullMask, cur.vbegin, j);
        task.vcount_kind = __shfl_sync(kFullMask, cur.vcount_kind, j);
        if (!mbar_wait(&empty[stage], phase ^ 1u)) {
          ok = false;
          break;
        }
        Stage st = stage_at(smem, stage);
        if ((task.vcount_kind >> 28) == kTaskStop) {
          if (lane == 0) {
            *st.desc = task;
            mbar_arrive(&full[stage]);
          }
          done = true;
          break;
        }
        issue_task(task, values, mis, value_count, d_off, st, &full[stage],
                   lane);
        if (armed < kRingStages) ++armed;
        if (++stage == kRingStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      cur = nxt;
      base_next = base_after;
    }
    if (!ok) {
      // A wait gave up: flag it, then let the copies already in flight land
      // (bounded) before this CTA's shared memory can be handed on.
      if (lane == 0) atomicExch(control + 2, 1u);
      int s = stage;
      uint32_t ph = phase;
      for (int k = 0; k < armed; ++k) {
        if (--s < 0) {
          s = kRingStages - 1;
          ph ^= 1u;
        }
        mbar_wait(&full[s], ph);
      }
    }
    if (lane == 0) {
      __threadfence();
      const uint32_t finished = atomicAdd(control + 1, 1u);
      if (finished == gridDim.x - 1) {
        atomicExch(control, 0u);
        atomicExch(control + 1, 0u);
      }
    }
    return;
  }

  // ---------------- consumer warps ----------------
  int stage = 0;
  uint32_t phase = 0;
  for (;;) {
    if (!mbar_wait(&full[stage], phase)) {
      if (tid == 0) atomicExch(control + 2, 1u);
      return;
    }
    Stage st = stage_at(smem, stage);
    if ((st.desc->vcount_kind >> 28) == kTaskStop) break;
    process_task<Op>(st, mis, out, partials, &scratch, tid);
    // process_task ends on a consumer barrier: every read of the stage is done
    if (tid == 0) mbar_arrive(&empty[stage]);
    if (++stage == kRingStages) {
      stage = 0;
      phase ^= 1u;
    }
  }
}

// Second pass of the split / persistent schedules: merge the partials of each
// chunked segment in slot order (fixed tree: lane-strided, then butterfly).
template <class Op>
__global__ void __launch_bounds__(256)
segreduce_combine_kernel(const SplitSegment *__restrict__ splits,
                         int32_t split_count,
                         const float *__restrict__ partials,
                         float *__restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t j = warp; j < split_count; j += nwarps) {
    const SplitSegment s = splits[j];
    float acc = Op::identity();
    for (int i = lane; i < s.slot_count; i += 32)
      acc = Op::apply(acc, partials[s.slot_begin + i]);
    acc = warp_reduce<Op>(acc);
    if (lane == 0) out[s.seg] = acc;
  }
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
cudaError_t configure_segreduce_kernels() {
  cudaError_t e;
  e = cudaFuncSetAttribute(segreduce_persistent_kernel<SumOp>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kRingStages * kStageBytes);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(segreduce_persistent_kernel<MaxOp>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kRingStages * kStageBytes);
  if (e != cudaSuccess) return e;
  e = cudaFuncSetAttribute(segreduce_split_kernel<SumOp>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kStageBytes);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(segreduce_split_kernel<MaxOp>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize,
                              kStageBytes);
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
  if (kind == SWG_KIND_SUM)
    segreduce_warp_kernel<SumOp><<<(unsigned)grid, kWarpKernelThreads, 0,
                                   stream>>>(values, offsets, out,
                                             segment_count);
  else
    segreduce_warp_kernel<MaxOp><<<(unsigned)grid, kWarpKernelThreads, 0,
                                   stream>>>(values, offsets, out,
                                             segment_count);
  probe_end(probe, stream);
  return cudaGetLastError();
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
  if (kind == SWG_KIND_SUM)
    segreduce_cta_kernel<SumOp><<<(unsigned)grid, block, 0, stream>>>(
        values, offsets, out, segment_count);
  else
    segreduce_cta_kernel<MaxOp><<<(unsigned)grid, block, 0, stream>>>(
        values, offsets, out, segment_count);
  probe_end(probe, stream);
  return cudaGetLastError();
}

static cudaError_t launch_combine(int kind, const DevicePlan &plan, float *out,
                                  cudaStream_t stream) {
  if (plan.split_count == 0) return cudaSuccess;
  int64_t grid = ((int64_t)plan.split_count + 7) / 8;
  const int64_t cap = (int64_t)plan.sm_count * 8;
  if (grid > cap) grid = cap;
  if (kind == SWG_KIND_SUM)
    segreduce_combine_kernel<SumOp><<<(unsigned)grid, 256, 0, stream>>>(
        plan.splits, plan.split_count, plan.partials, out);
  else
    segreduce_combine_kernel<MaxOp><<<(unsigned)grid, 256, 0, stream>>>(
        plan.splits, plan.split_count, plan.partials, out);
  return cudaGetLastError();
}

cudaError_t launch_segreduce_split(int kind, const float *values, float *out,
                                   int32_t value_count, const DevicePlan &plan,
                                   cudaStream_t stream, const Probe *probe) {
  if (plan.task_count == 0) return cudaSuccess;
  probe_begin(probe, stream);
  if (kind == SWG_KIND_SUM)
    segreduce_split_kernel<SumOp>
        <<<(unsigned)plan.task_count, kConsumerThreads, kStageBytes, stream>>>(
            values, out, value_count, plan.tasks, plan.offsets, plan.partials,
            plan.control);
  else
    segreduce_split_kernel<MaxOp>
        <<<(unsigned)plan.task_count, kConsumerThreads, kStageBytes, stream>>>(
            values, out, value_count, plan.tasks, plan.offsets, plan.partials,
            plan.control);
  probe_end(probe, stream);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  return launch_combine(kind, plan, out, stream);
}

cudaError_t launch_segreduce_persistent(int kind, const float *values,
                                        float *out, int32_t value_count,
                                        const DevicePlan &plan,
                                        cudaStream_t stream,
                                        const Probe *probe) {
  if (plan.task_count == 0) return cudaSuccess;
  int grid = plan.sm_count;
  if (grid > plan.task_count) grid = plan.task_count;
  const size_t smem = (size_t)kRingStages * kStageBytes;
  probe_begin(probe, stream);
  if (kind == SWG_KIND_SUM)
    segreduce_persistent_kernel<SumOp>
        <<<grid, kConsumerThreads + 32, smem, stream>>>(
            values, out, value_count, plan.tasks, plan.task_count, plan.offsets,
            plan.partials, plan.control);
  else
    segreduce_persistent_kernel<MaxOp>
        <<<grid, kConsumerThreads + 32, smem, stream>>>(
            values, out, value_count, plan.tasks, plan.task_count, plan.offsets,
            plan.partials, plan.control);
  probe_end(probe, stream);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  return launch_combine(kind, plan, out, stream);
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the split schedule.
//
// Everything the split schedule normally keeps in plan-owned cudaMalloc memory
// (task list, aligned offsets copy, split-segment list, partials, control
// words) lives instead in one file-scope device array of fixed size, so the
// call path contains no cudaMalloc / cudaFree.  Every GPU that loads this
// library holds the array (about 1.8 MB) until the process exits.
//
// The array's name is only a host-side handle: the address kernels can use is
// obtained once per device with cudaGetSymbolAddress, with that device
// current, the first time the entry point runs there.
// ---------------------------------------------------------------------------
constexpr size_t round256(size_t bytes) { return (bytes + 255) / 256 * 256; }
constexpr size_t kStaticOffsetBytes =
    round256(((size_t)kStaticMaxSegments + 8) * 4);
constexpr size_t kStaticTaskBytes = (size_t)kStaticMaxTasks * sizeof(Task);
constexpr size_t kStaticSplitBytes =
    (size_t)kStaticMaxSplits * sizeof(SplitSegment);
constexpr size_t kStaticPartialBytes = (size_t)kStaticMaxSlots * 4;
constexpr size_t kStaticControlBytes = 256;
constexpr size_t kStaticOffsetAt = 0;
constexpr size_t kStaticTaskAt = kStaticOffsetAt + kStaticOffsetBytes;
constexpr size_t kStaticSplitAt = kStaticTaskAt + kStaticTaskBytes;
constexpr size_t kStaticPartialAt = kStaticSplitAt + kStaticSplitBytes;
constexpr size_t kStaticControlAt = kStaticPartialAt + kStaticPartialBytes;
constexpr size_t kStaticBytes = kStaticControlAt + kStaticControlBytes;
static_assert(kStaticTaskAt % 256 == 0 && kStaticSplitAt % 256 == 0 &&
                  kStaticPartialAt % 256 == 0 && kStaticControlAt % 256 == 0,
              "regions of the static scratch keep 256-byte alignment");

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
  SplitSegment *d_splits =
      reinterpret_cast<SplitSegment *>(base + kStaticSplitAt);
  float *d_partials = reinterpret_cast<float *>(base + kStaticPartialAt);
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
  if (!plan.splits.empty()) {
    e = cudaMemcpyAsync(d_splits, plan.splits.data(),
                        plan.splits.size() * sizeof(SplitSegment),
                        cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return e;
  }
  DevicePlan dev;
  dev.device = device;
  dev.sm_count = sm_count;
  dev.tasks = d_tasks;
  dev.task_count = (int32_t)plan.tasks.size();
  dev.offsets = d_off;
  dev.splits = d_splits;
  dev.split_count = (int32_t)plan.splits.size();
  dev.partials = d_partials;
  dev.partial_slots = plan.partial_slots;
  dev.control = d_control;
  return launch_segreduce_split(kind, values, out, value_count, dev, stream,
                                nullptr);
}

}  // namespace swg
