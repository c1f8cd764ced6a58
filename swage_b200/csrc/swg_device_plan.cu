// Offsets validation and planning on the GPU: the offsets never leave the
// device.  The host reads back one small summary per validation (the first
// rule an offsets array breaks, in the order of the reference's host loop --
// python/swage/_segmented_qualification.py:30-55 -- plus a content hash, the
// last offset, the length histogram and the class counts); building a plan
// from validated offsets needs no further read-back.
//
// Reduce plan.  The host planner walks the segments one after the other; here
// every tile is found independently (merge-path): the sequence of items --
// per segment kHeaderItems header items, then its values -- is cut every
// kDeviceTile items, a binary search over p(s) = offsets[s] + kHeaderItems * s
// finds the segment each
// cut falls in, and a tile becomes one task of the same two kinds the host
// planner emits: a packed run of segments whose first and last may be pieces
// of segments that continue in the neighbouring tiles, or a chunk when the
// whole tile lies inside one segment.  A cut segment needs a partial slot per
// piece; tile t owns slots 2t (for the piece of a segment that began before
// it) and 2t + 1 (for the piece of a segment that goes on after it), so a
// segment whose header lies in tile t0 has its pieces at 2*t0 + 1, 2*(t0+1),
// 2*(t0+2), ...  The merge pass gets one record per tile: the segment that
// begins a cut there (none: an empty record).  Every tile derives all of this
// from the offsets alone -- no prefix sum, one kernel, nothing to bring to
// the host.
//
// Softmax plan.  A stable partition of the non-empty segments into the length
// classes (memory order inside a class): per-block class counts, a scan over
// the blocks, then every warp ranks its 32 segments with ballots.
#include <mutex>

#include "swg_common.cuh"
#include "swg_launch.h"

namespace swg {

namespace {

constexpr int kDeviceTile = kTileItems - 1;  // items per tile: values + count <= kTileItems
constexpr unsigned long long kNoViolation = ~0ull;

// Device -> host, written by the validation kernel.
struct Summary {
  unsigned long long first_bad;  // (index << 3) | rule, kNoViolation if none
  unsigned long long hash;       // of (index, offset) pairs
  long long histogram[kHistogramBins];
  long long elements[kHistogramBins];
  int softmax_count[kSoftmaxBuckets];
  int last_offset;
  int max_length;
};

// rules, in the order the host loop meets them at one index
constexpr unsigned kRuleStart = 0, kRuleNegative = 1, kRuleDecreasing = 2,
                   kRuleExceeds = 3;

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

__device__ __forceinline__ int device_length_bin(int length) {
  // 0 for an empty segment, else 2^(bin-1) <= length < 2^bin
  return length <= 0 ? 0 : 32 - __clz(length);
}

// kSoftmaxLimit for device code: the class of a non-empty segment
template <int k>
struct Limit {
  static constexpr int value = kSoftmaxLimit[k];
};
template <int k = 0>
__device__ __forceinline__ int device_bucket(int length) {
  if constexpr (k == kSoftmaxBuckets - 1) {
    return 0;
  } else {
    return (length > Limit<k>::value) + device_bucket<k + 1>(length);
  }
}

__global__ void __launch_bounds__(256)
summary_reset_kernel(Summary *summary) {
  const int i = threadIdx.x;
  if (i == 0) {
    summary->first_bad = kNoViolation;
    summary->hash = 0;
    summary->last_offset = 0;
    summary->max_length = 0;
  }
  if (i < kHistogramBins) {
    summary->histogram[i] = 0;
    summary->elements[i] = 0;
  }
  if (i < kSoftmaxBuckets) summary->softmax_count[i] = 0;
}

// One pass over offsets[0 .. segment_count]: the rules, the hash, the length
// statistics.
__global__ void __launch_bounds__(256)
validate_kernel(const int32_t *__restrict__ offsets, int32_t segment_count,
                int32_t value_count, Summary *summary) {
  __shared__ long long histogram[kHistogramBins];
  __shared__ long long elements[kHistogramBins];
  __shared__ int buckets[kSoftmaxBuckets];
  for (int i = threadIdx.x; i < kHistogramBins; i += blockDim.x) {
    histogram[i] = 0;
    elements[i] = 0;
  }
  if (threadIdx.x < kSoftmaxBuckets) buckets[threadIdx.x] = 0;
  __syncthreads();
  unsigned long long bad = kNoViolation, hash = 0;
  int longest = 0;
  const int lane = threadIdx.x & 31;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // whole warps walk together (the statistics are combined per warp)
  for (int64_t base = (int64_t)blockIdx.x * blockDim.x + (threadIdx.x & ~31);
       base <= segment_count; base += stride) {
    const int64_t i = base + lane;
    int bin = -1, bucket = -1, length = 0;
    if (i <= segment_count) {
      const int32_t o = __ldg(offsets + i);
      hash += mix64(((unsigned long long)i << 32) | (uint32_t)o);
      unsigned long long found = kNoViolation;
      if (i == 0 && o != 0) found = kRuleStart;  // before anything else
      else if (o < 0) found = ((unsigned long long)i << 3) | kRuleNegative;
      else if (i > 0 && o < __ldg(offsets + i - 1))
        found = ((unsigned long long)i << 3) | kRuleDecreasing;
      else if (i == segment_count && o > value_count)
        found = ((unsigned long long)i << 3) | kRuleExceeds;
      bad = found < bad ? found : bad;
      if (i == segment_count) {
        summary->last_offset = o;
      } else {
        const int64_t wide = (int64_t)__ldg(offsets + i + 1) - o;
        length = wide < 0 ? 0 : (int)wide;  // only read when valid
        bin = device_length_bin(length);
        if (length > 0) bucket = device_bucket(length);
        longest = length > longest ? length : longest;
      }
    }
    // lanes with the same bin add once
    const unsigned peers = __match_any_sync(kFullMask, bin);
    const unsigned together = __reduce_add_sync(peers, (unsigned)length);
    if (bin >= 0 && lane == __ffs(peers) - 1) {
      atomicAdd((unsigned long long *)&histogram[bin],
                (unsigned long long)__popc(peers));
      atomicAdd((unsigned long long *)&elements[bin],
                (unsigned long long)together);
    }
    const unsigned same = __match_any_sync(kFullMask, bucket);
    if (bucket >= 0 && lane == __ffs(same) - 1)
      atomicAdd(&buckets[bucket], __popc(same));
  }
  // warp-level combine, then one atomic per warp
  for (int delta = 16; delta > 0; delta >>= 1) {
    const unsigned long long other_bad = __shfl_xor_sync(kFullMask, bad, delta);
    bad = other_bad < bad ? other_bad : bad;
    hash += __shfl_xor_sync(kFullMask, hash, delta);
    const int other = __shfl_xor_sync(kFullMask, longest, delta);
    longest = other > longest ? other : longest;
  }
  if ((threadIdx.x & 31) == 0) {
    if (bad != kNoViolation) atomicMin(&summary->first_bad, bad);
    atomicAdd(&summary->hash, hash);
    atomicMax(&summary->max_length, longest);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kHistogramBins; i += blockDim.x) {
    if (histogram[i])
      atomicAdd((unsigned long long *)&summary->histogram[i],
                (unsigned long long)histogram[i]);
    if (elements[i])
      atomicAdd((unsigned long long *)&summary->elements[i],
                (unsigned long long)elements[i]);
  }
  if (threadIdx.x < kSoftmaxBuckets && buckets[threadIdx.x])
    atomicAdd(&summary->softmax_count[threadIdx.x], buckets[threadIdx.x]);
}

// ---------------------------------------------------------------------------
// reduce plan
// ---------------------------------------------------------------------------

// Item position of the first header item of segment s.
__device__ __forceinline__ int64_t header_at(const int32_t *offsets,
                                             int64_t s) {
  return (int64_t)__ldg(offsets + s) + kHeaderItems * s;
}

// The tile boundary at item d: the segment that item belongs to, whether the
// boundary cuts it (the item is not the first of its header: the segment began
// before d), and the first value at or behind the boundary.
struct Boundary {
  int32_t seg;
  bool cut;
  int64_t value;
};

__device__ __forceinline__ Boundary boundary_at(const int32_t *offsets,
                                                int32_t segment_count,
                                                int64_t d) {
  int64_t lo = 0, hi = (int64_t)segment_count - 1;  // header_at(lo) <= d
  while (lo < hi) {
    const int64_t mid = (lo + hi + 1) >> 1;
    if (header_at(offsets, mid) <= d) lo = mid;
    else hi = mid - 1;
  }
  const int64_t begin = __ldg(offsets + lo);
  const int64_t past_header = d - (begin + kHeaderItems * lo) - kHeaderItems;
  // a boundary inside the header leaves the whole segment behind it (its
  // piece before the boundary is empty)
  return Boundary{(int32_t)lo, d > begin + kHeaderItems * lo,
                  begin + (past_header > 0 ? past_header : 0)};
}

// Tile holding the first header item of segment s / its last value.
__device__ __forceinline__ int64_t first_tile(const int32_t *offsets,
                                              int64_t s) {
  return header_at(offsets, s) / kDeviceTile;
}
__device__ __forceinline__ int64_t last_tile(const int32_t *offsets,
                                             int64_t s) {
  return ((int64_t)__ldg(offsets + s + 1) + kHeaderItems * s +
          (kHeaderItems - 1)) /
         kDeviceTile;
}

// One thread per tile: its task and its merge record.  counts[0] += chunk
// tasks, counts[1] += cut segments (statistics only; one atomic per warp).
// A segment of more than kWarpMerge pieces spans more than kWarpMerge tiles,
// so there are fewer than tiles / kWarpMerge + 1 of them: the capacity of
// `bigs`.
__global__ void __launch_bounds__(256)
tile_plan_kernel(const int32_t *__restrict__ offsets, int32_t segment_count,
                 int32_t tile_count, Task *__restrict__ tasks,
                 MergeRecord *__restrict__ merges,
                 MergeRecord *__restrict__ bigs, int32_t big_capacity,
                 int32_t *__restrict__ big_count,
                 unsigned long long *__restrict__ counts) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  bool is_chunk = false, opens_cut = false;
  if (t < tile_count) {
    const int64_t d = t * kDeviceTile;
    const Boundary here = boundary_at(offsets, segment_count, d);
    const int32_t first = here.seg;
    const bool head_cut = here.cut;
    const int64_t vbegin = here.value;
    int32_t last;
    bool tail_cut;
    int64_t vend;
    if (t + 1 < tile_count) {
      const int64_t d1 = d + kDeviceTile;
      const Boundary next = boundary_at(offsets, segment_count, d1);
      tail_cut = next.cut;
      last = tail_cut ? next.seg : next.seg - 1;
      vend = next.value;
    } else {
      tail_cut = false;
      last = segment_count - 1;
      vend = __ldg(offsets + segment_count);
    }
    Task task;
    task.seg = first;
    task.vbegin = (int32_t)vbegin;
    if (first == last && head_cut && tail_cut) {
      // the whole tile lies inside one segment: piece t - t0 of it
      const int64_t t0 = first_tile(offsets, first);
      task.count = (int32_t)(2 * t);
      task.vcount_kind = (uint32_t)(vend - vbegin) | (kTaskChunk << 28);
      task.head_slot = task.tail_slot = -1;
      task.link_first = (int32_t)(2 * t0 + 1);
      task.link_pieces = (int32_t)(last_tile(offsets, first) - t0 + 1);
      is_chunk = true;
    } else {
      task.count = last - first + 1;
      task.vcount_kind = (uint32_t)(vend - vbegin) | (kTaskPack << 28);
      task.head_slot = head_cut ? (int32_t)(2 * t) : -1;
      task.tail_slot = tail_cut ? (int32_t)(2 * t + 1) : -1;
      task.link_first =
          head_cut ? (int32_t)(2 * first_tile(offsets, first) + 1) : -1;
      task.link_pieces =
          tail_cut ? (int32_t)(last_tile(offsets, last) - t + 1) : 0;
      opens_cut = tail_cut;
    }
    tasks[t] = task;
    MergeRecord record{0, 0, 0, 0};
    if (opens_cut) {
      record.seg = last;
      record.first = task.tail_slot;
      record.pieces = task.link_pieces;
      // the few segments of very many pieces are also listed apart: the
      // merge pass gives each of them a CTA (any order: they are independent)
      if (record.pieces > kWarpMerge) {
        const int32_t at = atomicAdd(big_count, 1);
        if (at < big_capacity) bigs[at] = record;
      }
    }
    merges[t] = record;
  }
  const unsigned chunks = __ballot_sync(kFullMask, is_chunk);
  const unsigned cuts = __ballot_sync(kFullMask, opens_cut);
  if ((threadIdx.x & 31) == 0) {
    if (chunks) atomicAdd(counts, (unsigned long long)__popc(chunks));
    if (cuts) atomicAdd(counts + 1, (unsigned long long)__popc(cuts));
  }
}

// ---------------------------------------------------------------------------
// softmax plan
// ---------------------------------------------------------------------------
constexpr int kListBlock = 1024;  // segments ranked by one warp
constexpr int kScanThreads = 1024;

struct BucketBegins {
  int32_t begin[kSoftmaxBuckets];
};

__device__ __forceinline__ int bucket_or_none(const int32_t *offsets,
                                              int64_t seg,
                                              int32_t segment_count) {
  if (seg >= segment_count) return -1;
  const int length = __ldg(offsets + seg + 1) - __ldg(offsets + seg);
  return length > 0 ? device_bucket(length) : -1;
}

// counts[bucket][block]: one warp per block of kListBlock segments
__global__ void __launch_bounds__(256)
bucket_count_kernel(const int32_t *__restrict__ offsets, int32_t segment_count,
                    int32_t blocks, int32_t *__restrict__ counts) {
  const int lane = threadIdx.x & 31;
  const int64_t block = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (block >= blocks) return;
  int mine[kSoftmaxBuckets] = {0};
  for (int i = lane; i < kListBlock; i += 32) {
    const int b = bucket_or_none(offsets, block * kListBlock + i, segment_count);
#pragma unroll
    for (int k = 0; k < kSoftmaxBuckets; ++k) mine[k] += b == k;
  }
#pragma unroll
  for (int k = 0; k < kSoftmaxBuckets; ++k) {
    int v = mine[k];
    for (int delta = 16; delta > 0; delta >>= 1)
      v += __shfl_xor_sync(kFullMask, v, delta);
    if (lane == 0) counts[(int64_t)k * blocks + block] = v;
  }
}

// exclusive scan over the blocks, in place: CTA k scans the row of bucket k
__global__ void __launch_bounds__(kScanThreads)
bucket_scan_kernel(int32_t blocks, int32_t *__restrict__ counts) {
  __shared__ int totals[kScanThreads];
  int32_t *row = counts + (int64_t)blockIdx.x * blocks;
  const int tid = threadIdx.x;
  const int64_t per = ((int64_t)blocks + kScanThreads - 1) / kScanThreads;
  const int64_t begin = tid * per;
  const int64_t end = begin + per < blocks ? begin + per : (int64_t)blocks;
  int sum = 0;
  for (int64_t i = begin; i < end; ++i) sum += row[i];
  totals[tid] = sum;
  __syncthreads();
  for (int delta = 1; delta < kScanThreads; delta <<= 1) {
    int a = 0;
    if (tid >= delta) a = totals[tid - delta];
    __syncthreads();
    totals[tid] += a;
    __syncthreads();
  }
  int running = totals[tid] - sum;
  for (int64_t i = begin; i < end; ++i) {
    const int n = row[i];
    row[i] = running;
    running += n;
  }
}

__global__ void __launch_bounds__(256)
bucket_fill_kernel(const int32_t *__restrict__ offsets, int32_t segment_count,
                   int32_t blocks, const int32_t *__restrict__ bases,
                   BucketBegins begins, int32_t *__restrict__ list) {
  const int lane = threadIdx.x & 31;
  const unsigned below = (1u << lane) - 1u;
  const int64_t block = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (block >= blocks) return;
  int32_t at[kSoftmaxBuckets];
#pragma unroll
  for (int k = 0; k < kSoftmaxBuckets; ++k)
    at[k] = begins.begin[k] + bases[(int64_t)k * blocks + block];
  for (int i = lane; i < kListBlock; i += 32) {
    const int64_t seg = block * kListBlock + i;
    const int b = bucket_or_none(offsets, seg, segment_count);
#pragma unroll
    for (int k = 0; k < kSoftmaxBuckets; ++k) {
      const unsigned votes = __ballot_sync(kFullMask, b == k);
      if (b == k) list[at[k] + __popc(votes & below)] = (int32_t)seg;
      at[k] += __popc(votes);
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
struct Scratch {
  bool ready = false;
  Summary *device = nullptr;
  Summary *host = nullptr;  // pinned
  // which array the summary in `host` describes (nullptr: none)
  const int32_t *seen_offsets = nullptr;
  int32_t seen_segments = 0;
  int32_t seen_values = 0;
};
std::mutex g_scratch_lock;
Scratch g_scratch[64];

cudaError_t scratch_for(int device, Scratch **out) {
  Scratch &s = g_scratch[device];
  if (!s.ready) {
    cudaError_t e = cudaMalloc((void **)&s.device, sizeof(Summary));
    if (e == cudaSuccess)
      e = cudaHostAlloc((void **)&s.host, sizeof(Summary), cudaHostAllocDefault);
    if (e != cudaSuccess) return e;
    s.ready = true;
  }
  *out = &s;
  return cudaSuccess;
}

int rule_to_reason(unsigned rule) {
  switch (rule) {
    case kRuleStart: return SWG_OFFSETS_NONZERO_START;
    case kRuleNegative: return SWG_OFFSETS_NEGATIVE;
    case kRuleDecreasing: return SWG_OFFSETS_DECREASING;
    default: return SWG_OFFSETS_EXCEEDS_VALUES;
  }
}

// Runs the validation pass and brings the summary to the host.  The caller
// holds g_scratch_lock.
cudaError_t summarise(const int32_t *offsets, int32_t segment_count,
                      int32_t value_count, int sm_count, cudaStream_t stream,
                      Scratch *scratch) {
  scratch->seen_offsets = nullptr;
  summary_reset_kernel<<<1, 256, 0, stream>>>(scratch->device);
  int64_t grid = ((int64_t)segment_count + 1 + 255) / 256;
  const int64_t cap = (int64_t)sm_count * 8;
  if (grid > cap) grid = cap;
  validate_kernel<<<(unsigned)grid, 256, 0, stream>>>(
      offsets, segment_count, value_count, scratch->device);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  e = cudaMemcpyAsync(scratch->host, scratch->device, sizeof(Summary),
                      cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return e;
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return e;
  scratch->seen_offsets = offsets;
  scratch->seen_segments = segment_count;
  scratch->seen_values = value_count;
  return cudaSuccess;
}

// Plan blocks come from the device's default stream-ordered pool, told once
// to keep what is freed: after the first plans a new one costs no cudaMalloc
// (and none of its implicit synchronisation).
bool g_pool_ready[64] = {false};
std::mutex g_pool_lock;

}  // namespace

cudaError_t plan_block_allocate(DevicePlan *dev, size_t bytes,
                                cudaStream_t stream) {
  {
    std::lock_guard<std::mutex> guard(g_pool_lock);
    if (!g_pool_ready[dev->device]) {
      cudaMemPool_t pool;
      cudaError_t e = cudaDeviceGetDefaultMemPool(&pool, dev->device);
      if (e != cudaSuccess) return e;
      unsigned long long keep = ~0ull;
      e = cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
      if (e != cudaSuccess) return e;
      g_pool_ready[dev->device] = true;
    }
  }
  dev->block = nullptr;
  dev->block_bytes = 0;
  if (bytes == 0) return cudaSuccess;
  const cudaError_t e = cudaMallocAsync(&dev->block, bytes, stream);
  if (e != cudaSuccess) return e;
  dev->block_bytes = bytes;
  dev->pooled = true;
  return cudaSuccess;
}

void plan_block_release(DevicePlan *dev, cudaStream_t after, bool ordered) {
  if (dev->block == nullptr) return;
  // stream-ordered behind the plan's last launch when every launch went to
  // one stream; otherwise (or if that stream is gone) a synchronising free
  cudaError_t e = cudaErrorUnknown;
  if (dev->pooled && ordered) e = cudaFreeAsync(dev->block, after);
  if (e != cudaSuccess) {
    cudaGetLastError();
    cudaFree(dev->block);
  }
  dev->block = nullptr;
  dev->block_bytes = 0;
}

cudaError_t device_validate(const int32_t *offsets, int32_t segment_count,
                            int32_t value_count, int device, int sm_count,
                            cudaStream_t stream, int32_t *reason,
                            int64_t *index, DeviceDigest *digest) {
  std::lock_guard<std::mutex> guard(g_scratch_lock);
  Scratch *scratch = nullptr;
  cudaError_t e = scratch_for(device, &scratch);
  if (e != cudaSuccess) return e;
  e = summarise(offsets, segment_count, value_count, sm_count, stream, scratch);
  if (e != cudaSuccess) return e;
  const Summary &s = *scratch->host;
  if (s.first_bad == kNoViolation) {
    *reason = SWG_OFFSETS_OK;
    *index = -1;
  } else {
    *reason = rule_to_reason((unsigned)(s.first_bad & 7u));
    *index = (int64_t)(s.first_bad >> 3);
  }
  if (digest) {
    digest->hash = s.hash;
    digest->last_offset = s.last_offset;
    digest->max_length = s.max_length;
  }
  return cudaSuccess;
}

namespace {

constexpr size_t aligned256(size_t bytes) { return (bytes + 255) / 256 * 256; }

// Carves the plan's block: padded offsets copy, control words (and the
// planner's two counters), tasks, merge records, partials.  What a launch
// expects to find at zero is cleared on `stream`; nothing here synchronises.
cudaError_t reduce_block(DevicePlan *dev, const int32_t *offsets,
                         int64_t tiles, cudaStream_t stream) {
  const size_t noffsets = (size_t)dev->segment_count + 1;
  const size_t padded = ((noffsets + 3) / 4) * 4 + 4;
  const size_t slots = (size_t)tiles * 2;
  const size_t offsets_bytes = aligned256(padded * sizeof(int32_t));
  const size_t control_bytes = aligned256(kControlWords * sizeof(uint32_t) +
                                          2 * sizeof(unsigned long long) +
                                          sizeof(int32_t));
  const size_t big_capacity = (size_t)tiles / kWarpMerge + 1;
  const size_t big_bytes = aligned256(big_capacity * sizeof(MergeRecord));
  const size_t task_bytes = aligned256((size_t)tiles * sizeof(Task));
  const size_t merge_bytes = aligned256((size_t)tiles * sizeof(MergeRecord));
  const size_t slot_bytes = aligned256(slots * sizeof(float));
  cudaError_t e = plan_block_allocate(
      dev,
      offsets_bytes + control_bytes + task_bytes + merge_bytes + big_bytes +
          slot_bytes,
      stream);
  if (e != cudaSuccess) return e;
  unsigned char *at = static_cast<unsigned char *>(dev->block);
  dev->offsets = reinterpret_cast<int32_t *>(at);
  at += offsets_bytes;
  dev->control = reinterpret_cast<uint32_t *>(at);
  dev->counts = reinterpret_cast<int64_t *>(dev->control + kControlWords);
  dev->big_count = reinterpret_cast<int32_t *>(dev->counts + 2);
  at += control_bytes;
  dev->tasks = reinterpret_cast<Task *>(at);
  at += task_bytes;
  dev->merges = reinterpret_cast<MergeRecord *>(at);
  dev->merge_count = (int32_t)tiles;
  at += merge_bytes;
  dev->bigs = reinterpret_cast<MergeRecord *>(at);
  dev->big_capacity = tiles > 0 ? (int32_t)big_capacity : 0;
  at += big_bytes;
  dev->partials = reinterpret_cast<float *>(at);
  dev->partial_slots = (int32_t)slots;
  dev->slot_step = 2;
  e = cudaMemsetAsync(dev->offsets + noffsets, 0,
                      (padded - noffsets) * sizeof(int32_t), stream);
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(dev->offsets, offsets, noffsets * sizeof(int32_t),
                        cudaMemcpyDeviceToDevice, stream);
  if (e == cudaSuccess)
    e = cudaMemsetAsync(dev->control, 0, control_bytes, stream);
  return e;
}

}  // namespace

cudaError_t device_plan(const int32_t *offsets, int32_t segment_count,
                        int32_t value_count, int op, cudaStream_t stream,
                        const unsigned long long *known_hash, DevicePlan *dev,
                        HostPlan *host, int32_t *reason, int64_t *index) {
  std::lock_guard<std::mutex> guard(g_scratch_lock);
  Scratch *scratch = nullptr;
  cudaError_t e = scratch_for(dev->device, &scratch);
  if (e != cudaSuccess) return e;
  const bool reusable =
      known_hash != nullptr && scratch->seen_offsets == offsets &&
      scratch->seen_segments == segment_count &&
      scratch->seen_values == value_count &&
      scratch->host->hash == *known_hash;
  if (!reusable) {
    e = summarise(offsets, segment_count, value_count, dev->sm_count, stream,
                  scratch);
    if (e != cudaSuccess) return e;
  }
  const Summary &s = *scratch->host;
  if (s.first_bad != kNoViolation) {
    *reason = rule_to_reason((unsigned)(s.first_bad & 7u));
    *index = (int64_t)(s.first_bad >> 3);
    return cudaSuccess;
  }
  *reason = SWG_OFFSETS_OK;
  *index = -1;

  host->segment_count = segment_count;
  host->value_count = s.last_offset;
  host->op = op;
  host->max_length = s.max_length;
  host->mean_length =
      segment_count > 0 ? (double)s.last_offset / segment_count : 0.0;
  for (int bin = 0; bin < kHistogramBins; ++bin) {
    host->histogram[bin] = s.histogram[bin];
    host->elements_in_bin[bin] = s.elements[bin];
  }
  dev->segment_count = segment_count;

  if (op == SWG_OP_SOFTMAX) {
    host->schedule = SWG_SCHED_SPLIT;
    int64_t total = 0;
    BucketBegins begins;
    for (int b = 0; b < kSoftmaxBuckets; ++b) {
      begins.begin[b] = (int32_t)total;
      dev->softmax_begin[b] = host->softmax_begin[b] = (int32_t)total;
      dev->softmax_count[b] = host->softmax_count[b] = s.softmax_count[b];
      total += s.softmax_count[b];
    }
    // one block: control words, the class lists, the planner's block counts
    const int32_t blocks = (segment_count + kListBlock - 1) / kListBlock;
    const size_t control_bytes = aligned256(kControlWords * sizeof(uint32_t));
    const size_t list_bytes = aligned256((size_t)total * sizeof(int32_t));
    const size_t count_bytes =
        aligned256((size_t)blocks * kSoftmaxBuckets * sizeof(int32_t));
    e = plan_block_allocate(dev, control_bytes + list_bytes + count_bytes,
                            stream);
    if (e != cudaSuccess) return e;
    unsigned char *at = static_cast<unsigned char *>(dev->block);
    dev->control = reinterpret_cast<uint32_t *>(at);
    dev->softmax_segments = reinterpret_cast<int32_t *>(at + control_bytes);
    int32_t *counts =
        reinterpret_cast<int32_t *>(at + control_bytes + list_bytes);
    e = cudaMemsetAsync(dev->control, 0, control_bytes, stream);
    if (e != cudaSuccess || total == 0) return e;
    const unsigned grid = (unsigned)(((int64_t)blocks * 32 + 255) / 256);
    bucket_count_kernel<<<grid, 256, 0, stream>>>(offsets, segment_count,
                                                  blocks, counts);
    bucket_scan_kernel<<<kSoftmaxBuckets, kScanThreads, 0, stream>>>(blocks,
                                                                     counts);
    bucket_fill_kernel<<<grid, 256, 0, stream>>>(
        offsets, segment_count, blocks, counts, begins, dev->softmax_segments);
    return cudaGetLastError();
  }

  host->schedule = choose_schedule(host->elements_in_bin, host->value_count,
                                   host->max_length, host->mean_length);
  const int64_t items =
      (int64_t)s.last_offset + (int64_t)kHeaderItems * segment_count;
  const int64_t tiles = (items + kDeviceTile - 1) / kDeviceTile;
  dev->task_count = (int32_t)tiles;
  host->task_total = tiles;
  host->slot_step = 2;
  e = reduce_block(dev, offsets, tiles, stream);
  if (e != cudaSuccess) return e;
  host->partial_slots = dev->partial_slots;
  if (tiles == 0) return cudaSuccess;
  const unsigned grid = (unsigned)((tiles + 255) / 256);
  tile_plan_kernel<<<grid, 256, 0, stream>>>(
      offsets, segment_count, (int32_t)tiles, dev->tasks, dev->merges,
      dev->bigs, dev->big_capacity, dev->big_count,
      reinterpret_cast<unsigned long long *>(dev->counts));
  return cudaGetLastError();
}

cudaError_t device_plan_counts(const DevicePlan &dev, int64_t *chunk_tasks,
                               int64_t *split_segments) {
  *chunk_tasks = *split_segments = 0;
  if (dev.counts == nullptr) return cudaSuccess;
  int64_t both[2] = {0, 0};
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess)
    e = cudaMemcpy(both, dev.counts, sizeof(both), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return e;
  *chunk_tasks = both[0];
  *split_segments = both[1];
  return cudaSuccess;
}

}  // namespace swg
