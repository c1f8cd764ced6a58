// Offsets validation and planning on the GPU: the offsets never leave the
// device.  The host reads back one small summary per call (the first rule an
// offsets array breaks, in the order of the reference's host loop --
// python/swage/_segmented_qualification.py:30-55 -- plus a content hash, the
// last offset, the length histogram and the bucket counts), and a second one
// (three counters) when a reduce plan is built.
//
// Reduce plan.  The host planner walks the segments one after the other; here
// every tile is found independently (merge-path): the sequence of items --
// per segment one header item, then its values -- is cut every kDeviceTile
// items, a binary search over p(s) = offsets[s] + s finds the segment each
// cut falls in, and a tile becomes one task of the same two kinds the host
// planner emits: a packed run of segments whose first and last may be pieces
// of segments that continue in the neighbouring tiles, or a chunk when the
// whole tile lies inside one segment.  Every piece of a cut segment needs a
// partial slot, contiguous per segment for the merge pass; with r(s) the rank
// of s among the cut segments, the piece of s in tile t gets slot t + r(s):
// consecutive tiles give consecutive slots, and the next cut segment starts
// one slot further even when it shares a tile.  r comes from one prefix sum
// over the tile boundaries (a boundary counts when the segment it cuts was
// not already cut by the boundary before).
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
  // written by the boundary scan
  int split_count, big_count, medium_count, pad;
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
    summary->split_count = summary->big_count = summary->medium_count = 0;
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

// Item position of segment s's header.
__device__ __forceinline__ int64_t header_at(const int32_t *offsets,
                                             int64_t s) {
  return (int64_t)__ldg(offsets + s) + s;
}

// Tile t starts at item t * kDeviceTile: the segment that item belongs to,
// with bit 31 set when the item is one of its values (the segment began in an
// earlier tile: the boundary cuts it).
__global__ void __launch_bounds__(256)
tile_start_kernel(const int32_t *__restrict__ offsets, int32_t segment_count,
                  int32_t tile_count, uint32_t *__restrict__ start) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tile_count) return;
  const int64_t d = t * kDeviceTile;
  int64_t lo = 0, hi = (int64_t)segment_count - 1;  // header_at(lo) <= d
  while (lo < hi) {
    const int64_t mid = (lo + hi + 1) >> 1;
    if (header_at(offsets, mid) <= d) lo = mid;
    else hi = mid - 1;
  }
  const bool cut = d > header_at(offsets, lo);
  start[t] = (uint32_t)lo | (cut ? 0x80000000u : 0u);
}

struct Boundary {
  bool first_cut;  // the segment this boundary cuts was not cut before it
  int pieces;      // then: pieces of that segment
};

__device__ __forceinline__ Boundary
boundary_at(const uint32_t *__restrict__ start,
            const int32_t *__restrict__ offsets, int64_t t) {
  Boundary b{false, 0};
  if (t == 0) return b;
  const uint32_t here = start[t], before = start[t - 1];
  if (!(here >> 31)) return b;
  if ((before >> 31) && ((before ^ here) & 0x7fffffffu) == 0) return b;
  const int64_t seg = here & 0x7fffffffu;
  // the segment's last item: its last value (or its header when empty, but an
  // empty segment is never cut)
  const int64_t last_item = (int64_t)__ldg(offsets + seg + 1) + seg;
  b.first_cut = true;
  b.pieces = (int)(last_item / kDeviceTile - t + 2);
  return b;
}

// One CTA: inclusive counts, per boundary, of first cuts (all / big / medium).
// The CTA walks the boundaries kScanThreads at a time (coalesced), scans the
// three flags of a batch with warp shuffles and carries the running totals.
constexpr int kScanThreads = 1024;

__global__ void __launch_bounds__(kScanThreads)
boundary_scan_kernel(const uint32_t *__restrict__ start,
                     const int32_t *__restrict__ offsets, int32_t tile_count,
                     int32_t *__restrict__ cuts, int32_t *__restrict__ bigs,
                     int32_t *__restrict__ mediums, Summary *summary) {
  __shared__ int warp_totals[3][kScanThreads / 32];
  __shared__ int carry[3];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < 3) carry[tid] = 0;
  __syncthreads();
  for (int64_t base = 0; base < tile_count; base += kScanThreads) {
    const int64_t t = base + tid;
    int v[3] = {0, 0, 0};
    if (t < tile_count) {
      const Boundary b = boundary_at(start, offsets, t);
      if (b.first_cut) {
        v[0] = 1;
        v[1] = b.pieces >= kBigSplit;
        v[2] = b.pieces < kBigSplit && b.pieces > kTinySplit;
      }
    }
    // inclusive scan inside the warp
#pragma unroll
    for (int k = 0; k < 3; ++k) {
#pragma unroll
      for (int delta = 1; delta < 32; delta <<= 1) {
        const int up = __shfl_up_sync(kFullMask, v[k], delta);
        if (lane >= delta) v[k] += up;
      }
      if (lane == 31) warp_totals[k][warp] = v[k];
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int k = 0; k < 3; ++k) {
        int w = warp_totals[k][lane];
#pragma unroll
        for (int delta = 1; delta < 32; delta <<= 1) {
          const int up = __shfl_up_sync(kFullMask, w, delta);
          if (lane >= delta) w += up;
        }
        warp_totals[k][lane] = w;  // inclusive over the warps
      }
    }
    __syncthreads();
    int before[3];
#pragma unroll
    for (int k = 0; k < 3; ++k)
      before[k] = carry[k] + (warp > 0 ? warp_totals[k][warp - 1] : 0);
    if (t < tile_count) {
      cuts[t] = before[0] + v[0];
      bigs[t] = before[1] + v[1];
      mediums[t] = before[2] + v[2];
    }
    __syncthreads();
    if (tid < 3) carry[tid] += warp_totals[tid][kScanThreads / 32 - 1];
    __syncthreads();
  }
  if (tid == 0) {
    summary->split_count = carry[0];
    summary->big_count = carry[1];
    summary->medium_count = carry[2];
  }
}

// One thread per tile: its task, and the merge-list entry of the segment its
// left boundary cuts for the first time.
__global__ void __launch_bounds__(256)
tile_emit_kernel(const int32_t *__restrict__ offsets, int32_t segment_count,
                 int32_t tile_count, const uint32_t *__restrict__ start,
                 const int32_t *__restrict__ cuts,
                 const int32_t *__restrict__ bigs,
                 const int32_t *__restrict__ mediums,
                 const Summary *__restrict__ summary, Task *__restrict__ tasks,
                 SplitSegment *__restrict__ splits) {
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tile_count) return;
  const uint32_t here = start[t];
  const int32_t first = (int32_t)(here & 0x7fffffffu);
  const bool head_cut = (here >> 31) != 0;
  const int64_t d = t * kDeviceTile;
  const int64_t vbegin = head_cut ? d - first - 1 : d - first;
  int32_t last;
  bool tail_cut;
  int64_t vend;
  if (t + 1 < tile_count) {
    const uint32_t next = start[t + 1];
    const int32_t next_first = (int32_t)(next & 0x7fffffffu);
    tail_cut = (next >> 31) != 0;
    last = tail_cut ? next_first : next_first - 1;
    const int64_t d1 = d + kDeviceTile;
    vend = tail_cut ? d1 - next_first - 1 : d1 - next_first;
  } else {
    tail_cut = false;
    last = segment_count - 1;
    vend = __ldg(offsets + segment_count);
  }
  const int32_t head_slot = head_cut ? (int32_t)(t + cuts[t] - 1) : -1;
  const int32_t tail_slot = tail_cut ? (int32_t)(t + cuts[t + 1] - 1) : -1;
  Task task;
  task.vbegin = (int32_t)vbegin;
  task.reserved0 = task.reserved1 = 0;
  if (first == last && head_cut && tail_cut) {
    task.seg = first;
    task.count = head_slot;  // == tail_slot: one piece, one slot
    task.vcount_kind = (uint32_t)(vend - vbegin) | (kTaskChunk << 28);
    task.head_slot = task.tail_slot = -1;
  } else {
    task.seg = first;
    task.count = last - first + 1;
    task.vcount_kind = (uint32_t)(vend - vbegin) | (kTaskPack << 28);
    task.head_slot = head_slot;
    task.tail_slot = tail_slot;
  }
  tasks[t] = task;

  const Boundary b = boundary_at(start, offsets, t);
  if (b.first_cut) {
    const int32_t rank = cuts[t] - 1;
    int32_t where;
    if (b.pieces >= kBigSplit) where = bigs[t] - 1;
    else if (b.pieces > kTinySplit)
      where = summary->big_count + mediums[t] - 1;
    else
      where = summary->big_count + summary->medium_count +
              (cuts[t] - bigs[t] - mediums[t]) - 1;
    SplitSegment s;
    s.seg = first;
    s.slot_begin = (int32_t)(t - 1) + rank;
    s.slot_count = b.pieces;
    s.pad = 0;
    splits[where] = s;
  }
}

// ---------------------------------------------------------------------------
// softmax plan
// ---------------------------------------------------------------------------
constexpr int kListBlock = 1024;  // segments ranked by one warp

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
  return cudaStreamSynchronize(stream);
}

}  // namespace

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

cudaError_t device_plan(const int32_t *offsets, int32_t segment_count,
                        int32_t value_count, int op, cudaStream_t stream,
                        DevicePlan *dev, HostPlan *host, int32_t *reason,
                        int64_t *index) {
  std::lock_guard<std::mutex> guard(g_scratch_lock);
  Scratch *scratch = nullptr;
  cudaError_t e = scratch_for(dev->device, &scratch);
  if (e != cudaSuccess) return e;
  e = summarise(offsets, segment_count, value_count, dev->sm_count, stream,
                scratch);
  if (e != cudaSuccess) return e;
  Summary &s = *scratch->host;
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

  // an aligned, padded copy of the offsets for the tile kernels' bulk copies
  const size_t noffsets = (size_t)segment_count + 1;
  const size_t padded = ((noffsets + 3) / 4) * 4 + 4;
  e = cudaMalloc((void **)&dev->offsets, padded * sizeof(int32_t));
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(dev->offsets + noffsets, 0,
                      (padded - noffsets) * sizeof(int32_t), stream);
  if (e != cudaSuccess) return e;
  e = cudaMemcpyAsync(dev->offsets, offsets, noffsets * sizeof(int32_t),
                      cudaMemcpyDeviceToDevice, stream);
  if (e != cudaSuccess) return e;
  e = cudaMalloc((void **)&dev->control, kControlWords * sizeof(uint32_t));
  if (e != cudaSuccess) return e;
  e = cudaMemsetAsync(dev->control, 0, kControlWords * sizeof(uint32_t),
                      stream);
  if (e != cudaSuccess) return e;

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
    if (total == 0) return cudaStreamSynchronize(stream);
    const int32_t blocks = (segment_count + kListBlock - 1) / kListBlock;
    int32_t *counts = nullptr;
    e = cudaMalloc((void **)&dev->softmax_segments, total * sizeof(int32_t));
    if (e != cudaSuccess) return e;
    e = cudaMalloc((void **)&counts,
                   (size_t)blocks * kSoftmaxBuckets * sizeof(int32_t));
    if (e != cudaSuccess) return e;
    const unsigned grid = (unsigned)(((int64_t)blocks * 32 + 255) / 256);
    bucket_count_kernel<<<grid, 256, 0, stream>>>(offsets, segment_count,
                                                  blocks, counts);
    bucket_scan_kernel<<<kSoftmaxBuckets, kScanThreads, 0, stream>>>(blocks,
                                                                     counts);
    bucket_fill_kernel<<<grid, 256, 0, stream>>>(
        offsets, segment_count, blocks, counts, begins, dev->softmax_segments);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    cudaFree(counts);
    return e;
  }

  host->schedule = choose_schedule(host->elements_in_bin, host->value_count,
                                   host->max_length, host->mean_length);
  const int64_t items = (int64_t)s.last_offset + segment_count;
  const int64_t tiles = (items + kDeviceTile - 1) / kDeviceTile;
  dev->task_count = (int32_t)tiles;
  if (tiles == 0) return cudaStreamSynchronize(stream);
  // one allocation for what the plan keeps (tasks, merge list, partials), one
  // for what only the planner needs (tile starts and the three scans)
  const size_t task_bytes = (size_t)tiles * sizeof(Task);
  const size_t split_bytes = (size_t)tiles * sizeof(SplitSegment);
  const size_t partial_bytes = (size_t)tiles * 2 * sizeof(float);
  unsigned char *kept = nullptr, *scratch_block = nullptr;
  e = cudaMalloc((void **)&kept, task_bytes + split_bytes + partial_bytes);
  if (e != cudaSuccess) return e;
  dev->tasks = reinterpret_cast<Task *>(kept);  // owns the block
  dev->splits = reinterpret_cast<SplitSegment *>(kept + task_bytes);
  dev->partials = reinterpret_cast<float *>(kept + task_bytes + split_bytes);
  dev->shared_block = true;
  e = cudaMalloc((void **)&scratch_block, (size_t)tiles * 4 * sizeof(int32_t));
  if (e == cudaSuccess) {
    uint32_t *start = reinterpret_cast<uint32_t *>(scratch_block);
    int32_t *scans = reinterpret_cast<int32_t *>(scratch_block) + tiles;
    const unsigned grid = (unsigned)((tiles + 255) / 256);
    tile_start_kernel<<<grid, 256, 0, stream>>>(offsets, segment_count,
                                                (int32_t)tiles, start);
    boundary_scan_kernel<<<1, kScanThreads, 0, stream>>>(
        start, offsets, (int32_t)tiles, scans, scans + tiles,
        scans + 2 * tiles, scratch->device);
    tile_emit_kernel<<<grid, 256, 0, stream>>>(
        offsets, segment_count, (int32_t)tiles, start, scans, scans + tiles,
        scans + 2 * tiles, scratch->device, dev->tasks, dev->splits);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(scratch->host, scratch->device, sizeof(Summary),
                        cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  cudaFree(scratch_block);
  if (e != cudaSuccess) return e;
  dev->split_count = s.split_count;
  dev->big_split_count = s.big_count;
  dev->medium_split_count = s.medium_count;
  dev->partial_slots = (int32_t)(tiles + s.split_count);
  host->partial_slots = dev->partial_slots;
  host->big_split_count = s.big_count;
  host->medium_split_count = s.medium_count;
  host->task_total = tiles;
  host->split_total = s.split_count;
  return cudaSuccess;
}

}  // namespace swg
