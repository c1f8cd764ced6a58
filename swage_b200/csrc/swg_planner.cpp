// Host planner: offsets validation, segment-length histogram, packing of
// segments into tile tasks, schedule choice and multi-GPU sharding.  Plain
// C++ (no CUDA) so it can be unit-tested without a device.
//
// Vocabulary follows the reference's docs/concepts/segments-tiles-tasks.md
// (:32-51): a segment is the logical unit, a tile the fixed-size physical
// unit, a task the schedulable bridge ("several short segments packed into
// one tile", "one chunk of a long segment", "a reduction merge").
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "swg_plan.h"

namespace swg {

namespace {
thread_local char g_error[512] = "";
}

void set_error(const char *format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(g_error, sizeof(g_error), format, args);
  va_end(args);
}

void clear_error() { g_error[0] = '\0'; }

const char *last_error_text() { return g_error; }

// Same checks, same order as _validate_offsets
// (python/swage/_segmented_qualification.py:30-55).  The reference walks a
// Python list; this is one pass over the int32 array.
int validate_offsets(const int32_t *offsets, int64_t count, int64_t value_count,
                     int64_t output_count, int32_t *reason, int64_t *index) {
  int32_t why = SWG_OFFSETS_OK;
  int64_t where = -1;
  const int64_t limit = int64_t(1) << 31;
  if (offsets == nullptr || count < 1) {
    why = SWG_OFFSETS_EMPTY;
  } else if (value_count < 0 || value_count >= limit || count - 1 >= limit) {
    why = SWG_OFFSETS_COUNT_RANGE;
  } else if (output_count < count - 1) {
    why = SWG_OFFSETS_OUTPUT_SMALL;
  } else if (offsets[0] != 0) {
    why = SWG_OFFSETS_NONZERO_START;
    where = 0;
  } else {
    int32_t previous = 0;
    for (int64_t i = 0; i < count; ++i) {
      int32_t offset = offsets[i];
      if (offset < 0) {
        why = SWG_OFFSETS_NEGATIVE;
        where = i;
        break;
      }
      if (offset < previous) {
        why = SWG_OFFSETS_DECREASING;
        where = i;
        break;
      }
      previous = offset;
    }
    if (why == SWG_OFFSETS_OK && offsets[count - 1] > value_count) {
      why = SWG_OFFSETS_EXCEEDS_VALUES;
      where = count - 1;
    }
  }
  if (reason) *reason = why;
  if (index) *index = where;
  if (why == SWG_OFFSETS_OK) return SWG_OK;
  set_error("offsets rejected: reason %d at index %lld", (int)why,
            (long long)where);
  return SWG_ERR_INVALID_OFFSETS;
}

static inline int length_bin(int64_t length) {
  if (length <= 0) return 0;
  int bin = 1;
  while ((int64_t(1) << bin) <= length && bin < kHistogramBins - 1) ++bin;
  return bin;  // 2^(bin-1) <= length < 2^bin
}

namespace {

// Walks the segments once and cuts the (values + segments) sequence into tile
// tasks of at most kTileItems items.  A segment that does not fit the open
// tile is either moved to the next tile whole (short ones: the waste is at
// most kSplitMinimum items) or cut: a tail piece fills the open tile, whole
// 2048-value pieces become chunk tasks, and the last piece opens the next
// tile, so tiles stay full whatever the length mix.
struct Packer {
  HostPlan *plan;
  int32_t seg_begin = 0, nseg = 0, vbegin = 0, vcount = 0;
  int32_t head_slot = -1, tail_slot = -1;
  int32_t head_first = -1, tail_pieces = 0;  // see Task::link_*

  int32_t room() const {
    return kTileItems - (vcount + kHeaderItems * nseg);
  }

  void flush() {
    if (nseg == 0) return;
    Task task;
    task.seg = seg_begin;
    task.count = nseg;
    task.vbegin = vbegin;
    task.vcount_kind = (kTaskPack << 28) | (uint32_t)vcount;
    task.head_slot = head_slot;
    task.tail_slot = tail_slot;
    task.link_first = head_first;
    task.link_pieces = tail_pieces;
    plan->tasks.push_back(task);
    plan->pack_tasks++;
    nseg = 0;
    vcount = 0;
    head_slot = tail_slot = head_first = -1;
    tail_pieces = 0;
  }

  // append `length` values of segment `seg` starting at value `start`
  void append(int32_t seg, int32_t start, int32_t length) {
    if (nseg == 0) {
      seg_begin = seg;
      vbegin = start;
    }
    nseg++;
    vcount += length;
  }

  // `first` / `pieces`: the slots of the segment this chunk is a piece of
  void chunk(int32_t seg, int32_t start, int32_t length, int32_t slot,
             int32_t first, int32_t pieces) {
    Task task;
    task.seg = seg;
    task.count = slot;
    task.vbegin = start;
    task.vcount_kind = (kTaskChunk << 28) | (uint32_t)length;
    task.head_slot = task.tail_slot = -1;
    task.link_first = first;
    task.link_pieces = pieces;
    plan->tasks.push_back(task);
    plan->chunk_tasks++;
  }
};

void plan_reduce(const int32_t *offsets, int32_t segment_count,
                 HostPlan *plan) {
  Packer packer{plan};
  plan->tasks.reserve((size_t)(offsets[segment_count] / kTileItems) + 64);
  for (int32_t seg = 0; seg < segment_count; ++seg) {
    const int32_t start = offsets[seg];
    const int32_t length = offsets[seg + 1] - start;
    if (packer.nseg >= kTileMaxSegments) packer.flush();
    if (length + kHeaderItems <= packer.room()) {
      packer.append(seg, start, length);
      continue;
    }
    if (length <= kSplitMinimum || length + kHeaderItems <= kTileItems) {
      // short: never cut.  Medium and the open tile nearly full: not worth
      // a cut either when the whole segment fits a tile and the open tile
      // has less than a useful piece of room.
      if (length <= kSplitMinimum ||
          packer.room() - kHeaderItems < kSplitMinimumPiece) {
        packer.flush();
        packer.append(seg, start, length);
        continue;
      }
    }
    // Cut the segment.  Pieces, in order: a tail piece that fills the open
    // tile, whole-tile chunks, and a head piece that opens the next tile.
    int32_t position = start, remaining = length;
    int32_t tail_piece = 0;
    if (packer.nseg > 0 &&
        packer.room() - kHeaderItems >= kSplitMinimumPiece)
      tail_piece = packer.room() - kHeaderItems;
    const int32_t after_tail = remaining - tail_piece;
    const int32_t whole_chunks = after_tail / kTileValues;
    const int32_t last_piece = after_tail - whole_chunks * kTileValues;
    const int32_t pieces =
        (tail_piece > 0) + whole_chunks + (last_piece > 0);
    if (pieces == 1) {
      // one chunk on its own (2032..2048 values): straight to out
      packer.flush();
      packer.chunk(seg, start, length, -1, -1, 0);
      continue;
    }
    const int32_t first = plan->partial_slots;
    int32_t slot = first;
    plan->partial_slots += pieces;
    plan->split_segments++;
    (pieces > kWarpMerge ? plan->big_merges : plan->merges)
        .push_back(MergeRecord{seg, first, pieces, 0});
    if (tail_piece > 0) {
      packer.append(seg, position, tail_piece);
      packer.tail_slot = slot++;
      packer.tail_pieces = pieces;
      position += tail_piece;
      remaining -= tail_piece;
    }
    packer.flush();
    for (int32_t c = 0; c < whole_chunks; ++c) {
      packer.chunk(seg, position, kTileValues, slot++, first, pieces);
      position += kTileValues;
      remaining -= kTileValues;
    }
    if (last_piece > 0) {
      if (last_piece + kHeaderItems <= kTileItems) {
        packer.append(seg, position, last_piece);
        packer.head_slot = slot++;
        packer.head_first = first;
      } else {
        packer.chunk(seg, position, last_piece, slot++, first, pieces);
      }
    }
  }
  packer.flush();
}

// Softmax: bucket the non-empty segments by length.  Inside a bucket segments
// keep their order in memory: CTAs walking the bucket side by side then read
// neighbouring addresses, which measured several per cent faster than any
// order by length.  The last bucket has no upper limit, so there segments are
// emitted bin by bin from the longest (a counting sort on the histogram
// bins): a few giant segments must start first.
static inline int softmax_bucket(int64_t length) {
  for (int b = 0; b < kSoftmaxBuckets - 1; ++b)
    if (length <= kSoftmaxLimit[b]) return b;
  return kSoftmaxBuckets - 1;
}

void plan_softmax(const int32_t *offsets, int32_t segment_count,
                  HostPlan *plan) {
  // slot = bucket for all buckets but the last, then one slot per length
  // bin, longest first, for the last: one counting sort over all of them
  const int slots = kSoftmaxBuckets - 1 + kHistogramBins;
  std::vector<int64_t> fill((size_t)slots, 0), start((size_t)slots, 0);
  auto slot_of = [](int64_t length) {
    const int bucket = softmax_bucket(length);
    if (bucket < kSoftmaxBuckets - 1) return bucket;
    return kSoftmaxBuckets - 1 + (kHistogramBins - 1 - length_bin(length));
  };
  int64_t total = 0;
  for (int32_t seg = 0; seg < segment_count; ++seg) {
    const int64_t length = (int64_t)offsets[seg + 1] - offsets[seg];
    if (length <= 0) continue;
    fill[(size_t)slot_of(length)]++;
    total++;
  }
  int64_t at = 0;
  for (int slot = 0; slot < slots; ++slot) {
    start[(size_t)slot] = at;
    at += fill[(size_t)slot];
  }
  for (int b = 0; b < kSoftmaxBuckets; ++b) {
    plan->softmax_begin[b] = (int32_t)start[(size_t)b];
    plan->softmax_count[b] = (int32_t)fill[(size_t)b];
  }
  plan->softmax_count[kSoftmaxBuckets - 1] =
      (int32_t)(total - start[(size_t)(kSoftmaxBuckets - 1)]);
  plan->softmax_segments.assign((size_t)total, 0);
  for (int32_t seg = 0; seg < segment_count; ++seg) {
    const int64_t length = (int64_t)offsets[seg + 1] - offsets[seg];
    if (length <= 0) continue;
    plan->softmax_segments[(size_t)start[(size_t)slot_of(length)]++] = seg;
  }
}

}  // namespace

void build_host_plan(const int32_t *offsets, int32_t segment_count, int op,
                     HostPlan *plan) {
  plan->segment_count = segment_count;
  plan->value_count = offsets[segment_count];
  plan->op = op;
  for (int32_t seg = 0; seg < segment_count; ++seg) {
    const int64_t length = (int64_t)offsets[seg + 1] - offsets[seg];
    const int bin = length_bin(length);
    plan->histogram[bin]++;
    plan->elements_in_bin[bin] += length;
    plan->max_length = std::max(plan->max_length, length);
  }
  plan->mean_length =
      segment_count > 0 ? (double)plan->value_count / segment_count : 0.0;
  if (op == SWG_OP_SOFTMAX) {
    plan_softmax(offsets, segment_count, plan);
    plan->schedule = SWG_SCHED_SPLIT;
    return;
  }
  plan_reduce(offsets, segment_count, plan);
  plan->schedule = choose_schedule(plan->elements_in_bin, plan->value_count,
                                   plan->max_length, plan->mean_length);
}

std::string describe_host_plan(const HostPlan &plan) {
  std::string text = "{";
  char buffer[1024];
  snprintf(buffer, sizeof(buffer),
           "\"segments\": %d, \"values\": %d, \"op\": %d, \"schedule\": %d, "
           "\"mean_length\": %.3f, \"max_length\": %lld, \"tasks\": %zu, "
           "\"pack_tasks\": %lld, \"chunk_tasks\": %lld, "
           "\"split_segments\": %zu, \"partial_slots\": %d, "
           "\"tile_values\": %d, \"tile_items\": %d, "
           "\"tile_max_segments\": %d, "
           "\"split_minimum\": %d, \"softmax_buckets\": [%d, %d, %d, %d, %d, %d, %d, %d], ",
           plan.segment_count, plan.value_count, plan.op, plan.schedule,
           plan.mean_length, (long long)plan.max_length,
           plan.task_total >= 0 ? (size_t)plan.task_total : plan.tasks.size(),
           (long long)plan.pack_tasks, (long long)plan.chunk_tasks,
           (size_t)plan.split_segments,
           plan.partial_slots, kTileValues, kTileItems,
           kTileMaxSegments,
           kSplitMinimum, plan.softmax_count[0], plan.softmax_count[1],
           plan.softmax_count[2], plan.softmax_count[3], plan.softmax_count[4],
           plan.softmax_count[5], plan.softmax_count[6], plan.softmax_count[7]);
  text += buffer;
  text += "\"histogram\": [";
  for (int bin = 0; bin < kHistogramBins; ++bin) {
    snprintf(buffer, sizeof(buffer), "%s%lld", bin ? ", " : "",
             (long long)plan.histogram[bin]);
    text += buffer;
  }
  text += "], \"elements_in_bin\": [";
  for (int bin = 0; bin < kHistogramBins; ++bin) {
    snprintf(buffer, sizeof(buffer), "%s%lld", bin ? ", " : "",
             (long long)plan.elements_in_bin[bin]);
    text += buffer;
  }
  text += "]}";
  return text;
}

// Element-balanced contiguous segment ranges: the cut before shard g is the
// segment boundary closest to g * total / shards.
int shard_offsets(const int32_t *offsets, int32_t segment_count, int32_t shards,
                  int32_t *seg_begin) {
  if (offsets == nullptr || seg_begin == nullptr || shards < 1 ||
      segment_count < 0) {
    set_error("shard_offsets: bad arguments");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  // A shard costs its values plus its segments (what the tile tasks count):
  // cost of segments [a, b) = items(b) - items(a), items(i) = offsets[i] + i.
  // The cuts minimise the largest shard: binary search on the bound, each
  // probe packing shards greedily from the left with binary searches.
  auto items = [&](int64_t i) { return (int64_t)offsets[i] + i; };
  // last boundary b >= from with items(b) - items(from) <= bound
  auto reach = [&](int64_t from, int64_t bound) {
    int64_t lo = from, hi = segment_count;
    const int64_t limit = items(from) + bound;
    while (lo < hi) {
      const int64_t mid = (lo + hi + 1) >> 1;
      if (items(mid) <= limit) lo = mid;
      else hi = mid - 1;
    }
    return lo;
  };
  auto fits = [&](int64_t bound) {
    int64_t at = 0;
    for (int32_t g = 0; g < shards && at < segment_count; ++g)
      at = reach(at, bound);
    return at >= segment_count;
  };
  const int64_t total = items(segment_count);
  int64_t low = (total + shards - 1) / shards, high = total;
  while (low < high) {
    const int64_t mid = low + (high - low) / 2;
    if (fits(mid)) high = mid;
    else low = mid + 1;
  }
  // With the best bound known, every cut goes as near its ideal position as
  // the bound allows: not before the point the shards to its left can reach
  // back from (so they stay within the bound) ... walking from the right
  // gives each cut's earliest position, from the left its latest.
  std::vector<int64_t> latest((size_t)shards + 1, segment_count);
  latest[0] = 0;
  for (int32_t g = 1; g < shards; ++g) latest[g] = reach(latest[g - 1], low);
  seg_begin[0] = 0;
  for (int32_t g = 1; g < shards; ++g) {
    const int64_t ideal = total / shards * g;
    // first boundary whose items reach the ideal position
    int64_t lo = seg_begin[g - 1], hi = latest[g];
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if (items(mid) >= ideal) hi = mid;
      else lo = mid + 1;
    }
    int64_t boundary = lo;
    // the rest must still fit behind this cut: move right while it does not
    auto rest_fits = [&](int64_t from) {
      int64_t at = from;
      for (int32_t r = g; r < shards && at < segment_count; ++r)
        at = reach(at, low);
      return at >= segment_count;
    };
    if (!rest_fits(boundary)) {
      int64_t a = boundary, z = latest[g];  // rest_fits(z) holds
      while (a < z) {
        const int64_t mid = (a + z) >> 1;
        if (rest_fits(mid)) z = mid;
        else a = mid + 1;
      }
      boundary = a;
    }
    seg_begin[g] = (int32_t)boundary;
  }
  seg_begin[shards] = segment_count;
  return SWG_OK;
}

}  // namespace swg
