// Host-side description of a segment plan, shared by the planner (plain C++)
// and the launch code (CUDA).
#pragma once

#include <stdint.h>

#include <string>
#include <vector>

#include "swage_b200.h"

namespace swg {

// Geometry shared by the planner and the tile kernels.
constexpr int kTileValues = 2048;      // values per tile task (8 KiB of fp32)
constexpr int kTileItems = 2032;       // values + segments of a packed task:
                                       // its offsets share the tile's stage
constexpr int kTileMaxSegments = 1024; // segments per packed tile task
constexpr int kLongSegment = 1792;     // longer segments become chunk tasks
constexpr int kBigSplit = 256;         // partials from which a merge gets a whole CTA
constexpr int kHistogramBins = 33;     // bin b: len == 0 | 2^(b-1) <= len < 2^b

// One schedulable unit.  16 bytes so a task is one 128-bit load.
//   PACK : `count` whole segments seg .. seg+count-1, whose values
//          [vbegin, vbegin+vcount) fit one tile; results go straight to out.
//   CHUNK: a piece [vbegin, vbegin+vcount) of the single long segment `seg`;
//          count = partial slot to write, or -1 when the piece is the whole
//          segment and the result goes straight to out[seg].
struct Task {
  int32_t seg;
  int32_t count;
  int32_t vbegin;
  uint32_t vcount_kind;  // bits 0..27 value count, bits 28..31 kind
};
constexpr uint32_t kTaskPack = 0u, kTaskChunk = 1u;
constexpr uint32_t kTaskCountMask = (1u << 28) - 1u;

// A long segment whose partials are merged by the combine pass.
struct SplitSegment {
  int32_t seg;
  int32_t slot_begin;
  int32_t slot_count;
  int32_t pad;
};

// Softmax buckets by segment length: the first three are held in the
// registers of a warp / a 128-thread CTA / a 512-thread CTA (16 values per
// thread; read once, written once), longer segments are streamed by a CTA in
// two sweeps.
constexpr int kSoftmaxBuckets = 4;
constexpr int kSoftmaxLimit[kSoftmaxBuckets - 1] = {512, 2048, 8192};

struct HostPlan {
  int32_t segment_count = 0;
  int32_t value_count = 0;   // offsets[last]: values covered by segments
  int op = SWG_OP_REDUCE;
  int schedule = SWG_SCHED_CTA;  // what AUTO resolves to
  int64_t histogram[kHistogramBins] = {0};
  int64_t elements_in_bin[kHistogramBins] = {0};
  int64_t max_length = 0;
  double mean_length = 0.0;
  std::vector<Task> tasks;
  std::vector<SplitSegment> splits;
  // softmax: ids of the non-empty segments, bucket after bucket; the last
  // (streamed) bucket is ordered by decreasing length bin so that a
  // round-robin over it is balanced
  std::vector<int32_t> softmax_segments;
  int32_t softmax_begin[kSoftmaxBuckets] = {0, 0, 0, 0};
  int32_t softmax_count[kSoftmaxBuckets] = {0, 0, 0, 0};
  int32_t partial_slots = 0;
  int32_t big_split_count = 0;  // splits are ordered big ones first
  int64_t pack_tasks = 0, chunk_tasks = 0;
};

// Builds the histogram, the task list and the schedule choice.
void build_host_plan(const int32_t *offsets, int32_t segment_count, int op,
                     HostPlan *plan);
std::string describe_host_plan(const HostPlan &plan);

int validate_offsets(const int32_t *offsets, int64_t count, int64_t value_count,
                     int64_t output_count, int32_t *reason, int64_t *index);
int shard_offsets(const int32_t *offsets, int32_t segment_count,
                  int32_t shards, int32_t *seg_begin);

// Thread-local error text.
void set_error(const char *format, ...);
void clear_error();

}  // namespace swg
