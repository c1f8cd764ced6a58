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
constexpr int kTileMaxSegments = kTileItems;  // segments per packed tile task
constexpr int kHeaderItems = 4;        // items a segment counts for besides its
                                       // values: a tile of very short segments
                                       // is bound by the per-segment work, not
                                       // by its bytes, and holds fewer of them
constexpr int kSplitMinimum = 128;     // segments up to here are never cut
constexpr int kSplitMinimumPiece = 32; // smallest piece left in an open tile
constexpr int kLaneMerge = 8;          // up to here one thread merges a segment's partials
constexpr int kWarpMerge = 256;        // up to here a warp does; a CTA above
constexpr int kHistogramBins = 33;     // bin b: len == 0 | 2^(b-1) <= len < 2^b

// One schedulable unit: what one warp reduces.  32 bytes (two 128-bit loads).
//   PACK : segments seg .. seg+count-1 and their values
//          [vbegin, vbegin+vcount).  All of them are whole, except that the
//          first may have begun in an earlier task (head_slot >= 0: this is
//          the LAST piece of that segment) and the last may continue in a
//          later one (tail_slot >= 0: this is the FIRST piece of that
//          segment): those two results go to the given partial slot, the
//          others straight to out.
//   CHUNK: a piece [vbegin, vbegin+vcount) of the single long segment `seg`
//          that fills the whole task; count = partial slot to write, or -1
//          when the piece is the whole segment and the result goes straight
//          to out[seg].
// A segment cut into P >= 2 pieces owns P partial slots: piece 0 has slot
// `first`, piece k > 0 slot first + k * step - (step - 1), with `step` a
// constant of the plan (1: slots handed out one after the other by the host
// planner; 2: two slots per tile, the device planner's numbering, which needs
// no prefix sum).  The merge pass that follows the tile kernel combines them
// in slot order; a task also says where its segments' slots lie:
//   link_first   PACK: slot of piece 0 of the segment whose last piece is this
//                task's head piece; CHUNK: slot of piece 0 of its segment
//   link_pieces  PACK: pieces of the segment whose first piece is this task's
//                tail piece; CHUNK: pieces of its segment
struct Task {
  int32_t seg;
  int32_t count;
  int32_t vbegin;
  uint32_t vcount_kind;  // bits 0..27 value count, bits 28..31 kind
  int32_t head_slot;     // PACK only, else -1
  int32_t tail_slot;     // PACK only, else -1
  int32_t link_first;
  int32_t link_pieces;
};
constexpr uint32_t kTaskPack = 0u, kTaskChunk = 1u;

// One cut segment for the merge pass: out[seg] = partials of its `pieces`
// slots, combined in slot order.  pieces < 2: nothing to merge (the device
// planner writes one record per tile, most of them empty).
struct MergeRecord {
  int32_t seg;
  int32_t first;
  int32_t pieces;
  int32_t pad;
};
constexpr uint32_t kTaskCountMask = (1u << 28) - 1u;

// Softmax buckets by segment length: the first three are held in the
// registers of eight lanes / a warp / a 128-thread CTA; the longer ones go
// through shared-memory rings whose size doubles from class to class, so that
// a segment -- in the last class, one of up to 57344 values -- stays on the SM
// between its two sweeps.
#ifndef SWG_SOFTMAX_LIMIT6
#define SWG_SOFTMAX_LIMIT6 24576  // a multiple of 2048: the ring of that class has LIMIT6 / 2048 warps
#endif
constexpr int kSoftmaxBuckets = 8;
constexpr int kSoftmaxLimit[kSoftmaxBuckets - 1] = {64,   512,  2048, 4096,
                                                    8192, 16384,
                                                    SWG_SOFTMAX_LIMIT6};

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
  std::vector<MergeRecord> merges;      // the cut segments of up to
                                        // kWarpMerge pieces
  std::vector<MergeRecord> big_merges;  // and those with more
  int64_t split_segments = 0;           // the number of both
  // softmax: ids of the non-empty segments, bucket after bucket; the last
  // (streamed) bucket is ordered by decreasing length bin so that a
  // round-robin over it is balanced
  std::vector<int32_t> softmax_segments;
  int32_t softmax_begin[kSoftmaxBuckets] = {0};
  int32_t softmax_count[kSoftmaxBuckets] = {0};
  int32_t partial_slots = 0;
  int32_t slot_step = 1;  // see Task
  int64_t pack_tasks = 0, chunk_tasks = 0;
  // plans built on the device keep no host copy of their task list
  int64_t task_total = -1;
};

// Schedule choice from the length statistics (measured on B200):
//  - small inputs whose segments are all of moderate length: one warp per
//    segment streams straight from global memory, no staging;
//  - most values in long segments (nearly every tile a chunk): tile tasks, a
//    CTA per pair (split) -- the hardware CTA scheduler then keeps the most
//    copies in flight (8 % ahead of resident on 2^30 values, 3 % on 2^27);
//  - otherwise, large inputs: the same tile tasks on resident CTAs, which
//    hide the time a warp spends reducing a tile of many segments (10 %
//    ahead of split on the lognormal and uniform mixes);
//  - small skewed inputs: split.
// The persistent (ticketed ring) schedule runs the same tasks and is
// selectable, but is never the fastest.
inline int choose_schedule(const int64_t *elements_in_bin, int64_t value_count,
                           int64_t max_length, double mean_length) {
  int64_t in_long = 0;  // values in segments of at least 4096
  for (int bin = 13; bin < kHistogramBins; ++bin) in_long += elements_in_bin[bin];
  if (2 * in_long >= value_count && value_count > 0) return SWG_SCHED_SPLIT;
  if (value_count >= (int64_t(1) << 24)) return SWG_SCHED_RESIDENT;
  return max_length <= 4096 && mean_length >= 256.0 ? SWG_SCHED_WARP
                                                    : SWG_SCHED_SPLIT;
}

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
