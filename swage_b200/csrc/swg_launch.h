// Internal launch interface between the C ABI (swg_api.cu) and the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "swg_plan.h"

namespace swg {

// Destinations of a launch that stores its results into every GPU's copy of
// a full result array (`peers`, may be null: results go to `out`); f32,
// unmapped launches only.  Defined beside the kernels.
struct PeerOut;

constexpr int kTicketBase = 4;
constexpr int kStatusWord = kTicketBase + kSoftmaxBuckets;  // 12
constexpr int kControlWords = kStatusWord + 4;              // 16

// Device-resident part of a plan; every pointer is owned by the plan.
struct DevicePlan {
  int device = -1;
  int sm_count = 0;
  Task *tasks = nullptr;
  int32_t task_count = 0;
  int32_t segment_count = 0;
  int32_t *offsets = nullptr;      // aligned, padded copy of the CSR offsets
  float *partials = nullptr;       // one float per partial slot of a cut segment
  int32_t partial_slots = 0;
  int32_t slot_step = 1;           // see Task
  MergeRecord *merges = nullptr;   // what the merge pass walks: cut segments
  int32_t merge_count = 0;         // of up to kWarpMerge pieces (or empty)
  MergeRecord *bigs = nullptr;     // and those with more, listed apart;
  int32_t *big_count = nullptr;    // how many (device-resident)
  int32_t big_capacity = 0;        // and how many the list can hold
  int32_t *softmax_segments = nullptr;  // bucketed segment ids
  int32_t softmax_begin[kSoftmaxBuckets] = {0};
  int32_t softmax_count[kSoftmaxBuckets] = {0};
  uint32_t *control = nullptr;     // [0] ticket, [1] finished, [2] error, [3] detail,
                                   // [kTicketBase + class] softmax ticket counters,
                                   // [kStatusWord, +1] address of the host-visible
                                   // copy of the error word (0: none)
  int64_t *counts = nullptr;       // device planner: {chunk tasks, cut segments}
  void *block = nullptr;           // the one allocation the pointers above live in
  size_t block_bytes = 0;
  bool pooled = false;             // block came from the stream-ordered pool
  uint32_t *host_status = nullptr; // pinned, device-visible: {error, detail}
};

// Optional pair of events recorded around the dominant kernel of a call.
struct Probe {
  cudaEvent_t start;
  cudaEvent_t stop;
};

inline void probe_begin(const Probe *probe, cudaStream_t stream) {
  if (probe) cudaEventRecord(probe->start, stream);
}
inline void probe_end(const Probe *probe, cudaStream_t stream) {
  if (probe) cudaEventRecord(probe->stop, stream);
}

cudaError_t launch_vadd(const float *x, const float *y, float *out, int32_t n,
                        cudaStream_t stream, const Probe *probe);

// dst_bases[p][dst_offset + i] = src[i] for every destination (device
// pointers, possibly peer-mapped memory of other GPUs); plain stores.
cudaError_t launch_scatter_results(const float *src, int64_t count,
                                   float *const *dst_bases, int peer_count,
                                   int64_t dst_offset, int sm_count,
                                   cudaStream_t stream);

cudaError_t launch_segreduce_warp(int kind, const float *values,
                                  const int32_t *offsets, float *out,
                                  int32_t segment_count, int sm_count,
                                  cudaStream_t stream, const Probe *probe);
cudaError_t launch_segreduce_cta(int kind, const float *values,
                                 const int32_t *offsets, float *out,
                                 int32_t segment_count, int32_t block,
                                 int sm_count, cudaStream_t stream,
                                 const Probe *probe);
// Sum and max of every segment in one pass (no plan).
cudaError_t launch_segreduce_sum_max(const float *values,
                                     const int32_t *offsets, float *out_sum,
                                     float *out_max, int32_t value_count,
                                     int32_t segment_count, int sm_count,
                                     cudaStream_t stream, const Probe *probe);
// One tile task per warp, two per CTA + merge pass.
// (dtype: SWG_DTYPE_*; `out` holds fp32, or int32 for i32 values)
cudaError_t launch_segreduce_split(int kind, int dtype, const void *values,
                                   void *out, int32_t value_count,
                                   const DevicePlan &plan, cudaStream_t stream,
                                   const Probe *probe,
                                   const swg_map *map = nullptr,
                                   const PeerOut *peers = nullptr);
// Persistent CTAs, bulk-copy ring, ticket counter + merge pass.
cudaError_t launch_segreduce_persistent(int kind, const float *values,
                                        float *out, int32_t value_count,
                                        const DevicePlan &plan,
                                        cudaStream_t stream,
                                        const Probe *probe);
// One resident CTA per SM, one stage per warp, tasks at a fixed stride +
// merge pass.
cudaError_t launch_segreduce_resident(int kind, int dtype, const void *values,
                                      void *out, int32_t value_count,
                                      const DevicePlan &plan,
                                      cudaStream_t stream, const Probe *probe,
                                      const swg_map *map = nullptr,
                                      const PeerOut *peers = nullptr);
// A warp or a CTA per segment for f16 / bf16 / i32 values, and for mapped
// reductions of every floating type (no plan).  `map` (may be null) is
// applied to every value before it is reduced; integer segments ignore it.
cudaError_t launch_segreduce_typed(int kind, int dtype, const void *values,
                                   const int32_t *offsets, void *out,
                                   int32_t value_count, int32_t segment_count,
                                   bool cta, int sm_count, cudaStream_t stream,
                                   const Probe *probe,
                                   const swg_map *map = nullptr);
// Runs a wait that cannot succeed for `limit_ns`, so that the plan's error
// words report a timeout (see swg_plan_selftest_timeout).
cudaError_t launch_wait_selftest(const DevicePlan &plan, uint64_t limit_ns,
                                 cudaStream_t stream);
cudaError_t configure_segreduce_kernels();
cudaError_t configure_softmax_kernels();

// Validation and planning on the device (swg_device_plan.cu).
struct DeviceDigest {
  unsigned long long hash;  // of the offsets' content
  int32_t last_offset;
  int32_t max_length;
};
// Checks device-resident offsets[0 .. segment_count] against the rules of
// validate_offsets; synchronises `stream` to read the verdict.
cudaError_t device_validate(const int32_t *offsets, int32_t segment_count,
                            int32_t value_count, int device, int sm_count,
                            cudaStream_t stream, int32_t *reason,
                            int64_t *index, DeviceDigest *digest);
// Fills `dev` (device, sm_count preset by the caller) and the summary fields
// of `host` for offsets that pass validation.  *reason != SWG_OFFSETS_OK:
// nothing was planned.  With `known_hash` the summary of the validation pass
// that returned this digest for the same array is reused when it is still the
// latest one on the device (no second pass, no synchronisation); else the
// pass runs here and `stream` is synchronised once to read it.
cudaError_t device_plan(const int32_t *offsets, int32_t segment_count,
                        int32_t value_count, int op, cudaStream_t stream,
                        const unsigned long long *known_hash, DevicePlan *dev,
                        HostPlan *host, int32_t *reason, int64_t *index);
// Brings the device planner's task statistics to the host (synchronises).
cudaError_t device_plan_counts(const DevicePlan &dev, int64_t *chunk_tasks,
                               int64_t *split_segments);
// Plan memory: one block per plan from the device's stream-ordered pool
// (kept by the library between plans, so a new plan costs no cudaMalloc).
cudaError_t plan_block_allocate(DevicePlan *dev, size_t bytes,
                                cudaStream_t stream);
void plan_block_release(DevicePlan *dev, cudaStream_t after, bool ordered);

// Allocation-free variant: the split schedule run out of a fixed-size
// file-scope device array.  Limits of that array:
constexpr int kStaticMaxSegments = 1 << 18;
constexpr int kStaticMaxTasks = 1 << 15;
constexpr int kStaticMaxSlots = 1 << 15;
cudaError_t launch_segreduce_static(int kind, const float *values, float *out,
                                    int32_t value_count,
                                    const int32_t *host_offsets,
                                    int32_t segment_count,
                                    const HostPlan &plan, int device,
                                    int sm_count, cudaStream_t stream);

cudaError_t launch_segsoftmax_cta(const float *values, const int32_t *offsets,
                                  float *out, int32_t segment_count,
                                  int sm_count, cudaStream_t stream,
                                  const Probe *probe);
cudaError_t launch_segsoftmax_warp(const float *values, const int32_t *offsets,
                                   float *out, int32_t segment_count,
                                   int sm_count, cudaStream_t stream,
                                   const Probe *probe);

// Planned softmax: the ring buckets and the register-resident buckets,
// concurrently.
cudaError_t launch_segsoftmax_planned(const float *values,
                                      const int32_t *offsets, float *out,
                                      int32_t value_count,
                                      const DevicePlan &plan,
                                      cudaStream_t stream, const Probe *probe);

const char *last_error_text();

}  // namespace swg
