// Internal launch interface between the C ABI (swg_api.cu) and the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "swg_plan.h"

namespace swg {

constexpr int kTicketBase = 4;
constexpr int kControlWords = kTicketBase + kSoftmaxBuckets + 4;  // 16

// Device-resident part of a plan; every pointer is owned by the plan.
struct DevicePlan {
  int device = -1;
  int sm_count = 0;
  Task *tasks = nullptr;
  int32_t task_count = 0;
  int32_t segment_count = 0;
  int32_t *offsets = nullptr;      // aligned, padded copy of the CSR offsets
  SplitSegment *splits = nullptr;
  int32_t split_count = 0;
  int32_t big_split_count = 0;     // leading splits that get a CTA each
  int32_t medium_split_count = 0;  // then those that get a warp each
  float *partials = nullptr;       // one float per partial slot
  int32_t partial_slots = 0;
  int32_t *softmax_segments = nullptr;  // bucketed segment ids
  int32_t softmax_begin[kSoftmaxBuckets] = {0};
  int32_t softmax_count[kSoftmaxBuckets] = {0};
  uint32_t *control = nullptr;     // [0] ticket, [1] finished, [2] error, [3] detail,
                                   // [kTicketBase + class] softmax ticket counters
  bool shared_block = false;       // tasks, splits and partials are one allocation
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
// One tile task per CTA + combine pass.
cudaError_t launch_segreduce_split(int kind, const float *values, float *out,
                                   int32_t value_count, const DevicePlan &plan,
                                   cudaStream_t stream, const Probe *probe);
// Persistent CTAs, bulk-copy ring, ticket counter + combine pass.
cudaError_t launch_segreduce_persistent(int kind, const float *values,
                                        float *out, int32_t value_count,
                                        const DevicePlan &plan,
                                        cudaStream_t stream,
                                        const Probe *probe);
// One resident CTA per SM, one stage per warp, tasks at a fixed stride +
// combine pass.
cudaError_t launch_segreduce_resident(int kind, const float *values,
                                      float *out, int32_t value_count,
                                      const DevicePlan &plan,
                                      cudaStream_t stream, const Probe *probe);
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
// Validates, then fills `dev` (device, sm_count preset by the caller) and the
// summary fields of `host`.  *reason != SWG_OFFSETS_OK: nothing was planned.
cudaError_t device_plan(const int32_t *offsets, int32_t segment_count,
                        int32_t value_count, int op, cudaStream_t stream,
                        DevicePlan *dev, HostPlan *host, int32_t *reason,
                        int64_t *index);

// Allocation-free variant: the split schedule run out of a fixed-size
// file-scope device array.  Limits of that array:
constexpr int kStaticMaxSegments = 1 << 18;
constexpr int kStaticMaxTasks = 1 << 15;
constexpr int kStaticMaxSlots = 1 << 15;
constexpr int kStaticMaxSplits = 1 << 13;
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
