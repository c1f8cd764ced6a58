/*
 * swage_b200 -- C ABI of the B200 segmented-reduction / vector-add library.
 *
 * This is the boundary a Swage maintainer binds instead of the reference's
 * "compile to PTX, load with the CUDA Driver, cuLaunchKernel" path:
 *   include/swage-c/Codegen.h:21-31            (swageCompile*ToPTX)
 *   python/SwageExtensionNanobind.cpp:27-99    (_compile_ptx, _compile_segmented_reduction_ptx)
 *   python/swage/_runtime.py:399-531           (_CudaDriver: load / launch / launch_segmented)
 * Kernels are prebuilt for sm_100a; nothing is compiled at run time.
 *
 * Conventions
 *   - plain pointers and sizes only; `stream` is a cudaStream_t / CUstream
 *     passed as void* (the integer PyTorch exposes as stream.cuda_stream);
 *   - every device pointer must belong to the CUDA device that is current on
 *     the calling thread; launches are asynchronous and never synchronise,
 *     copy, cast, switch device or fall back to the CPU;
 *   - every function returns a swg_status (0 = ok); on failure a thread-local
 *     message is available from swg_last_error();
 *   - the library keeps no caller pointer after a call returns; the only
 *     object it owns is swg_plan (until swg_plan_destroy).
 */
#ifndef SWAGE_B200_H
#define SWAGE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SWG_ABI_VERSION 1

typedef enum swg_status {
  SWG_OK = 0,
  SWG_ERR_INVALID_ARGUMENT = 1, /* bad kind / schedule / NULL pointer / negative count */
  SWG_ERR_INVALID_OFFSETS = 2,  /* offsets break the CSR contract */
  SWG_ERR_CUDA = 3,             /* a CUDA runtime call failed; text names it */
  SWG_ERR_PLAN_MISMATCH = 4,    /* plan built for other counts / device / operation */
  SWG_ERR_UNSUPPORTED = 5,      /* schedule needs a plan, or size beyond a stated limit */
  SWG_ERR_DEVICE_TIMEOUT = 6,   /* a bounded device-side wait gave up (read by swg_plan_status) */
  SWG_ERR_DEVICE_CHECK = 7      /* a kernel found a task or segment outside the launch's arrays:
                                   the plan does not belong to these offsets (swg_plan_status) */
} swg_status;

/* Reduction kinds: the two the reference lowers
 * (lib/Conversion/SegmentedReduction/SegmentedReduction.cpp:106-108 rejects the rest). */
#define SWG_KIND_SUM 0 /* identity +0.0f, fp32 add */
#define SWG_KIND_MAX 1 /* identity -inf, NaN-propagating maximum, -0 < +0 */
#define SWG_KIND_MIN 2 /* identity +inf, NaN-propagating minimum, -0 < +0: the
                          dialect's kind<min> (ADR-0008), which the reference's
                          lowering rejects (SegmentedReduction.cpp:106-108) */

/* Element types of segmented reductions.  The reference lowers f32 only
 * (SegmentedReduction.cpp:110-119); its dialect also admits f16, bf16 and
 * integer segments (include/swage/Dialect/Swage/IR/SwageOps.td:101-105).
 * f16 / bf16 values are widened exactly and reduced in fp32, results are fp32;
 * i32 values give i32 results (wrap-around sum, signed max / min). */
#define SWG_DTYPE_F32 0
#define SWG_DTYPE_F16 1
#define SWG_DTYPE_BF16 2
#define SWG_DTYPE_I32 3

/* Element maps in front of a reduction: the dialect's swage.map region feeding
 * a swage.reduce (test/Dialect/Swage/roundtrip.mlir:43-52; the composition of
 * test/Dialect/Swage/softmax.mlir:17-24), which the reference's lowering
 * rejects -- it accepts the identity region only
 * (SegmentedReduction.cpp:106-119).  A map is fn(scale * x + shift) with
 * `scale` and `shift` captured at launch time; the product and the sum are
 * rounded separately (arith.mulf then arith.addf, no contraction).  scale 1
 * and shift -0.0 leave every value, signed zeros included, as it is (+0.0
 * would turn a -0.0 into +0.0). */
#define SWG_MAP_IDENTITY 0 /* y            */
#define SWG_MAP_ABS 1      /* |y|          */
#define SWG_MAP_SQUARE 2   /* y * y        */
#define SWG_MAP_EXP 3      /* exp(y): one multiply and ex2.approx, relative error ~2^-22 */
typedef struct swg_map {
  int32_t fn; /* SWG_MAP_*; y = scale * x + shift */
  float scale;
  float shift;
} swg_map;

/* Operation a plan is built for. */
#define SWG_OP_REDUCE 0
#define SWG_OP_SOFTMAX 1

/* Schedules. AUTO lets the plan (or, without one, the mean segment length)
 * decide.  WARP and CTA need no plan; SPLIT, PERSISTENT and RESIDENT run the
 * plan's tile tasks and therefore need one.  Segments that cross a tile
 * boundary are cut into pieces whose partials a small merge pass, launched
 * right behind the tile kernel, combines in a fixed order. */
#define SWG_SCHED_AUTO 0
#define SWG_SCHED_WARP 1       /* one warp per segment */
#define SWG_SCHED_CTA 2        /* one CTA per segment: the reference's own mapping */
#define SWG_SCHED_SPLIT 3      /* one tile task per warp, two per CTA */
#define SWG_SCHED_PERSISTENT 4 /* one CTA per SM slot, bulk-copy ring, tasks drawn from a ticket counter */
#define SWG_SCHED_RESIDENT 5   /* one CTA per SM, one stage per warp, tile tasks at a fixed stride */

/* Why swg_validate_offsets_i32 rejected an array (order = order of the checks
 * in python/swage/_segmented_qualification.py:30-55). */
#define SWG_OFFSETS_OK 0
#define SWG_OFFSETS_EMPTY 1          /* no initial zero */
#define SWG_OFFSETS_COUNT_RANGE 2    /* value or segment count outside [0, 2^31) */
#define SWG_OFFSETS_OUTPUT_SMALL 3   /* fewer outputs than segments */
#define SWG_OFFSETS_NONZERO_START 4  /* offsets[0] != 0 */
#define SWG_OFFSETS_NEGATIVE 5       /* an offset < 0 */
#define SWG_OFFSETS_DECREASING 6     /* offsets[i] < offsets[i-1] */
#define SWG_OFFSETS_EXCEEDS_VALUES 7 /* offsets[last] > value_count */

typedef struct swg_plan swg_plan;

/* Text of the last failure on this thread ("" when none). */
const char *swg_last_error(void);
const char *swg_status_name(int status);
int swg_abi_version(void);

/* out[i] = x[i] + y[i] for 0 <= i < n.
 * Replaces the generated kernel add_kernel(void*, void*, void*, int32)
 * (lib/Conversion/FixedBlockToGPU/FixedBlockToGPU.cpp:177-226) and its launch
 * (python/swage/_runtime.py:500-503, 511-531).  `block_hint` is the caller's
 * logical BLOCK; it does not change any result bit and only has to be > 0.
 * Pointers may be 4-byte aligned (offset views). n == 0 is a no-op. */
int swg_vadd_f32(const float *x, const float *y, float *out, int32_t n,
                 int32_t block_hint, void *stream);

/* Host-side CSR validation, same rule set and order as
 * python/swage/_segmented_qualification.py:30-55 (_validate_offsets):
 * `count` = number of offsets (segments + 1).  Returns SWG_OK or
 * SWG_ERR_INVALID_OFFSETS with *reason = SWG_OFFSETS_*, *index = first
 * offending position (or -1). reason/index may be NULL. */
int swg_validate_offsets_i32(const int32_t *host_offsets, int64_t count,
                             int64_t value_count, int64_t output_count,
                             int32_t *reason, int64_t *index);

/* Host planner: segment-length histogram -> buckets -> tile tasks -> schedule.
 * `host_offsets` has segment_count + 1 validated entries.  The plan owns
 * device copies of the task list, of the offsets (16-byte aligned and padded,
 * so they can be bulk-copied) and the scratch in which cut segments are
 * merged, all in one block on the current device (taken from the device's
 * stream-ordered memory pool, which the library tells to keep freed memory, so
 * that later plans cost no cudaMalloc).  It is the planned scheduling layer of the reference
 * (its design document, lines 143-151: warp, packed_warp, cta, split_cta,
 * merge, persistent) made concrete.  A plan is valid only for launches whose device
 * offsets hold the same numbers. */
int swg_plan_create(const int32_t *host_offsets, int32_t segment_count,
                    int32_t value_count, int op, swg_plan **plan);
int swg_plan_destroy(swg_plan *plan);
/* JSON text: counts, histogram, bucket shares, task counts, chosen schedule.
 * Returns SWG_ERR_INVALID_ARGUMENT when `capacity` is too small. */
int swg_plan_describe(const swg_plan *plan, char *json, size_t capacity);
/* Synchronises the plan's device and reports what the kernels flagged in any
 * launch since the last call: a bounded wait that gave up
 * (SWG_ERR_DEVICE_TIMEOUT) or a task / segment that does not fit the launch's
 * arrays and was skipped instead of dereferenced (SWG_ERR_DEVICE_CHECK);
 * else SWG_OK.  After an error the plan's counters are cleared, so it can be
 * launched again. */
int swg_plan_status(swg_plan *plan);
/* The same report without any CUDA call or synchronisation: the kernels also
 * leave their first error in pinned host memory, which this reads.  It
 * therefore only knows about launches that have finished; each error is
 * returned once.  Meant to be called before every launch of a cached plan, so
 * that a launch that went wrong is noticed at the next one.  No reference
 * counterpart (the reference's kernels have no device-side checks). */
int swg_plan_peek_status(const swg_plan *plan);

/* Self-test of the kernels' bounded waits: queues a one-warp kernel on `stream`
 * that waits `limit_us` microseconds (1 .. 1e6) for a copy nobody issues and
 * then reports the timeout through the plan's error words, exactly as a tile
 * kernel whose copy never lands would after its two seconds.  Afterwards
 * swg_plan_status returns SWG_ERR_DEVICE_TIMEOUT (and clears it) and
 * swg_plan_peek_status reports it once.  Touches no caller memory; the context
 * stays usable.  No reference counterpart. */
int swg_plan_selftest_timeout(swg_plan *plan, int32_t limit_us, void *stream);

/* The same rules, order and reason codes as swg_validate_offsets_i32, for
 * offsets[0 .. segment_count] that live on the GPU: one pass on the device, one
 * small read-back (`stream` is synchronised).  *hash (optional) receives a
 * 64-bit digest of the offsets' content, *last_offset offsets[segment_count].
 * No reference counterpart: the reference copies the offsets to the host and
 * walks them in Python (python/swage/_segmented_qualification.py:30-55,78) and
 * lists device-only offset validation as future work (its design document,
 * lines 100-102). */
int swg_validate_offsets_device(const int32_t *device_offsets,
                                int32_t segment_count, int32_t value_count,
                                int64_t output_count, void *stream,
                                int32_t *reason, int64_t *index,
                                uint64_t *hash, int32_t *last_offset);

/* swg_plan_create for device-resident offsets: validation (as above), the
 * length histogram, the tile tasks (op = SWG_OP_REDUCE) or the length-class
 * lists (SWG_OP_SOFTMAX) are all computed on the GPU; the offsets are never
 * copied to the host.  On SWG_ERR_INVALID_OFFSETS *reason / *index say which
 * rule broke first and no plan is returned.  `stream` is synchronised once, to
 * read the validation's verdict; the planner's own kernels are only queued on
 * it, so launch the plan on that stream (or order other streams behind it).
 * The tiles are cut at fixed item positions (merge-path), not by the host
 * planner's walk, so the task list differs from swg_plan_create's; results
 * agree to the documented tolerance (max: bit-exact). */
int swg_plan_create_device(const int32_t *device_offsets,
                           int32_t segment_count, int32_t value_count,
                           int64_t output_count, int op, void *stream,
                           swg_plan **plan, int32_t *reason, int64_t *index);

/* swg_plan_create_device for offsets that swg_validate_offsets_device has just
 * accepted on this device, returning `hash`: when that validation is still the
 * latest one on the device and was of the same array, its summary is reused
 * and this call neither reads the offsets a second time nor synchronises --
 * the planner's kernels are queued on `stream` and the call returns.
 * Otherwise it behaves like swg_plan_create_device.  This is what a launch
 * on new offsets costs beyond validation.  No reference counterpart. */
int swg_plan_create_validated(const int32_t *device_offsets,
                              int32_t segment_count, int32_t value_count,
                              int op, void *stream, uint64_t hash,
                              swg_plan **plan);

/* The planner alone, on the host: no device is touched.  Writes up to
 * `task_capacity` tasks as 8 x int32 each {first segment, segment count or
 * partial slot (-1 = whole segment), first value, value count | kind << 28
 * (kind 0 = packed segments, 1 = chunk of one long segment), partial slot of a
 * first segment that began in an earlier task (else -1), partial slot of a
 * last segment that continues in a later task (else -1), first partial slot of
 * the segment a chunk or a first segment belongs to, number of pieces of the
 * segment a chunk or a last segment belongs to}, the total
 * number of tasks to *task_count, and the same JSON as swg_plan_describe.
 * `tasks` and `json` may be NULL.  For inspection and for tests. */
int swg_plan_host_tasks(const int32_t *host_offsets, int32_t segment_count,
                        int op, int32_t *tasks, int64_t task_capacity,
                        int64_t *task_count, char *json, size_t json_capacity);

/* out[s] = reduce(values[offsets[s] .. offsets[s+1])) for 0 <= s < segment_count.
 * Replaces the generated kernels segmented_sum / segmented_max(void* values,
 * void* offsets, void* out, int32 value_count, int32 segment_count)
 * (lib/Conversion/SegmentedReduction/SegmentedReduction.cpp:185-283) and their
 * launch (python/swage/_segmented_qualification.py:154-169,
 * python/swage/_runtime.py:505-509).  Empty segment -> identity.  Only the
 * first segment_count outputs are written.  `plan` may be NULL (then only
 * AUTO / WARP / CTA are accepted).  `block_hint` is the reference's
 * block_size (threads per CTA for the CTA schedule; ignored elsewhere; 0 =
 * library default).  Results are bit-reproducible from run to run for a given
 * schedule and plan (no floating-point atomics). */
int swg_segreduce_f32(int kind, const float *values, const int32_t *offsets,
                      float *out, int32_t value_count, int32_t segment_count,
                      const swg_plan *plan, int schedule, int32_t block_hint,
                      void *stream);

/* swg_segreduce_f32 for the other element types the dialect admits:
 * `values` holds elements of `dtype` (SWG_DTYPE_*), `out` fp32 results for the
 * floating types (f16 / bf16 are widened exactly and reduced in fp32) and
 * int32 results for SWG_DTYPE_I32 (sum wraps around in two's complement --
 * integer addition is associative, so the bits are those of the sequential
 * sum; max / min are signed).  Same plans (a plan does not depend on the
 * element type), same schedules: the tile schedules stage 2048 elements per
 * task whatever their size; without a plan a warp or a CTA reduces each
 * segment.  WARP with a plan and PERSISTENT fall back to SPLIT for these
 * types.  No reference counterpart: the reference's lowering accepts f32
 * only (lib/Conversion/SegmentedReduction/SegmentedReduction.cpp:110-119);
 * identities per its ADR-0008 (lines 34-39). */
int swg_segreduce(int kind, int dtype, const void *values,
                  const int32_t *offsets, void *out, int32_t value_count,
                  int32_t segment_count, const swg_plan *plan, int schedule,
                  int32_t block_hint, void *stream);

/* Map fused into the reduction: out[s] = reduce over the segment of
 * map->fn(map->scale * x + map->shift), each value read once and never
 * written back (a sum of squares, an L1 norm, a max of |x|, the sum of
 * exponentials of a log-sum-exp, ...).  `dtype` is SWG_DTYPE_F32, F16 or BF16
 * (the map acts on the value widened to fp32; results are fp32); integer
 * segments are not mapped.  Same plans and schedules as swg_segreduce; WARP
 * and CTA run the generic warp / CTA-per-segment kernel, PERSISTENT falls
 * back to SPLIT.  An empty segment gives the identity of `kind`, not the map
 * of it.  No reference counterpart (see SWG_MAP_* above). */
int swg_segreduce_map(int kind, int dtype, const swg_map *map,
                      const void *values, const int32_t *offsets, float *out,
                      int32_t value_count, int32_t segment_count,
                      const swg_plan *plan, int schedule, int32_t block_hint,
                      void *stream);

/* A device buffer that other processes of the node can map and store into:
 * what swg_scatter_results_f32 writes to.  create: cudaMalloc on the current
 * device plus its 64-byte CUDA IPC handle, to be sent to the other processes
 * by any means (torch.distributed.all_gather_object does); open: maps a
 * peer's buffer into the CURRENT device's address space (peer access over
 * NVLink is enabled on first use) -- the owner does not open its own; close /
 * destroy undo open / create (close every mapping before the owner destroys).
 * Plumbing, no kernels.  No reference counterpart. */
#define SWG_PEER_HANDLE_BYTES 64
#define SWG_MAX_PEERS 16 /* destinations of one scatter / fused launch */
int swg_peer_buffer_create(int64_t bytes, void **buffer, unsigned char *handle);
int swg_peer_buffer_open(const unsigned char *handle, void **buffer);
int swg_peer_buffer_close(void *buffer);
int swg_peer_buffer_destroy(void *buffer);

/* Result exchange of a sharded reduction without a collective:
 * dst_bases[p][dst_offset + i] = src[i] for 0 <= p < dst_count (at most 16),
 * 0 <= i < count.  `src` is this GPU's result shard; the destinations are
 * device pointers to every GPU's copy of the full result array -- this GPU's
 * own and its peers', mapped into this process through CUDA IPC or peer
 * access -- each 16-byte aligned at its base.  One kernel on `stream`, queued
 * behind the reduction; over NVLink it issues plain 128-bit stores only: no
 * multicast, no load from peer memory, no wait on another GPU.  A destination
 * is complete when this call's stream has passed the call; telling the peers
 * so (a barrier, an event) is the caller's.  No reference counterpart: the
 * reference is single-GPU (python/swage/_runtime.py:146-151). */
int swg_scatter_results_f32(const float *src, int64_t count,
                            void *const *dst_bases, int32_t dst_count,
                            int64_t dst_offset, void *stream);

/* Reduction and result exchange in one launch: swg_segreduce_f32 with a plan,
 * except that the result of segment s is stored by the reducing warp (or by
 * the merge pass, for a segment cut across tiles) at
 * dst_bases[p][dst_offset + s] for EVERY destination p -- this GPU's copy of
 * the full result array of a sharded reduction and its peers' copies
 * (swg_peer_buffer_open) -- instead of a local out[s].  The stores over
 * NVLink ride along with the reduction: no collective, no copy kernel, plain
 * st.global only (no multicast, no load from peer memory, no wait on another
 * GPU).  Tile schedules only (SPLIT or RESIDENT; anything else runs SPLIT), so
 * a plan is required.  Same bits as swg_segreduce_f32 with that plan and
 * schedule.  Completion on the peers as for swg_scatter_results_f32.  No
 * reference counterpart. */
int swg_segreduce_peers_f32(int kind, const float *values,
                            const int32_t *offsets, void *const *dst_bases,
                            int32_t dst_count, int64_t dst_offset,
                            int32_t value_count, int32_t segment_count,
                            const swg_plan *plan, int schedule, void *stream);

/* Sum AND max of every segment in one pass over the values:
 * out_sum[s] = swg_segreduce_f32(SWG_KIND_SUM)[s] to the documented tolerance,
 * out_max[s] = swg_segreduce_f32(SWG_KIND_MAX)[s] bit for bit, for
 * 0 <= s < segment_count; each value is read once and the call is one kernel
 * launch.  Plan-free (a warp or a CTA per segment, chosen by the mean length):
 * meant for inputs of moderate size such as the canonical 4096-segment
 * configuration, where two separate launches cost more than the data.  This
 * entry point has no counterpart in the reference, which runs the two kinds
 * as two kernels; identities and combiners are those of
 * lib/Conversion/SegmentedReduction/SegmentedReduction.cpp:156-161, 236-267. */
int swg_segreduce_sum_max_f32(const float *values, const int32_t *offsets,
                              float *out_sum, float *out_max,
                              int32_t value_count, int32_t segment_count,
                              void *stream);

/* Same result as swg_segreduce_f32 with a plan and SWG_SCHED_SPLIT, for
 * callers that must not allocate device memory: code running inside a
 * framework whose memory pool already owns the GPU's memory, a serving loop
 * that cannot afford cudaMalloc's implicit synchronisation, or a client whose
 * allocations are capped by its host process.  This entry point has no
 * counterpart in the reference.
 *
 * The planner runs on the host from `host_offsets` (segment_count + 1 entries,
 * validated here) and the task list, an aligned copy of the offsets and the
 * list and partials of cut segments are placed in a fixed array that is part of
 * the library image on every GPU (2,490,880 bytes, about 2.5 MB, held until
 * the process exits).  No cudaMalloc, cudaFree or other allocating call is
 * made.
 * Limits: at most 262144 segments, 32768 tile tasks (about 6.6e7 values) and
 * 32768 partials of cut segments; larger inputs are rejected with
 * SWG_ERR_UNSUPPORTED and a message naming the limit.
 * The first call on a device looks up the array's device address; that first
 * call should come before any stream capture.  Every call copies the offsets
 * and the task list from host memory on `stream`: `host_offsets` must stay
 * unchanged until `stream` has passed the call (a pinned buffer is read by the
 * copy engine after the call has returned).  All calls share the array, which
 * keeps the last call's contents (the parts that must start at zero are
 * cleared on `stream` each time), so two calls that can overlap on the GPU --
 * different streams, or different host threads -- race: serialise them.
 * The kernel's device-side checks write their verdict into the array; it is
 * not read back (the tasks are built from the very offsets passed in, so only
 * the two-second wait limit could trip). */
int swg_segreduce_f32_noalloc(int kind, const float *values,
                              const int32_t *host_offsets, float *out,
                              int32_t value_count, int32_t segment_count,
                              void *stream);

/* out[i] = exp(values[i] - m_s) / d_s over each segment s, with m_s the
 * segment maximum and d_s the sum of exp(values - m_s); empty segments write
 * nothing; positions outside every segment are not touched.  `out` must not
 * alias `values`.  The reference defines this only as a semantic form
 * (test/Dialect/Swage/softmax.mlir:13-31; roadmap M5) and has no lowering. */
int swg_segsoftmax_f32(const float *values, const int32_t *offsets, float *out,
                       int32_t value_count, int32_t segment_count,
                       const swg_plan *plan, int schedule, void *stream);

/* Cut segment_count segments into `shards` contiguous ranges balanced by
 * element count: shard g owns segments [seg_begin[g], seg_begin[g+1]).
 * seg_begin has shards + 1 entries.  No reference counterpart (the reference
 * is single-GPU: python/swage/_runtime.py:146-151); it is the sharding rule of
 * the multi-GPU path. */
int swg_shard_offsets(const int32_t *host_offsets, int32_t segment_count,
                      int32_t shards, int32_t *seg_begin);

/* Per-launch device timing of the dominant kernel of every call made between
 * start and stop (the tile kernel of a planned reduce, not its combine pass;
 * the only kernel otherwise).  The library records a pair of CUDA events
 * around that kernel on the launch stream.  swg_profile_stop synchronises
 * those events, writes up to `capacity` durations in milliseconds and the
 * number of launches recorded.  Every `stride`-th call is recorded (stride 1 =
 * every call; a pair of event records costs a few microseconds of stream
 * time, so a sparse sample perturbs a timed loop less), at most `capacity` of
 * them; the rest run untimed.  No reference counterpart: the reference
 * has no timing facility (its debugging switches are the SWAGE_DUMP_*
 * variables, python/swage/_runtime.py:381-396). */
int swg_profile_start(int32_t capacity, int32_t stride);
int swg_profile_stop(float *milliseconds, int32_t capacity, int32_t *count);

#ifdef __cplusplus
}
#endif

#endif /* SWAGE_B200_H */
