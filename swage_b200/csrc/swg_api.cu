// extern "C" entry points declared in include/swage_b200.h.
#include <algorithm>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "swg_common.cuh"
#include "swg_launch.h"

struct swg_plan {
  swg::HostPlan host;
  swg::DevicePlan dev;
  // the stream of the launches so far (the plan's memory is freed behind it)
  mutable cudaStream_t last_stream = nullptr;
  mutable bool launched = false;
  mutable bool many_streams = false;
  // device planner: the task statistics are fetched when first asked for
  mutable bool counts_known = true;
};

namespace {

struct DeviceInfo {
  bool ready = false;
  bool configured = false;  // kernel attributes are per device
  int sm_count = 0;
};

std::mutex g_lock;
DeviceInfo g_devices[64];

// Per-launch timing (swg_profile_start / swg_profile_stop).
struct Profile {
  bool active = false;
  std::vector<swg::Probe> probes;
  size_t used = 0;
  int64_t calls = 0;
  int64_t stride = 1;
};
Profile g_profile;

const swg::Probe *next_probe() {
  std::lock_guard<std::mutex> guard(g_lock);
  if (!g_profile.active) return nullptr;
  const bool sampled = (g_profile.calls++ % g_profile.stride) == 0;
  if (!sampled || g_profile.used >= g_profile.probes.size()) return nullptr;
  return &g_profile.probes[g_profile.used++];
}

void drop_probes() {
  for (swg::Probe &probe : g_profile.probes) {
    cudaEventDestroy(probe.start);
    cudaEventDestroy(probe.stop);
  }
  g_profile.probes.clear();
  g_profile.used = 0;
  g_profile.calls = 0;
  g_profile.active = false;
}

int cuda_failure(const char *what, cudaError_t error) {
  swg::set_error("%s failed: %s (%d): %s", what, cudaGetErrorName(error),
                 (int)error, cudaGetErrorString(error));
  return SWG_ERR_CUDA;
}

// Current device + its SM count; configures kernel attributes once.
int current_device(int *device, int *sm_count) {
  cudaError_t e = cudaGetDevice(device);
  if (e != cudaSuccess) return cuda_failure("cudaGetDevice", e);
  if (*device < 0 || *device >= 64) {
    swg::set_error("device index %d out of range", *device);
    return SWG_ERR_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> guard(g_lock);
  DeviceInfo &info = g_devices[*device];
  if (!info.ready) {
    e = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount,
                               *device);
    if (e != cudaSuccess) return cuda_failure("cudaDeviceGetAttribute", e);
    info.ready = true;
  }
  if (!info.configured) {
    e = swg::configure_segreduce_kernels();
    if (e == cudaSuccess) e = swg::configure_softmax_kernels();
    if (e != cudaSuccess) return cuda_failure("cudaFuncSetAttribute", e);
    info.configured = true;
  }
  *sm_count = info.sm_count;
  return SWG_OK;
}

// Host-visible error words, one pair per plan: a page of pinned, mapped
// memory per device, handed out in 8-byte slots.
struct StatusPool {
  uint32_t *page = nullptr;
  std::vector<int> free_slots;
  bool tried = false;
};
constexpr int kStatusSlots = 512;
StatusPool g_status[64];

uint32_t *status_acquire(int device) {
  std::lock_guard<std::mutex> guard(g_lock);
  StatusPool &pool = g_status[device];
  if (!pool.tried) {
    pool.tried = true;
    void *page = nullptr;
    if (cudaHostAlloc(&page, kStatusSlots * 8, cudaHostAllocMapped |
                                                   cudaHostAllocPortable) ==
        cudaSuccess) {
      pool.page = static_cast<uint32_t *>(page);
      memset(page, 0, kStatusSlots * 8);
      for (int i = kStatusSlots - 1; i >= 0; --i) pool.free_slots.push_back(i);
    } else {
      cudaGetLastError();
    }
  }
  if (pool.page == nullptr || pool.free_slots.empty()) return nullptr;
  const int slot = pool.free_slots.back();
  pool.free_slots.pop_back();
  uint32_t *words = pool.page + 2 * slot;
  words[0] = words[1] = 0;
  return words;
}

void status_release(int device, uint32_t *words) {
  if (words == nullptr) return;
  std::lock_guard<std::mutex> guard(g_lock);
  StatusPool &pool = g_status[device];
  pool.free_slots.push_back((int)((words - pool.page) / 2));
}

// Tells the plan's kernels where the host-visible error words are.
cudaError_t status_attach(swg::DevicePlan *dev, cudaStream_t stream) {
  dev->host_status = status_acquire(dev->device);
  if (dev->host_status == nullptr || dev->control == nullptr)
    return cudaSuccess;
  void *seen_by_device = nullptr;
  cudaError_t e =
      cudaHostGetDevicePointer(&seen_by_device, dev->host_status, 0);
  if (e != cudaSuccess) return e;
  const unsigned long long address =
      (unsigned long long)(uintptr_t)seen_by_device;
  // (a small copy from pageable memory is staged before the call returns)
  return cudaMemcpyAsync(dev->control + swg::kStatusWord, &address,
                         sizeof(address), cudaMemcpyHostToDevice, stream);
}

void release(swg_plan *plan) {
  swg::DevicePlan &dev = plan->dev;
  status_release(dev.device, dev.host_status);
  swg::plan_block_release(&dev, plan->last_stream,
                          plan->launched && !plan->many_streams);
  dev = swg::DevicePlan();
}

void note_launch(const swg_plan *plan, cudaStream_t stream) {
  if (plan->launched && plan->last_stream != stream)
    plan->many_streams = true;
  plan->last_stream = stream;
  plan->launched = true;
}

std::string describe(const swg_plan *plan) {
  if (!plan->counts_known) {
    int64_t chunks = 0, cuts = 0;
    if (swg::device_plan_counts(plan->dev, &chunks, &cuts) == cudaSuccess) {
      swg_plan *writable = const_cast<swg_plan *>(plan);
      writable->host.chunk_tasks = chunks;
      writable->host.pack_tasks = plan->host.task_total - chunks;
      writable->host.split_segments = cuts;
      writable->counts_known = true;
    }
  }
  return swg::describe_host_plan(plan->host);
}

constexpr size_t aligned256(size_t bytes) { return (bytes + 255) / 256 * 256; }

}  // namespace

extern "C" {

const char *swg_last_error(void) { return swg::last_error_text(); }

const char *swg_status_name(int status) {
  switch (status) {
    case SWG_OK: return "SWG_OK";
    case SWG_ERR_INVALID_ARGUMENT: return "SWG_ERR_INVALID_ARGUMENT";
    case SWG_ERR_INVALID_OFFSETS: return "SWG_ERR_INVALID_OFFSETS";
    case SWG_ERR_CUDA: return "SWG_ERR_CUDA";
    case SWG_ERR_PLAN_MISMATCH: return "SWG_ERR_PLAN_MISMATCH";
    case SWG_ERR_UNSUPPORTED: return "SWG_ERR_UNSUPPORTED";
    case SWG_ERR_DEVICE_TIMEOUT: return "SWG_ERR_DEVICE_TIMEOUT";
    case SWG_ERR_DEVICE_CHECK: return "SWG_ERR_DEVICE_CHECK";
    default: return "SWG_ERR_UNKNOWN";
  }
}

int swg_abi_version(void) { return SWG_ABI_VERSION; }

int swg_vadd_f32(const float *x, const float *y, float *out, int32_t n,
                 int32_t block_hint, void *stream) {
  swg::clear_error();
  if (n < 0 || block_hint <= 0) {
    swg::set_error("swg_vadd_f32: n must be >= 0 and block_hint > 0");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (n == 0) return SWG_OK;
  if (!x || !y || !out) {
    swg::set_error("swg_vadd_f32: null pointer");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  cudaError_t e = swg::launch_vadd(x, y, out, n, (cudaStream_t)stream,
                                   next_probe());
  if (e != cudaSuccess) return cuda_failure("vector add launch", e);
  return SWG_OK;
}

int swg_validate_offsets_i32(const int32_t *host_offsets, int64_t count,
                             int64_t value_count, int64_t output_count,
                             int32_t *reason, int64_t *index) {
  swg::clear_error();
  return swg::validate_offsets(host_offsets, count, value_count, output_count,
                               reason, index);
}

int swg_plan_create(const int32_t *host_offsets, int32_t segment_count,
                    int32_t value_count, int op, swg_plan **plan_out) {
  swg::clear_error();
  if (!plan_out) {
    swg::set_error("swg_plan_create: plan is null");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  *plan_out = nullptr;
  if (!host_offsets || segment_count < 0 || value_count < 0 ||
      (op != SWG_OP_REDUCE && op != SWG_OP_SOFTMAX)) {
    swg::set_error("swg_plan_create: bad arguments");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  int status = swg::validate_offsets(host_offsets, (int64_t)segment_count + 1,
                                     value_count, segment_count, nullptr,
                                     nullptr);
  if (status != SWG_OK) return status;
  int device = 0, sm_count = 0;
  status = current_device(&device, &sm_count);
  if (status != SWG_OK) return status;

  swg_plan *plan = new (std::nothrow) swg_plan();
  if (!plan) {
    swg::set_error("swg_plan_create: out of host memory");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  swg::build_host_plan(host_offsets, segment_count, op, &plan->host);
  swg::DevicePlan &dev = plan->dev;
  dev.device = device;
  dev.sm_count = sm_count;
  dev.task_count = (int32_t)plan->host.tasks.size();
  dev.segment_count = segment_count;
  dev.partial_slots = plan->host.partial_slots;
  dev.slot_step = plan->host.slot_step;
  for (int b = 0; b < swg::kSoftmaxBuckets; ++b) {
    dev.softmax_begin[b] = plan->host.softmax_begin[b];
    dev.softmax_count[b] = plan->host.softmax_count[b];
  }
  // one block: padded offsets, control words, tasks, merge records, partials,
  // softmax class lists
  const size_t noffsets = (size_t)segment_count + 1;
  const size_t padded = ((noffsets + 3) / 4) * 4 + 4;
  const size_t offsets_bytes = aligned256(padded * sizeof(int32_t));
  const size_t control_bytes =
      aligned256(swg::kControlWords * sizeof(uint32_t) + sizeof(int32_t));
  const size_t task_bytes =
      aligned256(plan->host.tasks.size() * sizeof(swg::Task));
  const size_t merge_bytes =
      aligned256(plan->host.merges.size() * sizeof(swg::MergeRecord));
  const size_t big_bytes =
      aligned256(plan->host.big_merges.size() * sizeof(swg::MergeRecord));
  const size_t slot_bytes =
      aligned256((size_t)dev.partial_slots * sizeof(float));
  const size_t list_bytes =
      aligned256(plan->host.softmax_segments.size() * sizeof(int32_t));
  cudaError_t e = swg::plan_block_allocate(
      &dev,
      offsets_bytes + control_bytes + task_bytes + merge_bytes + big_bytes +
          slot_bytes + list_bytes,
      nullptr);
  if (e == cudaSuccess) e = cudaMemset(dev.block, 0, dev.block_bytes);
  if (e == cudaSuccess) {
    unsigned char *at = static_cast<unsigned char *>(dev.block);
    dev.offsets = reinterpret_cast<int32_t *>(at);
    at += offsets_bytes;
    dev.control = reinterpret_cast<uint32_t *>(at);
    dev.big_count = reinterpret_cast<int32_t *>(dev.control + swg::kControlWords);
    at += control_bytes;
    dev.tasks = reinterpret_cast<swg::Task *>(at);
    at += task_bytes;
    dev.merges = reinterpret_cast<swg::MergeRecord *>(at);
    dev.merge_count = (int32_t)plan->host.merges.size();
    at += merge_bytes;
    dev.bigs = reinterpret_cast<swg::MergeRecord *>(at);
    dev.big_capacity = (int32_t)plan->host.big_merges.size();
    at += big_bytes;
    dev.partials = reinterpret_cast<float *>(at);
    at += slot_bytes;
    dev.softmax_segments = reinterpret_cast<int32_t *>(at);
    e = cudaMemcpy(dev.offsets, host_offsets, noffsets * sizeof(int32_t),
                   cudaMemcpyHostToDevice);
  }
  if (e == cudaSuccess && !plan->host.tasks.empty())
    e = cudaMemcpy(dev.tasks, plan->host.tasks.data(),
                   plan->host.tasks.size() * sizeof(swg::Task),
                   cudaMemcpyHostToDevice);
  if (e == cudaSuccess && !plan->host.merges.empty())
    e = cudaMemcpy(dev.merges, plan->host.merges.data(),
                   plan->host.merges.size() * sizeof(swg::MergeRecord),
                   cudaMemcpyHostToDevice);
  if (e == cudaSuccess && !plan->host.big_merges.empty())
    e = cudaMemcpy(dev.bigs, plan->host.big_merges.data(),
                   plan->host.big_merges.size() * sizeof(swg::MergeRecord),
                   cudaMemcpyHostToDevice);
  if (e == cudaSuccess)
    e = cudaMemcpy(dev.big_count, &dev.big_capacity, sizeof(int32_t),
                   cudaMemcpyHostToDevice);
  if (e == cudaSuccess && !plan->host.softmax_segments.empty())
    e = cudaMemcpy(dev.softmax_segments, plan->host.softmax_segments.data(),
                   plan->host.softmax_segments.size() * sizeof(int32_t),
                   cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = status_attach(&dev, nullptr);
  if (e == cudaSuccess) e = cudaStreamSynchronize(nullptr);
  if (e != cudaSuccess) {
    release(plan);
    delete plan;
    return cuda_failure("plan upload", e);
  }
  // host vectors are no longer needed once uploaded
  plan->host.task_total = (int64_t)plan->host.tasks.size();
  std::vector<swg::Task>().swap(plan->host.tasks);
  std::vector<swg::MergeRecord>().swap(plan->host.merges);
  std::vector<swg::MergeRecord>().swap(plan->host.big_merges);
  std::vector<int32_t>().swap(plan->host.softmax_segments);
  *plan_out = plan;
  return SWG_OK;
}

// The checks of validate_offsets that need no offset value, in its order.
static int precheck_counts(const void *offsets, int64_t segment_count,
                           int64_t value_count, int64_t output_count,
                           int32_t *reason, int64_t *index) {
  const int64_t limit = int64_t(1) << 31;
  int32_t why = SWG_OFFSETS_OK;
  if (!offsets || segment_count < 0) why = SWG_OFFSETS_EMPTY;
  else if (value_count < 0 || value_count >= limit || segment_count >= limit)
    why = SWG_OFFSETS_COUNT_RANGE;
  else if (output_count < segment_count) why = SWG_OFFSETS_OUTPUT_SMALL;
  if (reason) *reason = why;
  if (index) *index = -1;
  if (why == SWG_OFFSETS_OK) return SWG_OK;
  swg::set_error("offsets rejected: reason %d at index -1", (int)why);
  return SWG_ERR_INVALID_OFFSETS;
}

int swg_validate_offsets_device(const int32_t *device_offsets,
                                int32_t segment_count, int32_t value_count,
                                int64_t output_count, void *stream,
                                int32_t *reason, int64_t *index,
                                uint64_t *hash, int32_t *last_offset) {
  swg::clear_error();
  int status = precheck_counts(device_offsets, segment_count, value_count,
                               output_count, reason, index);
  if (status != SWG_OK) return status;
  int device = 0, sm_count = 0;
  status = current_device(&device, &sm_count);
  if (status != SWG_OK) return status;
  int32_t why = SWG_OFFSETS_OK;
  int64_t where = -1;
  swg::DeviceDigest digest{0, 0, 0};
  cudaError_t e = swg::device_validate(device_offsets, segment_count,
                                       value_count, device, sm_count,
                                       (cudaStream_t)stream, &why, &where,
                                       &digest);
  if (e != cudaSuccess) return cuda_failure("device offsets validation", e);
  if (reason) *reason = why;
  if (index) *index = where;
  if (hash) *hash = digest.hash;
  if (last_offset) *last_offset = digest.last_offset;
  if (why == SWG_OFFSETS_OK) return SWG_OK;
  swg::set_error("offsets rejected: reason %d at index %lld", (int)why,
                 (long long)where);
  return SWG_ERR_INVALID_OFFSETS;
}

static int create_on_device(const char *who, const int32_t *device_offsets,
                            int32_t segment_count, int32_t value_count,
                            int64_t output_count, int op, void *stream,
                            const unsigned long long *known_hash,
                            swg_plan **plan_out, int32_t *reason,
                            int64_t *index) {
  swg::clear_error();
  if (!plan_out || (op != SWG_OP_REDUCE && op != SWG_OP_SOFTMAX)) {
    swg::set_error("%s: bad arguments", who);
    return SWG_ERR_INVALID_ARGUMENT;
  }
  *plan_out = nullptr;
  int status = precheck_counts(device_offsets, segment_count, value_count,
                               output_count, reason, index);
  if (status != SWG_OK) return status;
  int device = 0, sm_count = 0;
  status = current_device(&device, &sm_count);
  if (status != SWG_OK) return status;
  swg_plan *plan = new (std::nothrow) swg_plan();
  if (!plan) {
    swg::set_error("%s: out of host memory", who);
    return SWG_ERR_INVALID_ARGUMENT;
  }
  plan->dev.device = device;
  plan->dev.sm_count = sm_count;
  int32_t why = SWG_OFFSETS_OK;
  int64_t where = -1;
  cudaError_t e = swg::device_plan(device_offsets, segment_count, value_count,
                                   op, (cudaStream_t)stream, known_hash,
                                   &plan->dev, &plan->host, &why, &where);
  if (e == cudaSuccess && why == SWG_OFFSETS_OK)
    e = status_attach(&plan->dev, (cudaStream_t)stream);
  if (reason) *reason = why;
  if (index) *index = where;
  if (e != cudaSuccess || why != SWG_OFFSETS_OK) {
    release(plan);
    delete plan;
    if (e != cudaSuccess) return cuda_failure("device planner", e);
    swg::set_error("offsets rejected: reason %d at index %lld", (int)why,
                   (long long)where);
    return SWG_ERR_INVALID_OFFSETS;
  }
  // the planner's kernels are queued on `stream`; launches of the plan on
  // that stream follow them, and the plan's memory is released behind it
  note_launch(plan, (cudaStream_t)stream);
  plan->counts_known = op != SWG_OP_REDUCE;
  *plan_out = plan;
  return SWG_OK;
}

int swg_plan_create_device(const int32_t *device_offsets,
                           int32_t segment_count, int32_t value_count,
                           int64_t output_count, int op, void *stream,
                           swg_plan **plan_out, int32_t *reason,
                           int64_t *index) {
  return create_on_device("swg_plan_create_device", device_offsets,
                          segment_count, value_count, output_count, op, stream,
                          nullptr, plan_out, reason, index);
}

int swg_plan_create_validated(const int32_t *device_offsets,
                              int32_t segment_count, int32_t value_count,
                              int op, void *stream, uint64_t hash,
                              swg_plan **plan_out) {
  const unsigned long long known = hash;
  return create_on_device("swg_plan_create_validated", device_offsets,
                          segment_count, value_count, segment_count, op,
                          stream, &known, plan_out, nullptr, nullptr);
}

int swg_plan_host_tasks(const int32_t *host_offsets, int32_t segment_count,
                        int op, int32_t *tasks, int64_t task_capacity,
                        int64_t *task_count, char *json, size_t json_capacity) {
  swg::clear_error();
  if (!host_offsets || segment_count < 0 ||
      (op != SWG_OP_REDUCE && op != SWG_OP_SOFTMAX)) {
    swg::set_error("swg_plan_host_tasks: bad arguments");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  int status = swg::validate_offsets(
      host_offsets, (int64_t)segment_count + 1,
      host_offsets[segment_count] < 0 ? 0 : host_offsets[segment_count],
      segment_count, nullptr, nullptr);
  if (status != SWG_OK) return status;
  swg::HostPlan plan;
  swg::build_host_plan(host_offsets, segment_count, op, &plan);
  if (task_count) *task_count = (int64_t)plan.tasks.size();
  if (tasks) {
    const int64_t n = std::min<int64_t>(task_capacity, plan.tasks.size());
    static_assert(sizeof(swg::Task) == 32, "task is eight 32-bit words");
    memcpy(tasks, plan.tasks.data(), (size_t)n * sizeof(swg::Task));
  }
  if (json) {
    const std::string text = swg::describe_host_plan(plan);
    if (json_capacity <= text.size()) {
      swg::set_error("swg_plan_host_tasks: need %zu bytes", text.size() + 1);
      return SWG_ERR_INVALID_ARGUMENT;
    }
    memcpy(json, text.c_str(), text.size() + 1);
  }
  return SWG_OK;
}

int swg_plan_destroy(swg_plan *plan) {
  swg::clear_error();
  if (!plan) return SWG_OK;
  int previous = -1;
  const int owner = plan->dev.device;
  cudaGetDevice(&previous);
  if (owner >= 0 && previous != owner) cudaSetDevice(owner);
  release(plan);
  if (previous >= 0 && previous != owner) cudaSetDevice(previous);
  delete plan;
  return SWG_OK;
}

int swg_plan_describe(const swg_plan *plan, char *json, size_t capacity) {
  swg::clear_error();
  if (!plan || !json) {
    swg::set_error("swg_plan_describe: null argument");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  const std::string text = describe(plan);
  if (capacity <= text.size()) {
    swg::set_error("swg_plan_describe: need %zu bytes", text.size() + 1);
    return SWG_ERR_INVALID_ARGUMENT;
  }
  memcpy(json, text.c_str(), text.size() + 1);
  return SWG_OK;
}

// The message and status for an error code left by a kernel.
static int device_error(uint32_t code, uint32_t detail) {
  const char *what = code == 1 ? "a bounded device-side wait gave up"
                     : code == 2
                         ? "a task of the plan does not fit the launch's "
                           "arrays"
                         : "the device offsets do not match the plan";
  swg::set_error("%s (code %u, detail %u)", what, code, detail);
  return code == 1 ? SWG_ERR_DEVICE_TIMEOUT : SWG_ERR_DEVICE_CHECK;
}

int swg_plan_selftest_timeout(swg_plan *plan, int32_t limit_us, void *stream) {
  swg::clear_error();
  if (!plan || limit_us < 1 || limit_us > 1000000) {
    swg::set_error(
        "swg_plan_selftest_timeout: needs a plan and a limit of 1 .. 1e6 us");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  int device = 0, sm_count = 0;
  const int status = current_device(&device, &sm_count);
  if (status != SWG_OK) return status;
  if (plan->dev.device != device || plan->dev.control == nullptr) {
    swg::set_error("swg_plan_selftest_timeout: plan of another device");
    return SWG_ERR_PLAN_MISMATCH;
  }
  note_launch(plan, (cudaStream_t)stream);
  const cudaError_t e = swg::launch_wait_selftest(
      plan->dev, (uint64_t)limit_us * 1000ull, (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_failure("wait self-test launch", e);
  return SWG_OK;
}

int swg_plan_peek_status(const swg_plan *plan) {
  swg::clear_error();
  if (!plan) {
    swg::set_error("swg_plan_peek_status: plan is null");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  volatile uint32_t *words = plan->dev.host_status;
  if (words == nullptr || words[0] == 0) return SWG_OK;
  const uint32_t code = words[0], detail = words[1];
  words[0] = 0;  // reported once here; swg_plan_status still sees it
  return device_error(code, detail);
}

int swg_plan_status(swg_plan *plan) {
  swg::clear_error();
  if (!plan) {
    swg::set_error("swg_plan_status: plan is null");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  // the plan's own device, whichever one is current on this thread
  int previous = -1;
  const int owner = plan->dev.device;
  cudaGetDevice(&previous);
  const bool switched = owner >= 0 && previous != owner;
  if (switched) cudaSetDevice(owner);
  uint32_t control[4] = {0, 0, 0, 0};
  cudaError_t e = cudaDeviceSynchronize();
  const char *failed = "cudaDeviceSynchronize";
  if (e == cudaSuccess) {
    e = cudaMemcpy(control, plan->dev.control, sizeof(control),
                   cudaMemcpyDeviceToHost);
    failed = "cudaMemcpy";
  }
  // an error leaves the ticket and finished counters of the persistent
  // schedule wherever the kernel stopped: start the next launch from zero
  if (e == cudaSuccess && control[2] != 0) {
    cudaMemset(plan->dev.control, 0, sizeof(control));
    if (plan->dev.host_status != nullptr) plan->dev.host_status[0] = 0;
  }
  if (switched && previous >= 0) cudaSetDevice(previous);
  if (e != cudaSuccess) return cuda_failure(failed, e);
  if (control[2] != 0) return device_error(control[2], control[3]);
  return SWG_OK;
}

static int segreduce(const char *who, int kind, int dtype, const void *values,
                     const int32_t *offsets, void *out, int32_t value_count,
                     int32_t segment_count, const swg_plan *plan, int schedule,
                     int32_t block_hint, void *stream,
                     const swg_map *map = nullptr) {
  swg::clear_error();
  if (map) {
    if (map->fn < SWG_MAP_IDENTITY || map->fn > SWG_MAP_EXP) {
      swg::set_error("%s: map function must be one of SWG_MAP_*", who);
      return SWG_ERR_INVALID_ARGUMENT;
    }
    if (dtype == SWG_DTYPE_I32) {
      swg::set_error("%s: integer segments are not mapped", who);
      return SWG_ERR_UNSUPPORTED;
    }
  }
  if (kind != SWG_KIND_SUM && kind != SWG_KIND_MAX && kind != SWG_KIND_MIN) {
    swg::set_error(
        "reduction kind must be SWG_KIND_SUM, SWG_KIND_MAX or SWG_KIND_MIN");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (dtype < SWG_DTYPE_F32 || dtype > SWG_DTYPE_I32) {
    swg::set_error("%s: element type must be one of SWG_DTYPE_*", who);
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (value_count < 0 || segment_count < 0 || block_hint < 0 ||
      schedule < SWG_SCHED_AUTO || schedule > SWG_SCHED_RESIDENT) {
    swg::set_error("%s: bad count, block or schedule", who);
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (segment_count == 0) return SWG_OK;
  if (!offsets || !out || (!values && value_count > 0)) {
    swg::set_error("%s: null pointer", who);
    return SWG_ERR_INVALID_ARGUMENT;
  }
  int device = 0, sm_count = 0;
  int status = current_device(&device, &sm_count);
  if (status != SWG_OK) return status;
  if (plan) {
    if (plan->host.op != SWG_OP_REDUCE ||
        plan->host.segment_count != segment_count ||
        plan->host.value_count > value_count || plan->dev.device != device) {
      swg::set_error(
          "plan was built for %d segments / %d values on device %d, launch "
          "has %d segments / %d values on device %d",
          plan->host.segment_count, plan->host.value_count, plan->dev.device,
          segment_count, value_count, device);
      return SWG_ERR_PLAN_MISMATCH;
    }
    if (schedule == SWG_SCHED_AUTO) schedule = plan->host.schedule;
    // the plan-free and ticketed schedules exist for f32 only: the other
    // element types run the same tile tasks on the split schedule instead
    if (dtype != SWG_DTYPE_F32 &&
        (schedule == SWG_SCHED_WARP || schedule == SWG_SCHED_PERSISTENT))
      schedule = SWG_SCHED_SPLIT;
    if (map && schedule == SWG_SCHED_PERSISTENT) schedule = SWG_SCHED_SPLIT;
  } else {
    if (schedule == SWG_SCHED_SPLIT || schedule == SWG_SCHED_PERSISTENT ||
        schedule == SWG_SCHED_RESIDENT) {
      swg::set_error(
          "the split, persistent and resident schedules need a plan");
      return SWG_ERR_UNSUPPORTED;
    }
    if (schedule == SWG_SCHED_AUTO)
      schedule = (int64_t)value_count >= (int64_t)segment_count * 2048
                     ? SWG_SCHED_CTA
                     : SWG_SCHED_WARP;
  }
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
  const swg::Probe *probe = next_probe();
  if (plan) note_launch(plan, s);
  const bool f32 = dtype == SWG_DTYPE_F32;
  switch (schedule) {
    case SWG_SCHED_WARP:
    case SWG_SCHED_CTA:
      if (!f32 || map)
        e = swg::launch_segreduce_typed(kind, dtype, values, offsets, out,
                                        value_count, segment_count,
                                        schedule == SWG_SCHED_CTA, sm_count, s,
                                        probe, map);
      else if (schedule == SWG_SCHED_WARP)
        e = swg::launch_segreduce_warp(kind, (const float *)values, offsets,
                                       (float *)out, segment_count, sm_count,
                                       s, probe);
      else
        e = swg::launch_segreduce_cta(kind, (const float *)values, offsets,
                                      (float *)out, segment_count, block_hint,
                                      sm_count, s, probe);
      break;
    case SWG_SCHED_SPLIT:
      e = swg::launch_segreduce_split(kind, dtype, values, out, value_count,
                                      plan->dev, s, probe, map);
      break;
    case SWG_SCHED_RESIDENT:
      e = swg::launch_segreduce_resident(kind, dtype, values, out, value_count,
                                         plan->dev, s, probe, map);
      break;
    default:
      e = swg::launch_segreduce_persistent(kind, (const float *)values,
                                           (float *)out, value_count,
                                           plan->dev, s, probe);
      break;
  }
  if (e != cudaSuccess) return cuda_failure("segmented reduce launch", e);
  return SWG_OK;
}

int swg_segreduce_f32(int kind, const float *values, const int32_t *offsets,
                      float *out, int32_t value_count, int32_t segment_count,
                      const swg_plan *plan, int schedule, int32_t block_hint,
                      void *stream) {
  return segreduce("swg_segreduce_f32", kind, SWG_DTYPE_F32, values, offsets,
                   out, value_count, segment_count, plan, schedule, block_hint,
                   stream);
}

int swg_segreduce(int kind, int dtype, const void *values,
                  const int32_t *offsets, void *out, int32_t value_count,
                  int32_t segment_count, const swg_plan *plan, int schedule,
                  int32_t block_hint, void *stream) {
  return segreduce("swg_segreduce", kind, dtype, values, offsets, out,
                   value_count, segment_count, plan, schedule, block_hint,
                   stream);
}

int swg_segreduce_map(int kind, int dtype, const swg_map *map,
                      const void *values, const int32_t *offsets, float *out,
                      int32_t value_count, int32_t segment_count,
                      const swg_plan *plan, int schedule, int32_t block_hint,
                      void *stream) {
  if (!map) {
    swg::clear_error();
    swg::set_error("swg_segreduce_map: null map");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  return segreduce("swg_segreduce_map", kind, dtype, values, offsets, out,
                   value_count, segment_count, plan, schedule, block_hint,
                   stream, map);
}

int swg_segreduce_peers_f32(int kind, const float *values,
                            const int32_t *offsets, void *const *dst_bases,
                            int32_t dst_count, int64_t dst_offset,
                            int32_t value_count, int32_t segment_count,
                            const swg_plan *plan, int schedule, void *stream) {
  swg::clear_error();
  const char *who = "swg_segreduce_peers_f32";
  if (kind != SWG_KIND_SUM && kind != SWG_KIND_MAX && kind != SWG_KIND_MIN) {
    swg::set_error(
        "reduction kind must be SWG_KIND_SUM, SWG_KIND_MAX or SWG_KIND_MIN");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (value_count < 0 || segment_count < 0 || dst_offset < 0 ||
      dst_count < 1 || dst_count > SWG_MAX_PEERS) {
    swg::set_error("%s: bad count or offset, or not 1..%d destinations", who,
                   SWG_MAX_PEERS);
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (segment_count == 0) return SWG_OK;
  if (!offsets || !dst_bases || (!values && value_count > 0)) {
    swg::set_error("%s: null pointer", who);
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (!plan) {
    swg::set_error("%s needs a plan (it runs the tile schedules)", who);
    return SWG_ERR_UNSUPPORTED;
  }
  int device = 0, sm_count = 0;
  const int status = current_device(&device, &sm_count);
  if (status != SWG_OK) return status;
  if (plan->host.op != SWG_OP_REDUCE ||
      plan->host.segment_count != segment_count ||
      plan->host.value_count > value_count || plan->dev.device != device) {
    swg::set_error("%s: the plan does not belong to this launch", who);
    return SWG_ERR_PLAN_MISMATCH;
  }
  if (schedule == SWG_SCHED_AUTO) schedule = plan->host.schedule;
  if (schedule != SWG_SCHED_RESIDENT) schedule = SWG_SCHED_SPLIT;
  swg::PeerOut peers = {};
  for (int p = 0; p < dst_count; ++p) {
    if (!dst_bases[p] || ((uintptr_t)dst_bases[p] & 3u) != 0) {
      swg::set_error("%s: destination %d is null or misaligned", who, p);
      return SWG_ERR_INVALID_ARGUMENT;
    }
    peers.base[p] = static_cast<float *>(dst_bases[p]);
  }
  peers.count = dst_count;
  peers.offset = dst_offset;
  cudaStream_t s = (cudaStream_t)stream;
  const swg::Probe *probe = next_probe();
  note_launch(plan, s);
  // `out` is unused by a peer launch: every result goes to the destinations
  const cudaError_t e =
      schedule == SWG_SCHED_RESIDENT
          ? swg::launch_segreduce_resident(kind, SWG_DTYPE_F32, values,
                                           nullptr, value_count, plan->dev, s,
                                           probe, nullptr, &peers)
          : swg::launch_segreduce_split(kind, SWG_DTYPE_F32, values, nullptr,
                                        value_count, plan->dev, s, probe,
                                        nullptr, &peers);
  if (e != cudaSuccess) return cuda_failure("segmented reduce launch", e);
  return SWG_OK;
}

// ---------------------------------------------------------------------------
// Buffers other processes of the node can store into (CUDA IPC)
// ---------------------------------------------------------------------------
static_assert(sizeof(cudaIpcMemHandle_t) == SWG_PEER_HANDLE_BYTES,
              "swg_peer_buffer handles carry one cudaIpcMemHandle_t");

int swg_peer_buffer_create(int64_t bytes, void **buffer,
                           unsigned char *handle) {
  swg::clear_error();
  if (bytes <= 0 || !buffer || !handle) {
    swg::set_error("swg_peer_buffer_create: bad size or null pointer");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return cuda_failure("cudaMalloc (peer buffer)", e);
  cudaIpcMemHandle_t ipc;
  e = cudaIpcGetMemHandle(&ipc, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_failure("cudaIpcGetMemHandle", e);
  }
  memcpy(handle, &ipc, sizeof(ipc));
  *buffer = p;
  return SWG_OK;
}

int swg_peer_buffer_open(const unsigned char *handle, void **buffer) {
  swg::clear_error();
  if (!handle || !buffer) {
    swg::set_error("swg_peer_buffer_open: null pointer");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  cudaIpcMemHandle_t ipc;
  memcpy(&ipc, handle, sizeof(ipc));
  void *p = nullptr;
  // mapped into the CURRENT device's address space; access to the owning
  // GPU over NVLink / PCIe is enabled on first use
  const cudaError_t e =
      cudaIpcOpenMemHandle(&p, ipc, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_failure("cudaIpcOpenMemHandle", e);
  *buffer = p;
  return SWG_OK;
}

int swg_peer_buffer_close(void *buffer) {
  swg::clear_error();
  if (!buffer) return SWG_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(buffer);
  if (e != cudaSuccess) return cuda_failure("cudaIpcCloseMemHandle", e);
  return SWG_OK;
}

int swg_peer_buffer_destroy(void *buffer) {
  swg::clear_error();
  if (!buffer) return SWG_OK;
  const cudaError_t e = cudaFree(buffer);
  if (e != cudaSuccess) return cuda_failure("cudaFree (peer buffer)", e);
  return SWG_OK;
}

int swg_scatter_results_f32(const float *src, int64_t count,
                            void *const *dst_bases, int32_t dst_count,
                            int64_t dst_offset, void *stream) {
  swg::clear_error();
  if (count < 0 || dst_offset < 0 || dst_count < 0 ||
      dst_count > SWG_MAX_PEERS) {
    swg::set_error(
        "swg_scatter_results_f32: negative count or offset, or more than %d "
        "destinations", SWG_MAX_PEERS);
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (count == 0 || dst_count == 0) return SWG_OK;
  if (!src || !dst_bases) {
    swg::set_error("swg_scatter_results_f32: null pointer");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  float *bases[SWG_MAX_PEERS];
  for (int p = 0; p < dst_count; ++p) {
    if (!dst_bases[p] || ((uintptr_t)dst_bases[p] & 15u) != 0) {
      swg::set_error(
          "swg_scatter_results_f32: destination %d is null or not 16-byte "
          "aligned", p);
      return SWG_ERR_INVALID_ARGUMENT;
    }
    bases[p] = static_cast<float *>(dst_bases[p]);
  }
  int device = 0, sm_count = 0;
  const int status = current_device(&device, &sm_count);
  if (status != SWG_OK) return status;
  const cudaError_t e = swg::launch_scatter_results(
      src, count, bases, dst_count, dst_offset, sm_count,
      (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_failure("result scatter launch", e);
  return SWG_OK;
}

int swg_segreduce_sum_max_f32(const float *values, const int32_t *offsets,
                              float *out_sum, float *out_max,
                              int32_t value_count, int32_t segment_count,
                              void *stream) {
  swg::clear_error();
  if (value_count < 0 || segment_count < 0) {
    swg::set_error("swg_segreduce_sum_max_f32: negative count");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (segment_count == 0) return SWG_OK;
  if (!offsets || !out_sum || !out_max || (!values && value_count > 0)) {
    swg::set_error("swg_segreduce_sum_max_f32: null pointer");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (out_sum == out_max) {
    swg::set_error("swg_segreduce_sum_max_f32: the two outputs must differ");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  int device = 0, sm_count = 0;
  const int status = current_device(&device, &sm_count);
  if (status != SWG_OK) return status;
  const cudaError_t e = swg::launch_segreduce_sum_max(
      values, offsets, out_sum, out_max, value_count, segment_count, sm_count,
      (cudaStream_t)stream, next_probe());
  if (e != cudaSuccess) return cuda_failure("fused sum + max launch", e);
  return SWG_OK;
}

int swg_segreduce_f32_noalloc(int kind, const float *values,
                              const int32_t *host_offsets, float *out,
                              int32_t value_count, int32_t segment_count,
                              void *stream) {
  swg::clear_error();
  if (kind != SWG_KIND_SUM && kind != SWG_KIND_MAX && kind != SWG_KIND_MIN) {
    swg::set_error(
        "reduction kind must be SWG_KIND_SUM, SWG_KIND_MAX or SWG_KIND_MIN");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (value_count < 0 || segment_count < 0 || !host_offsets) {
    swg::set_error("swg_segreduce_f32_noalloc: bad count or null offsets");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (segment_count > swg::kStaticMaxSegments) {
    swg::set_error(
        "swg_segreduce_f32_noalloc: %d segments exceed the fixed scratch "
        "(at most %d); use swg_plan_create + swg_segreduce_f32",
        segment_count, swg::kStaticMaxSegments);
    return SWG_ERR_UNSUPPORTED;
  }
  int status = swg::validate_offsets(host_offsets, (int64_t)segment_count + 1,
                                     value_count, segment_count, nullptr,
                                     nullptr);
  if (status != SWG_OK) return status;
  if (segment_count == 0) return SWG_OK;
  if (!out || (!values && value_count > 0)) {
    swg::set_error("swg_segreduce_f32_noalloc: null pointer");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  swg::HostPlan plan;
  swg::build_host_plan(host_offsets, segment_count, SWG_OP_REDUCE, &plan);
  // (the list of cut segments shares its region with the list of the long
  // ones, which takes kStaticMaxSlots / kWarpMerge records off its end)
  if ((int64_t)plan.tasks.size() > swg::kStaticMaxTasks ||
      plan.partial_slots > swg::kStaticMaxSlots ||
      (int64_t)plan.merges.size() >
          swg::kStaticMaxSlots / 2 - swg::kStaticMaxSlots / swg::kWarpMerge) {
    swg::set_error(
        "swg_segreduce_f32_noalloc: input needs %zu tile tasks / %d partials, "
        "the fixed scratch holds %d / %d; use swg_plan_create + "
        "swg_segreduce_f32",
        plan.tasks.size(), plan.partial_slots, swg::kStaticMaxTasks,
        swg::kStaticMaxSlots);
    return SWG_ERR_UNSUPPORTED;
  }
  int device = 0, sm_count = 0;
  status = current_device(&device, &sm_count);
  if (status != SWG_OK) return status;
  cudaError_t e = swg::launch_segreduce_static(
      kind, values, out, value_count, host_offsets, segment_count, plan,
      device, sm_count, (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_failure("allocation-free reduce", e);
  return SWG_OK;
}

int swg_segsoftmax_f32(const float *values, const int32_t *offsets, float *out,
                       int32_t value_count, int32_t segment_count,
                       const swg_plan *plan, int schedule, void *stream) {
  swg::clear_error();
  if (value_count < 0 || segment_count < 0 || schedule < SWG_SCHED_AUTO ||
      schedule > SWG_SCHED_RESIDENT) {
    swg::set_error("swg_segsoftmax_f32: bad count or schedule");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (segment_count == 0 || value_count == 0) return SWG_OK;
  if (!offsets || !out || !values) {
    swg::set_error("swg_segsoftmax_f32: null pointer");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  if (values == out) {
    swg::set_error("swg_segsoftmax_f32: out must not alias values");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  int device = 0, sm_count = 0;
  int status = current_device(&device, &sm_count);
  if (status != SWG_OK) return status;
  if (plan) {
    if (plan->host.op != SWG_OP_SOFTMAX ||
        plan->host.segment_count != segment_count ||
        plan->host.value_count > value_count || plan->dev.device != device) {
      swg::set_error("plan was not built for this softmax launch");
      return SWG_ERR_PLAN_MISMATCH;
    }
  } else if (schedule >= SWG_SCHED_SPLIT) {
    swg::set_error("the planned softmax schedule needs a plan");
    return SWG_ERR_UNSUPPORTED;
  }
  if (schedule == SWG_SCHED_AUTO)
    schedule = plan ? SWG_SCHED_SPLIT
               : (int64_t)value_count >= (int64_t)segment_count * 1024
                   ? SWG_SCHED_CTA
                   : SWG_SCHED_WARP;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e;
  const swg::Probe *probe = next_probe();
  if (plan) note_launch(plan, s);
  if (plan && schedule >= SWG_SCHED_SPLIT)
    e = swg::launch_segsoftmax_planned(values, offsets, out, value_count,
                                       plan->dev, s, probe);
  else if (schedule == SWG_SCHED_WARP)
    e = swg::launch_segsoftmax_warp(values, offsets, out, segment_count,
                                    sm_count, s, probe);
  else
    e = swg::launch_segsoftmax_cta(values, offsets, out, segment_count,
                                   sm_count, s, probe);
  if (e != cudaSuccess) return cuda_failure("segmented softmax launch", e);
  return SWG_OK;
}

int swg_shard_offsets(const int32_t *host_offsets, int32_t segment_count,
                      int32_t shards, int32_t *seg_begin) {
  swg::clear_error();
  return swg::shard_offsets(host_offsets, segment_count, shards, seg_begin);
}

int swg_profile_start(int32_t capacity, int32_t stride) {
  swg::clear_error();
  if (capacity < 1 || capacity > (1 << 20) || stride < 1) {
    swg::set_error(
        "swg_profile_start: capacity must be in [1, 2^20] and stride >= 1");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> guard(g_lock);
  drop_probes();
  g_profile.stride = stride;
  g_profile.probes.reserve((size_t)capacity);
  for (int32_t i = 0; i < capacity; ++i) {
    swg::Probe probe;
    cudaError_t e = cudaEventCreate(&probe.start);
    if (e == cudaSuccess) {
      e = cudaEventCreate(&probe.stop);
      if (e != cudaSuccess) cudaEventDestroy(probe.start);
    }
    if (e != cudaSuccess) {
      drop_probes();
      return cuda_failure("cudaEventCreate", e);
    }
    g_profile.probes.push_back(probe);
  }
  g_profile.active = true;
  return SWG_OK;
}

int swg_profile_stop(float *milliseconds, int32_t capacity, int32_t *count) {
  swg::clear_error();
  std::lock_guard<std::mutex> guard(g_lock);
  if (!g_profile.active) {
    swg::set_error("swg_profile_stop: profiling was not started");
    return SWG_ERR_INVALID_ARGUMENT;
  }
  const size_t used = g_profile.used;
  int status = SWG_OK;
  for (size_t i = 0; i < used; ++i) {
    cudaError_t e = cudaEventSynchronize(g_profile.probes[i].stop);
    float ms = 0.0f;
    if (e == cudaSuccess)
      e = cudaEventElapsedTime(&ms, g_profile.probes[i].start,
                               g_profile.probes[i].stop);
    if (e != cudaSuccess) {
      status = cuda_failure("cudaEventElapsedTime", e);
      break;
    }
    if (milliseconds && (int32_t)i < capacity) milliseconds[i] = ms;
  }
  if (count) *count = (int32_t)used;
  drop_probes();
  return status;
}

}  // extern "C"
