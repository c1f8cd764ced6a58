// Result exchange of a sharded reduction: every GPU stores the results of its
// own segments into every GPU's copy of the full result array, so that no
// collective is needed for "every rank sees every result".
//
//   dst[p][dst_offset + i] = src[i]   for every destination p, 0 <= i < count
//
// `src` is this GPU's result shard (written a moment ago by the reduce kernels,
// so the loads hit L2); the destinations are device pointers that may live on
// other GPUs of the node (peer-mapped through CUDA IPC).  The traffic over
// NVLink is plain st.global: no multicast, no load from peer memory, no wait on
// another GPU -- the kernel is an ordinary grid that ends by itself.  When the
// results are complete on a peer is for the host to say (a barrier after this
// kernel's stream has been synchronised, or an event).
//
// The reference is single-GPU (python/swage/_runtime.py:146-151); nothing
// here mirrors a reference function.
#include "swg_common.cuh"
#include "swg_launch.h"

namespace swg {

constexpr int kScatterThreads = 256;

struct PeerBases {
  float *base[kMaxPeers];
};

// Launched with programmatic stream serialisation: the grid may be placed
// while the kernel before it (the merge pass) drains and waits for that
// kernel's results to be visible before it reads one.
__global__ void __launch_bounds__(kScatterThreads)
scatter_results_kernel(const float *__restrict__ src, int64_t count,
                       PeerBases peers, int peer_count, int64_t dst_offset) {
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // Destination element j = dst_offset + i.  Whole 16-byte lines of the
  // destinations are [body_begin, body_end) in source indices; the ragged
  // ends are stored element by element.  (Every destination shares the
  // alignment of its base: allocations are at least 256-byte aligned, the
  // launcher checks 16.)
  int64_t head = (4 - (dst_offset & 3)) & 3;
  if (head > count) head = count;
  const int64_t lines = (count - head) >> 2;
  const int64_t tail_begin = head + (lines << 2);
  const int64_t thread = (int64_t)blockIdx.x * kScatterThreads + threadIdx.x;
  const int64_t threads = (int64_t)gridDim.x * kScatterThreads;
  for (int64_t line = thread; line < lines; line += threads) {
    const int64_t i = head + (line << 2);
    float4 q;
    q.x = src[i];
    q.y = src[i + 1];
    q.z = src[i + 2];
    q.w = src[i + 3];
    for (int p = 0; p < peer_count; ++p)
      *reinterpret_cast<float4 *>(peers.base[p] + dst_offset + i) = q;
  }
  if (thread < head)
    for (int p = 0; p < peer_count; ++p)
      peers.base[p][dst_offset + thread] = src[thread];
  if (tail_begin + thread < count)
    for (int p = 0; p < peer_count; ++p)
      peers.base[p][dst_offset + tail_begin + thread] = src[tail_begin + thread];
}

cudaError_t launch_scatter_results(const float *src, int64_t count,
                                   float *const *dst_bases, int peer_count,
                                   int64_t dst_offset, int sm_count,
                                   cudaStream_t stream) {
  if (count == 0 || peer_count == 0) return cudaSuccess;
  PeerBases peers = {};
  for (int p = 0; p < peer_count; ++p) peers.base[p] = dst_bases[p];
  int64_t grid = ((count >> 2) + kScatterThreads - 1) / kScatterThreads;
  if (grid < 1) grid = 1;
  if (grid > (int64_t)sm_count * 8) grid = (int64_t)sm_count * 8;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)grid);
  config.blockDim = dim3(kScatterThreads);
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, scatter_results_kernel, src, count, peers,
                            peer_count, dst_offset);
}

}  // namespace swg
