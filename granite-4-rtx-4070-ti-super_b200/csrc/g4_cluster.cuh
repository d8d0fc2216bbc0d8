// One thread-block cluster as the whole grid: the small-batch form of the ops
// whose FP8 scale depends on every element of the tensor.
//
// A decode or verify step has 1..16 token rows (the reference caps a verify
// batch at 16 rows, engine/src/model_config.h kMaxVerifyRows). At that size an
// op is a few microseconds of work, and the two-sweep form (clear the amax
// slot, stats sweep, encode sweep) costs three stream operations. With at most
// 16 CTAs the whole tensor fits in the registers of one cluster, so one launch
// does it: every CTA computes its part and the part's max |x|, the CTAs
// exchange the maxima through distributed shared memory, meet at the hardware
// cluster barrier, and encode from registers. Nothing is re-read, nothing is
// cleared beforehand, no global atomics.
//
// The cluster barrier is a hardware barrier (no spin loop of ours); every
// thread of every CTA reaches it exactly once - CTAs with no work do not
// return early.
#pragma once

#include "g4_host.h"
#include "g4_math.cuh"

#include <cooperative_groups.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

namespace g4 {

constexpr int kMaxClusterCtas = 16;  // 8 is the portable limit, 16 needs the opt-in attribute

// A CTA's shared memory may be written from another CTA of the cluster only once that CTA is
// known to be executing. Every kernel that runs as one cluster therefore announces itself as its
// first statement (after pdl_begin) with cluster_announce(), and waits with cluster_all_started()
// just before its first store into a peer's shared memory: one split phase of the hardware cluster
// barrier, whose wait is long over by the time the data for the store has been loaded. Every
// thread of every CTA executes both, exactly once and in this order.
__device__ __forceinline__ void cluster_announce() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_all_started() {
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
}

// Max of `thread_amax` (packed sign-cleared bf16 pairs) over every thread of
// every CTA in the cluster, as float bits. s_warp: one word per warp of the
// CTA; s_slots: kMaxClusterCtas words. Called by all threads, in a kernel that
// began with cluster_announce().
__device__ __forceinline__ uint32_t cluster_amax_bits(uint32_t thread_amax, uint32_t* s_warp,
                                                      uint32_t* s_slots) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31, nwarps = (blockDim.x + 31) >> 5;
  thread_amax = amax_warp(thread_amax);
  if (lane == 0) s_warp[warp] = thread_amax;
  __syncthreads();
  cluster_all_started();  // pairs with the cluster_announce() at the top of the calling kernel
  const unsigned n = cluster.num_blocks();
  if (warp == 0) {
    uint32_t m = 0u;
    for (int i = lane; i < nwarps; i += 32) m = max_u16x2(m, s_warp[i]);
    m = amax_warp(m);
    // lane d delivers this CTA's maximum into CTA d's slot for this CTA
    if (static_cast<unsigned>(lane) < n)
      *cluster.map_shared_rank(s_slots + cluster.block_rank(), lane) = __float_as_uint(amax_value(m));
  }
  cluster.sync();  // release / acquire: the remote stores above are visible after it
  uint32_t g = 0u;
  for (unsigned i = 0; i < n; ++i) g = max(g, s_slots[i]);  // non-negative floats order as integers; NaN stays on top
  return g;
}

// G4_CLUSTER=0 in the environment keeps every op on its multi-launch form (A/B runs, tests that
// compare the two forms).
inline bool cluster_enabled() {
  const char* v = std::getenv("G4_CLUSTER");  // read per call: a test flips it between calls
  return !(v != nullptr && v[0] == '0');
}

// Whether the current device can co-schedule one cluster of `ctas` CTAs of `kernel`; asked of the
// runtime once per (device, kernel, shape) and remembered, so that steady-state calls - and calls
// made while a stream is being captured, after a first call outside capture - only launch.
inline bool cluster_fits(const void* kernel, const cudaLaunchConfig_t& cfg, int ctas, int threads) {
  static std::mutex mu;
  static std::map<std::tuple<int, const void*, int, int>, bool> known;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  const auto key = std::make_tuple(dev, kernel, ctas, threads);
  std::lock_guard<std::mutex> lock(mu);
  const auto it = known.find(key);
  if (it != known.end()) return it->second;
  bool ok = true;
  if (ctas > 8)
    ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
  int fit = 0;
  if (ok) ok = cudaOccupancyMaxActiveClusters(&fit, kernel, &cfg) == cudaSuccess && fit >= 1;
  if (!ok) (void)cudaGetLastError();
  known[key] = ok;
  return ok;
}

// Launch `kernel` as one cluster of `ctas` CTAs (a power of two, at most 16).
// Returns cudaErrorInvalidConfiguration without launching when the device
// cannot co-schedule such a cluster; the caller then takes the multi-launch form.
template <typename Params>
cudaError_t cluster_launch(void (*kernel)(Params), int ctas, int threads, const Params& p,
                           cudaStream_t st) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas));
  cfg.blockDim = dim3(static_cast<unsigned>(threads));
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(ctas);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // the kernels launched through here all start with pdl_begin() (g4_math.cuh)
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (!cluster_fits(reinterpret_cast<const void*>(kernel), cfg, ctas, threads))
    return cudaErrorInvalidConfiguration;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

inline int cluster_ctas_for(long long units) {
  int c = 1;
  while (c < units) c <<= 1;
  return c;
}

}  // namespace g4
