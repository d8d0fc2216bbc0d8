// Host-side conventions shared by the launchers.
//
// They follow the reference engine's launchers (engine/src/kernels_phase2.cu:
// 822-836, engine/src/prefill_gemm.cu "G4_PF_CHECK"): validate, launch on the
// calling thread's stream, never synchronise, never allocate, return 0 on
// success and -1 on invalid arguments or a launch error with one diagnostic
// line on stderr.
#pragma once

#include <cuda_runtime.h>

#include <climits>
#include <cmath>
#include <cstdint>
#include <cstdio>

namespace g4 {

// Stream every launcher of this library uses on the calling thread. Defaults
// to the per-thread default stream, as the reference build does
// (--default-stream per-thread, engine/CMakeLists.txt:43-48); a host that
// drives its own streams (PyTorch, a serving loop) sets it per thread.
cudaStream_t current_stream();
void set_current_stream(cudaStream_t s);

int sm_count();  // SMs of the current device (cached per device)

// Device address of the library's status word on the current device (kernels
// with bounded waits report a wait that ran out there). NULL if the address
// could not be resolved.
unsigned int* device_status_ptr();

inline int fail(const char* fn, const char* why) {
  std::fprintf(stderr, "granite4: %s: %s\n", fn, why);
  return -1;
}

#define G4_LAUNCH_CHECK(fn)                                                        \
  do {                                                                             \
    cudaError_t e_ = cudaGetLastError();                                           \
    if (e_ != cudaSuccess) {                                                       \
      std::fprintf(stderr, "granite4: %s: CUDA error at %s:%d: %s\n", fn, __FILE__, \
                   __LINE__, cudaGetErrorString(e_));                              \
      return -1;                                                                   \
    }                                                                              \
  } while (0)

#define G4_CUDA_TRY(fn, expr)                                                      \
  do {                                                                             \
    cudaError_t e_ = (expr);                                                       \
    if (e_ != cudaSuccess) {                                                       \
      std::fprintf(stderr, "granite4: %s: CUDA error at %s:%d: %s\n", fn, __FILE__, \
                   __LINE__, cudaGetErrorString(e_));                              \
      return -1;                                                                   \
    }                                                                              \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// granite4_glue_layer clears the {scale, amax} slots of all three FP8 ops of a layer with one
// memset and sets this (per thread) while it calls the launchers, which then skip their own.
bool amax_prezeroed();
void set_amax_prezeroed(bool on);

// Fraction of a `bytes`-large intermediate to mark evict_last in L2 between the two sweeps of
// add + norm -> FP8 (g4_math.cuh, l2_policy_evict_last): G4_L2_KEEP_MB in the environment (read
// once) is the share of L2 set aside for it; all of the tensor while it fits, else that share
// spread evenly over it. Off (0) by default: measured on B200, the default replacement policy
// already leaves about 80 MB of the hidden state in L2 for the second sweep (DRAM reads of that
// sweep: 0.2 MB of 67 at 8192 rows, 20 of 101 at 12288, 53 of 134 at 16384, 120 of 201 at 24576)
// and a 96 MB hint moved those figures by under 8 MB.
float l2_keep_fraction(double bytes);

// Programmatic dependent launch: a kernel launched through launch_pdl may be staged on the GPU
// while the kernel before it on the stream is still draining; it must (and every kernel launched
// this way does, as its first statements, in every CTA) execute pdl_begin() from g4_math.cuh,
// which holds it until the preceding kernel has completed and its writes are visible. What is
// saved is the launch latency and the ramp of each kernel boundary, which is all a decode-size
// or small-shard launch consists of. G4_PDL=0 in the environment launches everything fully
// serialised (read per call).
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1u : 0u;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define G4_LAUNCH_PDL(fn, ...)                                                      \
  do {                                                                             \
    cudaError_t e_ = g4::launch_pdl(__VA_ARGS__);                                  \
    if (e_ != cudaSuccess) {                                                       \
      (void)cudaGetLastError();                                                    \
      std::fprintf(stderr, "granite4: %s: CUDA error at %s:%d: %s\n", fn, __FILE__, \
                   __LINE__, cudaGetErrorString(e_));                              \
      return -1;                                                                   \
    }                                                                              \
  } while (0)

}  // namespace g4
