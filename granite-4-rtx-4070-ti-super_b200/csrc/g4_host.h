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

}  // namespace g4
