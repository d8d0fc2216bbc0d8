// Bulk asynchronous copies (the TMA engine's untiled form) and the mbarrier
// they signal, as inline PTX for sm_100a.
//
// Rules these helpers rely on: both addresses of a bulk copy are 16-byte
// aligned and the size is a multiple of 16 bytes; a CTA only ever copies into
// its own shared memory (the destination is named in the CTA's own window, so
// no copy is ever delivered to another CTA);
// every wait is bounded - a wait that runs out reports failure to the caller,
// which records it in the library's device status word and winds the CTA down
// instead of spinning.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace g4 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals)
               : "memory");
}
// Makes freshly initialised barriers visible to the async proxy.
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// One arrival that also announces `bytes` of copy traffic the phase waits for.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
// One plain arrival on a barrier of this CTA.
__device__ __forceinline__ void mbar_arrive_local(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait for the phase with the given parity. try_wait itself blocks for
// a hardware-defined interval, so the iteration cap is a time cap of the order
// of a second; a copy of a few KB completes in microseconds.
constexpr uint32_t kMbarWaitLimit = 1u << 20;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kMbarWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 64) __nanosleep(64);
  }
  return false;
}

// global -> this CTA's shared memory; completion is counted on `bar`.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// this CTA's shared memory -> global, tracked by the thread's bulk groups.
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's store groups still read shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Wait until at most N store groups are incomplete (their writes performed).
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Orders this thread's ordinary shared-memory writes before later async-proxy
// reads of them (a bulk store issued after a barrier).
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Bits of the library's device status word (0 = fine). A kernel ORs its bit
// into the word (passed to it as a pointer) when a bounded wait runs out; the
// host reads the word with granite4_b200_device_status().
enum DeviceStatusBits : unsigned int {
  kStatusEmbedWaitTimeout = 1u << 0,
  kStatusNormWaitTimeout = 1u << 1,
  kStatusSwigluWaitTimeout = 1u << 2,
  kStatusRopeWaitTimeout = 1u << 3,
  kStatusGemmWaitTimeout = 1u << 4,
  kStatusAttnWaitTimeout = 1u << 5,
};

}  // namespace g4
