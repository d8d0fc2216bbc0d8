// Token-embedding gather with the embedding multiplier.
//
// Formulation (reference: engine/src/prefill_gemm.cu:281-301, helper
// engine/src/device_math.cuh:258-265, host twin engine/src/kernel_math.h:450-453):
//   out[r][j] = bf16(mult * f32(emb[tok[r]][j]))      one f32 multiply, one RNE
//
// Data layout: table bf16 [vocab][H] (822 MB for Granite), ids int32 [rows],
// out bf16 [rows][H]; a row is H * 2 bytes (8 KB) and 16-byte aligned.
// Algorithmic bytes per row: 4 + 8192 read, 8192 written = 16 388.
//
// Two kernels:
//  * embed_bulk_kernel (default): persistent CTAs, each streaming its rows
//    through a ring of shared-memory stages. One elected thread gathers: it
//    reads the token id and issues one bulk asynchronous copy (TMA engine) of
//    the whole table row into a stage, signalled on an mbarrier; the CTA scales
//    the row in shared memory and the elected thread sends it out with one bulk
//    store. Rows in flight are bounded by shared memory, not registers.
//  * embed_vec_kernel (G4_EMBED_BULK=0, and rows that are not a multiple of 16
//    bytes): a warp per row, four 128-bit loads in flight per lane.
#include "g4_host.h"
#include "g4_math.cuh"
#include "g4_tma.cuh"

#include "../../include/granite4_b200.h"
#include "../../include/granite4_b200.hpp"

#include <atomic>
#include <algorithm>
#include <cstdlib>
#include <cstring>

namespace g4 {
namespace {

__device__ __forceinline__ uint4 scale8(uint4 v, float mult) {
  uint4 o;
  o.x = pack_bf16x2(__fmul_rn(mult, bf16_lo(v.x)), __fmul_rn(mult, bf16_hi(v.x)));
  o.y = pack_bf16x2(__fmul_rn(mult, bf16_lo(v.y)), __fmul_rn(mult, bf16_hi(v.y)));
  o.z = pack_bf16x2(__fmul_rn(mult, bf16_lo(v.z)), __fmul_rn(mult, bf16_hi(v.z)));
  o.w = pack_bf16x2(__fmul_rn(mult, bf16_lo(v.w)), __fmul_rn(mult, bf16_hi(v.w)));
  return o;
}

// vocab <= 0: ids are trusted (the reference's contract); otherwise a row whose
// id is out of range is written as zeros.
__global__ void __launch_bounds__(256)
    embed_vec_kernel(const int32_t* tokens, long long start, long long rows, const uint4* emb,
                     int vocab, float mult, uint4* out, int H8) {
  pdl_begin();
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += nwarps) {
    const int32_t tok = __ldg(tokens + start + r);
    const bool bad = vocab > 0 && (tok < 0 || tok >= vocab);
    const uint4* src = emb + static_cast<size_t>(bad ? 0 : tok) * H8;
    uint4* dst = out + static_cast<size_t>(r) * H8;
    for (int c0 = 0; c0 < H8; c0 += 128) {
      uint4 v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = c0 + k * 32 + lane;
        if (c < H8) v[k] = ld_stream(src + c);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int c = c0 + k * 32 + lane;
        if (c < H8) st_stream(dst + c, bad ? make_uint4(0, 0, 0, 0) : scale8(v[k], mult));
      }
    }
  }
}

constexpr int kStages = 4;
constexpr int kBulkThreads = 128;

// Dynamic shared memory: kStages rows, then kStages mbarriers.
__global__ void __launch_bounds__(kBulkThreads)
    embed_bulk_kernel(const int32_t* tokens, long long start, long long rows, const uint16_t* emb,
                      int vocab, float mult, uint16_t* out, int H, unsigned int* status) {
  pdl_begin();
  extern __shared__ __align__(128) unsigned char smem[];
  const uint32_t row_bytes = static_cast<uint32_t>(H) * 2u;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kStages) * row_bytes);
  const int t = threadIdx.x;
  // rows of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...
  const long long n_local = (rows - blockIdx.x + gridDim.x - 1) / gridDim.x;

  if (t == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(full + s, 1);
    mbar_init_fence();
  }
  __syncthreads();

  // The elected thread keeps kStages - 2 loads ahead: the stage it refills was
  // handed to a bulk store two iterations ago, and that store has finished
  // reading shared memory once at most one newer store group is outstanding.
  auto issue = [&](long long i) {
    const long long r = blockIdx.x + i * static_cast<long long>(gridDim.x);
    const int s = static_cast<int>(i % kStages);
    int32_t tok = tokens[start + r];
    if (vocab > 0 && (tok < 0 || tok >= vocab)) tok = 0;  // flagged bad below; load stays in range
    mbar_arrive_expect_tx(full + s, row_bytes);
    bulk_load(smem + static_cast<size_t>(s) * row_bytes, emb + static_cast<size_t>(tok) * H,
              row_bytes, full + s);
  };
  constexpr int kAhead = kStages - 2;
  if (t == 0)
    for (long long i = 0; i < kAhead && i < n_local; ++i) issue(i);

  const bool copy_only = (mult == 1.0f);
  long long issued_until = kAhead < n_local ? kAhead : n_local;  // meaningful in thread 0
  bool failed = false;
  for (long long i = 0; i < n_local; ++i) {
    const int s = static_cast<int>(i % kStages);
    const uint32_t parity = static_cast<uint32_t>((i / kStages) & 1);
    if (t == 0 && i + kAhead < n_local) {
      bulk_wait_read<1>();
      issue(i + kAhead);
      issued_until = i + kAhead + 1;
    }
    // the verdict is made CTA-wide so that every thread leaves the loop together
    const bool landed = mbar_wait_bounded(full + s, parity);
    if (__syncthreads_or(!landed)) {
      failed = true;
      break;
    }
    const long long r = blockIdx.x + i * static_cast<long long>(gridDim.x);
    unsigned char* stage = smem + static_cast<size_t>(s) * row_bytes;
    const int32_t tok = __ldg(tokens + start + r);
    const bool bad = vocab > 0 && (tok < 0 || tok >= vocab);
    if (!copy_only || bad) {
      uint4* v = reinterpret_cast<uint4*>(stage);
      for (int c = t; c < H / 8; c += kBulkThreads)
        v[c] = bad ? make_uint4(0, 0, 0, 0) : scale8(v[c], mult);
      fence_async_smem();
    }
    __syncthreads();
    if (t == 0) {
      bulk_store(out + static_cast<size_t>(r) * H, stage, row_bytes);
      bulk_commit();
    }
  }
  if (failed) {
    // A copy never signalled. Record it; thread 0 then gives every load it
    // issued one more bounded chance to land, so none is in flight towards
    // this CTA's shared memory when the CTA exits.
    if (t == 0) {
      atomicOr(status, kStatusEmbedWaitTimeout);
      for (long long i = 0; i < issued_until; ++i)
        (void)mbar_wait_bounded(full + (i % kStages), static_cast<uint32_t>((i / kStages) & 1));
    }
  }
  if (t == 0) bulk_wait_all<0>();
}

bool bulk_enabled() {
  const char* v = std::getenv("G4_EMBED_BULK");
  return !(v != nullptr && std::strcmp(v, "0") == 0);
}

int embed_launch(const char* fn, const int32_t* d_tokens, long long start, long long rows,
                 const uint16_t* emb, int vocab, float mult, uint16_t* out, int H) {
  cudaStream_t st = current_stream();
  const bool vec_ok = H % 8 == 0 && aligned16(emb) && aligned16(out);
  if (!vec_ok) return fail(fn, "H must be a multiple of 8 and the buffers 16-byte aligned");
  const size_t smem = static_cast<size_t>(kStages) * H * 2 + kStages * sizeof(uint64_t);
  unsigned int* status = device_status_ptr();
  if (bulk_enabled() && smem <= 200 * 1024 && status != nullptr) {
    static std::atomic<bool> attr_set[64];  // per device; relaxed: setting the attribute twice is harmless
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(fn, "cannot identify the current device");
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_relaxed)) {
      G4_CUDA_TRY(fn, cudaFuncSetAttribute(embed_bulk_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      attr_set[dev].store(true, std::memory_order_relaxed);
    }
    const long long per_sm = std::max<long long>(1, std::min<long long>(8, (200 * 1024) / smem));
    const unsigned grid = static_cast<unsigned>(std::min<long long>(rows, sm_count() * per_sm));
    G4_LAUNCH_PDL(fn, embed_bulk_kernel, dim3(grid), dim3(kBulkThreads), smem, st, d_tokens, start, rows, emb,
                  vocab, mult, out, H, status);
  } else {
    const long long warps = rows;
    const unsigned grid =
        static_cast<unsigned>(std::min<long long>((warps + 7) / 8, sm_count() * 8LL));
    G4_LAUNCH_PDL(fn, embed_vec_kernel, dim3(grid), dim3(256), 0, st, d_tokens, start, rows,
                  reinterpret_cast<const uint4*>(emb), vocab, mult, reinterpret_cast<uint4*>(out), H / 8);
  }
  G4_LAUNCH_CHECK(fn);
  return 0;
}

// H not a multiple of 8: scalar gather (the reference's embed_rows_kernel case).
__global__ void __launch_bounds__(256)
    embed_scalar_kernel(const int32_t* tokens, long long start, const uint16_t* emb, float mult,
                        uint16_t* out, int H) {
  const long long r = blockIdx.x;
  const int32_t tok = tokens[start + r];
  for (int j = threadIdx.x; j < H; j += blockDim.x)
    out[r * H + j] = static_cast<uint16_t>(
        f32_to_bf16_bits(__fmul_rn(mult, bf16_to_f32(emb[static_cast<size_t>(tok) * H + j]))));
}

}  // namespace
}  // namespace g4

extern "C" {

int granite4_prefill_embed_rows(const int32_t* d_tokens, int start, int rows, const uint16_t* emb,
                                float mult, uint16_t* out, int H) {
  const char* fn = "prefill_embed_rows";
  if (rows <= 0 || rows > 65535 || H <= 0) return -1;  // engine/src/prefill_gemm.cu:1302
  if (d_tokens == nullptr || emb == nullptr || out == nullptr || start < 0)
    return g4::fail(fn, "invalid arguments");
  if (H % 8 != 0 || !g4::aligned16(emb) || !g4::aligned16(out)) {
    g4::embed_scalar_kernel<<<rows, 256, 0, g4::current_stream()>>>(d_tokens, start, emb, mult, out,
                                                                   H);
    G4_LAUNCH_CHECK(fn);
    return 0;
  }
  return g4::embed_launch(fn, d_tokens, start, rows, emb, 0, mult, out, H);
}

int granite4_kernel_embed_gather(const int32_t* d_tokens, long long rows, const uint16_t* d_emb,
                                 int vocab, float mult, uint16_t* d_out, int H) {
  const char* fn = "granite4_kernel_embed_gather";
  if (d_tokens == nullptr || d_emb == nullptr || d_out == nullptr || rows <= 0 || vocab <= 0 ||
      H <= 0 || !std::isfinite(mult))
    return g4::fail(fn, "invalid arguments");
  return g4::embed_launch(fn, d_tokens, 0, rows, d_emb, vocab, mult, d_out, H);
}

}  // extern "C"

namespace granite4 {
int prefill_embed_rows(const std::int32_t* d_tokens, int start, int rows, const std::uint16_t* emb,
                       float mult, std::uint16_t* out, int H) {
  return granite4_prefill_embed_rows(d_tokens, start, rows, emb, mult, out, H);
}
}  // namespace granite4
