// FP8 x FP8 prefill GEMM on the 5th-generation tensor cores (sm_100a).
//
//   C[m][n] = a_scale * w_scale(n) * sum_k A[m][k] * W[n][k]
//
// A [M][K] is what the glue's FP8 outputs are (e4m3 codes + one device-resident
// dequantisation scale), W [N][K] is the reference's weight layout (row-major
// e4m3, one scale per stacked tensor). This is the FP8-activation counterpart of
// granite4::prefill_gemm (engine/src/prefill_gemm.h:12-36, kernel
// engine/src/prefill_gemm.cu:134-258), which takes bf16 activations and decodes
// the weights to bf16 per mma.sync fragment; the epilogue (GemmOut::kBf16 / kF32
// / kResidual and the three-segment weight scale) is the reference's
// (engine/src/prefill_gemm.cu:65-88).
//
// Shape of the kernel: persistent, one CTA per SM, 128 x 256 output tiles,
// K consumed in 128-byte blocks. Roles by warp:
//   warp 0   one thread issues the tiled TMA loads (128-byte swizzle) of the A
//            and W blocks into a 4-stage shared-memory ring;
//   warp 1   allocates tensor memory; one thread issues tcgen05.mma
//            (kind::f8f6f4, M 128, N 256, K 32 per instruction) straight from
//            the ring into one of two 256-column accumulators, and commits each
//            stage back to the loader and each finished tile to the epilogue;
//   warps 2-5 read the finished accumulator out of tensor memory (each warp its
//            own 32 lanes = 32 output rows), scale, convert and store, while
//            the next tile's MMAs fill the other accumulator.
// Every wait on an mbarrier is bounded; a wait that runs out sets the library's
// device status word and an abort flag that winds all roles down, after which
// the CTA waits a bounded time for copies in flight and frees its tensor memory.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>

#include "../../include/granite4_b200.h"
#include "g4_host.h"
#include "g4_math.cuh"
#include "g4_tma.cuh"

namespace {

using namespace g4;

constexpr int kBM = 128, kBN = 256, kBK = 128;  // kBK in bytes = e4m3 elements
constexpr int kStages = 4, kAccs = 2;
constexpr uint32_t kABytes = kBM * kBK, kWBytes = kBN * kBK, kStageBytes = kABytes + kWBytes;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = kAccs * kBN;  // 512: the whole tensor memory of the SM

struct Ring {
  uint64_t full[kStages], empty[kStages], acc_full[kAccs], acc_empty[kAccs];
  uint32_t tmem_base;
  int abort;
};
constexpr size_t kSmemBytes = 1024 + size_t(kStages) * kStageBytes + sizeof(Ring);

struct GemmParams {
  int M, N, K, ldc, out_kind, seg1, seg2, vec;
  float s0, s1, s2, resid_scale;
  const float* a_scale;
  uint16_t* out_bf16;
  float* out_f32;
  const uint16_t* residual;
  unsigned int* status;
};

// ---- PTX wrappers -----------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D (tensor memory) (+)= A (smem) x B (smem)^T, both K-major; accumulate = 0 overwrites D.
__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when every MMA this thread issued so far has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor of a K-major tile whose rows are 128 bytes
// with the 128-byte swizzle (what the TMA load writes): 8-row groups 1024 bytes
// apart (stride byte offset), leading byte offset unused (1), descriptor version
// 1, layout type 2 (128-byte swizzle). Fields are in 16-byte units.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t smem_addr) {
  return uint64_t((smem_addr & 0x3ffffu) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) |
         (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// Instruction descriptor: f32 accumulator, e4m3 x e4m3, both operands K-major, N 256, M 128.
constexpr uint32_t kIdesc = (1u << 4) | (uint32_t(kBN >> 3) << 17) | (uint32_t(kBM >> 4) << 24);

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, Ring* ring, unsigned int* status) {
  volatile int* ab = &ring->abort;
  for (uint32_t i = 0; i < kMbarWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*ab) return false;
    if (i > 256) __nanosleep(64);
  }
  *ab = 1;
  if (status != nullptr) atomicOr(status, kStatusGemmWaitTimeout);
  return false;
}

__device__ __forceinline__ float seg_scale(const GemmParams& p, int n) {
  return n < p.seg1 ? p.s0 : (n < p.seg2 ? p.s1 : p.s2);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw + 1023u) & ~1023u;  // swizzled tiles sit on 1024-byte boundaries
  uint8_t* tiles_ptr = smem_raw + (tiles_addr - raw);
  Ring* ring = reinterpret_cast<Ring*>(tiles_ptr + size_t(kStages) * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(&ring->full[s], 1), mbar_init(&ring->empty[s], 1);
    for (int a = 0; a < kAccs; ++a) mbar_init(&ring->acc_full[a], 1), mbar_init(&ring->acc_empty[a], 4);
    ring->abort = 0;
    mbar_init_fence();
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc(smem_u32(&ring->tmem_base), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ring->tmem_base;

  pdl_begin();  // everything above touches no global memory

  const int mt = (p.M + kBM - 1) / kBM, nt = (p.N + kBN - 1) / kBN;
  const int tiles = mt * nt, kblocks = (p.K + kBK - 1) / kBK;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
        const int m0 = (t % mt) * kBM, n0 = (t / mt) * kBN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          if (!(ok = wait_or_abort(&ring->empty[s], ph ^ 1u, ring, p.status))) break;
          mbar_arrive_expect_tx(&ring->full[s], kStageBytes);
          const uint32_t dst = tiles_addr + s * kStageBytes;
          tma_load_2d(dst, &map_a, kb * kBK, m0, smem_u32(&ring->full[s]));
          tma_load_2d(dst + kABytes, &map_w, kb * kBK, n0, smem_u32(&ring->full[s]));
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++local) {
        const uint32_t acc = local & 1u, aph = (local >> 1) & 1u;
        if (!(ok = wait_or_abort(&ring->acc_empty[acc], aph ^ 1u, ring, p.status))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          if (!(ok = wait_or_abort(&ring->full[s], ph, ring, p.status))) break;
          tc_fence_after();
          const uint32_t a_addr = tiles_addr + s * kStageBytes;
          const uint64_t a_desc = smem_desc_k128(a_addr), w_desc = smem_desc_k128(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 32; ++k)  // 32 bytes of K per instruction: +2 in 16-byte units
            mma_f8(d_tmem, a_desc + uint64_t(2 * k), w_desc + uint64_t(2 * k), kIdesc, (kb | k) != 0);
          mma_commit(smem_u32(&ring->empty[s]));
        }
        if (ok) mma_commit(smem_u32(&ring->acc_full[acc]));
      }
    }
  } else {
    const int q = warp & 3;  // the 32 tensor-memory lanes this warp may read
    const float a_scale = p.a_scale != nullptr ? __ldg(p.a_scale) : 1.0f;
    const bool vec = p.vec != 0;
    uint32_t local = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++local) {
      const uint32_t acc = local & 1u, aph = (local >> 1) & 1u;
      const int m0 = (t % mt) * kBM, n0 = (t / mt) * kBN;
      if (!(ok = wait_or_abort(&ring->acc_full[acc], aph, ring, p.status))) break;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * kBN;
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        const int n = n0 + c * 32;
        if (n >= p.N) break;  // uniform over the warp
        uint32_t v[32];
        __syncwarp();  // the load below is a warp-wide instruction: rejoin lanes that skipped the stores
        tmem_ld32(taddr + c * 32, v);
        tmem_ld_wait();
        if (row >= p.M) continue;
        const bool one_scale = (n >= p.seg1 || n + 32 <= p.seg1) && (n >= p.seg2 || n + 32 <= p.seg2);
        const float sc0 = a_scale * seg_scale(p, n);
        float y[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) y[j] = (one_scale ? sc0 : a_scale * seg_scale(p, n + j)) * __uint_as_float(v[j]);
        const size_t off = size_t(row) * p.ldc + n;
        const bool full = vec && n + 32 <= p.N;
        if (p.out_kind == GRANITE4_GEMM_OUT_F32) {
          if (full) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<float4*>(p.out_f32 + off + j) = make_float4(y[j], y[j + 1], y[j + 2], y[j + 3]);
          } else {
            for (int j = 0; j < 32 && n + j < p.N; ++j) p.out_f32[off + j] = y[j];
          }
        } else {
          if (p.out_kind == GRANITE4_GEMM_OUT_RESIDUAL) {
            if (full) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                float r[8];
                unpack8(__ldg(reinterpret_cast<const uint4*>(p.residual + off + j)), r);
#pragma unroll
                for (int e = 0; e < 8; ++e) y[j + e] = __fadd_rn(r[e], __fmul_rn(p.resid_scale, y[j + e]));
              }
            } else {
              for (int j = 0; j < 32 && n + j < p.N; ++j)
                y[j] = __fadd_rn(bf16_to_f32(p.residual[off + j]), __fmul_rn(p.resid_scale, y[j]));
            }
          }
          if (full) {
#pragma unroll
            for (int j = 0; j < 32; j += 8)
              *reinterpret_cast<uint4*>(p.out_bf16 + off + j) =
                  make_uint4(pack_bf16x2(y[j], y[j + 1]), pack_bf16x2(y[j + 2], y[j + 3]),
                             pack_bf16x2(y[j + 4], y[j + 5]), pack_bf16x2(y[j + 6], y[j + 7]));
          } else {
            for (int j = 0; j < 32 && n + j < p.N; ++j) p.out_bf16[off + j] = uint16_t(f32_to_bf16_bits(y[j]));
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ring->acc_empty[acc]));
    }
  }

  // Wind down. On the normal path the epilogue has seen the last accumulator
  // complete, so no MMA and no copy is in flight. After an abort, give copies
  // and MMAs already issued a bounded time to land before the tensor memory and
  // the shared memory go away.
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (ring->abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---- host ---------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q{};
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

// A [rows][K] e4m3 matrix with row pitch ld bytes, fetched in boxes of 128 bytes x box_rows rows.
bool make_map(CUtensorMap* map, const void* base, int rows, int K, long long ld, int box_rows) {
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr) return false;
  const cuuint64_t dims[2] = {cuuint64_t(K), cuuint64_t(rows)};
  const cuuint64_t strides[1] = {cuuint64_t(ld)};
  const cuuint32_t box[2] = {cuuint32_t(kBK), cuuint32_t(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

extern "C" int granite4_kernel_gemm_fp8(int out_kind, const uint8_t* d_a, long long lda, const uint8_t* d_w, int M,
                                        int N, int K, const granite4_gemm_fp8_epilogue* ep) {
  static const char* fn = "granite4_kernel_gemm_fp8";
  if (M == 0 && N > 0 && K > 0 && ep != nullptr) return 0;  // no rows (an empty shard): nothing to do
  if (d_a == nullptr || d_w == nullptr || ep == nullptr) return fail(fn, "null argument");
  if (M < 0 || N <= 0 || K <= 0 || K % 16 != 0 || lda < K || lda % 16 != 0 || !aligned16(d_a) || !aligned16(d_w))
    return fail(fn, "needs K % 16 == 0, lda % 16 == 0, lda >= K and 16-byte aligned A and W");
  if (out_kind != GRANITE4_GEMM_OUT_BF16 && out_kind != GRANITE4_GEMM_OUT_F32 && out_kind != GRANITE4_GEMM_OUT_RESIDUAL)
    return fail(fn, "unknown output kind");
  if (ep->ldc < N) return fail(fn, "ldc < N");
  if (out_kind == GRANITE4_GEMM_OUT_F32 ? ep->d_out_f32 == nullptr : ep->d_out_bf16 == nullptr)
    return fail(fn, "the output of the requested kind is null");
  if (out_kind == GRANITE4_GEMM_OUT_RESIDUAL && ep->d_residual == nullptr) return fail(fn, "null residual");

  CUtensorMap map_a, map_w;
  if (!make_map(&map_a, d_a, M, K, lda, kBM) || !make_map(&map_w, d_w, N, K, K, kBN))
    return fail(fn, "the tensor map could not be encoded");

  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes));
  });
  G4_CUDA_TRY(fn, attr_err);

  GemmParams p{};
  p.M = M, p.N = N, p.K = K, p.ldc = ep->ldc, p.out_kind = out_kind;
  p.seg1 = ep->seg1, p.seg2 = ep->seg2;
  p.s0 = ep->w_scale0, p.s1 = ep->w_scale1, p.s2 = ep->w_scale2, p.resid_scale = ep->resid_scale;
  p.a_scale = ep->d_a_scale, p.out_bf16 = ep->d_out_bf16, p.out_f32 = ep->d_out_f32, p.residual = ep->d_residual;
  p.vec = (ep->ldc % 8 == 0) &&
          aligned16(out_kind == GRANITE4_GEMM_OUT_F32 ? static_cast<const void*>(ep->d_out_f32)
                                                      : static_cast<const void*>(ep->d_out_bf16)) &&
          (out_kind != GRANITE4_GEMM_OUT_RESIDUAL || aligned16(ep->d_residual));
  p.status = device_status_ptr();
  const int tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  G4_LAUNCH_PDL(fn, gemm_fp8_kernel, dim3(grid), dim3(kThreads), kSmemBytes, current_stream(), map_a, map_w, p);
  return 0;
}
