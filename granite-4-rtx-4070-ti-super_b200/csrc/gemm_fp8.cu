// FP8 x FP8 GEMM on the 5th-generation tensor cores (sm_100a).
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
// Shape of the kernel (its single-CTA form; the CTA-pair form for more than 128
// rows, the 16-row form with split K and the fused SwiGLU epilogue are described
// at Cfg, plan_split and store_accumulator_swiglu): persistent, one CTA per SM,
// 128 x 256 output tiles, K consumed in 128-byte blocks. Roles by warp:
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
#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>

#include "../../include/granite4_b200.h"
#include "g4_host.h"
#include "g4_math.cuh"
#include "g4_tcgen05.cuh"
#include "g4_tma.cuh"

namespace {

using namespace g4;

constexpr int kBM = 128, kBN = 256, kBK = 128;  // kBK in bytes = e4m3 elements
constexpr int kAccs = 2;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = kAccs * kBN;  // 512: the whole tensor memory of the SM
constexpr int kMaxStages = 6;
constexpr int kMaxSplits = 16;

// Forms of the kernel; all compute 256 output columns per tile: a stage costs the loader thread
// about 0.3 us of issue (barrier wait, expect_tx, two TMA instructions) whatever its size, so only
// 256-row W blocks (32 KB per stage) carry enough bytes per stage to keep up with HBM; 32- and
// 64-column tiles were measured at a quarter and a half of that rate.
// kPair = true: the two CTAs of a cluster own a 256 x 256 tile; each loads its 128 rows of A and
//   its 128 rows of W, and one thread of the leader CTA issues MMAs that run on both SMs
//   (cta_group::2), so each SM reads half as many W bytes from shared memory per flop.
// kPair = false: one CTA owns a 128 x 256 tile and both operand blocks. kARows = 16 loads only 16
//   rows of A per block (decode and verify steps): the MMA still reads 128 rows of shared
//   memory, the rest being whatever lies behind the 16 (rows of D that nobody reads).
// With at most 128 rows of A the GEMM is a stream of the weights and N / 256 tiles are too few to
// occupy the SMs; the single forms then also split K (see plan_split).
template <bool kPair, int kARows_, int kStages_>
struct Cfg {
  static constexpr int kARows = kARows_, kStages = kStages_;
  static constexpr int kWRows = kPair ? kBN / 2 : kBN;
  static constexpr uint32_t kABytes = kARows * kBK, kWBytes = kWRows * kBK;
  static constexpr uint32_t kStageBytes = kABytes + kWBytes;
  static constexpr int kTileM = kPair ? 2 * kBM : kBM;
  // the MMA reads kBM rows of A wherever kARows ends: keep that inside the allocation
  static constexpr size_t kSmemBytes = 1024 + size_t(kStages) * kStageBytes + (kBM - kARows) * kBK + 256;
  // Instruction descriptor: f32 accumulator, e4m3 x e4m3, both operands K-major, N 256, M 128 / 256.
  static constexpr uint32_t kIdesc = (1u << 4) | (uint32_t(kBN >> 3) << 17) | (uint32_t(kTileM >> 4) << 24);
  static_assert(kStages <= kMaxStages && kSmemBytes <= 227 * 1024, "ring too large");
  static_assert(!kPair || kARows == kBM, "the pair form loads whole A blocks");
};
using CfgPair = Cfg<true, 128, 6>;
using CfgWide = Cfg<false, 128, 4>;
using CfgSkinny = Cfg<false, 16, 5>;

struct Ring {
  uint64_t full[kMaxStages], empty[kMaxStages], acc_full[kAccs], acc_empty[kAccs];
  uint32_t tmem_base;
  int abort;
  int last;  // split K: whether this CTA delivered the last partial of the current tile
};
static_assert(sizeof(Ring) <= 256, "the ring's bookkeeping has 256 bytes after the tiles");

struct GemmParams {
  int M, N, K, ldc, out_kind, seg1, seg2, vec;
  float s0, s1, s2, resid_scale;
  const float* a_scale;
  uint16_t* out_bf16;
  float* out_f32;
  const uint16_t* residual;
  unsigned int* status;
  // split K: unit u covers k blocks [(u % splits) * kb_per, ...) of tile u / splits; partial sums go
  // to ws [tile][split][rows kept][256] and the CTA that brings a tile's count to `splits` adds them
  int splits, kb_per, ws_rows;
  int early;  // decode-size launch: see the dependent-launch note in the kernel
  // stream form (gemm_fp8_stream_kernel): tile columns, k blocks per stage, rows of A fetched, ring depth
  int bn, kc, a_rows, stages;
  int box3d;  // one TMA box spans the kc k-blocks of a stage (needs K % 128 == 0)
  // fused SwiGLU (out_kind SWIGLU): W is gate rows [0, I) then up rows [I, 2 I); a tile is 128 output
  // columns whose accumulator holds gate in columns 0..127 and up in 128..255
  int swiglu_i;      // I, or 0 when the epilogue is not the fused SwiGLU
  float* amax_slot;  // {scale, amax} of the activations: the epilogue maxes |a| into [1]
  float* ws;
  unsigned int* counters;
};

// ---- PTX wrappers -----------------------------------------------------------
// Tiled TMA load of one box into this CTA's shared memory. In the pair form the completion is
// counted on the leader CTA's barrier (`bar` is then a cluster-window address).
template <bool kPair>
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  if constexpr (kPair) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
  }
}
// 3-D box {128 bytes, rows, k-blocks}: lands as consecutive K-major 128-byte-swizzled blocks [k-block][row][128].
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
// D (tensor memory) (+)= A (smem) x B (smem)^T, both K-major; accumulate = 0 overwrites D.
template <bool kPair>
__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if constexpr (kPair) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
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

// AND of `ok` over the 128 epilogue threads (named barrier 1); every one of them calls it.
__device__ __forceinline__ bool epilogue_all(bool ok) {
  uint32_t all;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(all)
      : "r"(uint32_t(ok))
      : "memory");
  return all != 0;
}

__device__ __forceinline__ float seg_scale(const GemmParams& p, int n) {
  return n < p.seg1 ? p.s0 : (n < p.seg2 ? p.s1 : p.s2);
}

// Epilogue of 32 consecutive columns n .. n + 31 of one output row from the f32 sums v: scale,
// add the residual where asked, convert, store (engine/src/prefill_gemm.cu:65-88).
// n_end: first column that is not this call's to write (the tile's end or N).
__device__ __forceinline__ void store_chunk(const GemmParams& p, const float (&v)[32], int row, int n, float a_scale,
                                            int n_end) {
  const bool one_scale = (n >= p.seg1 || n + 32 <= p.seg1) && (n >= p.seg2 || n + 32 <= p.seg2);
  const float sc0 = a_scale * seg_scale(p, n);
  float y[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) y[j] = (one_scale ? sc0 : a_scale * seg_scale(p, n + j)) * v[j];
  const size_t off = size_t(row) * p.ldc + n;
  const bool full = p.vec != 0 && n + 32 <= n_end;
  if (p.out_kind == GRANITE4_GEMM_OUT_F32) {
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(p.out_f32 + off + j) = make_float4(y[j], y[j + 1], y[j + 2], y[j + 3]);
    } else {
      for (int j = 0; j < 32 && n + j < n_end; ++j) p.out_f32[off + j] = y[j];
    }
    return;
  }
  if (p.out_kind == GRANITE4_GEMM_OUT_RESIDUAL) {
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        float r[8];
        unpack8(*reinterpret_cast<const uint4*>(p.residual + off + j), r);  // may alias the output: plain load
#pragma unroll
        for (int e = 0; e < 8; ++e) y[j + e] = __fadd_rn(r[e], __fmul_rn(p.resid_scale, y[j + e]));
      }
    } else {
      for (int j = 0; j < 32 && n + j < n_end; ++j)
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
    for (int j = 0; j < 32 && n + j < n_end; ++j) p.out_bf16[off + j] = uint16_t(f32_to_bf16_bits(y[j]));
  }
}

// The same epilogue for four consecutive columns n .. n + 3 (n a multiple of 4) of one row.
__device__ __forceinline__ void store4(const GemmParams& p, float4 v, int row, int n, float a_scale) {
  float y[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) y[j] = (a_scale * seg_scale(p, n + j)) * y[j];
  const size_t off = size_t(row) * p.ldc + n;
  const bool full = p.vec != 0 && n + 4 <= p.N;
  if (p.out_kind == GRANITE4_GEMM_OUT_F32) {
    if (full) {
      *reinterpret_cast<float4*>(p.out_f32 + off) = make_float4(y[0], y[1], y[2], y[3]);
    } else {
      for (int j = 0; j < 4 && n + j < p.N; ++j) p.out_f32[off + j] = y[j];
    }
    return;
  }
  if (p.out_kind == GRANITE4_GEMM_OUT_RESIDUAL) {
    if (full) {
      const uint2 r = *reinterpret_cast<const uint2*>(p.residual + off);  // may alias the output: plain load
      y[0] = __fadd_rn(bf16_lo(r.x), __fmul_rn(p.resid_scale, y[0])), y[1] = __fadd_rn(bf16_hi(r.x), __fmul_rn(p.resid_scale, y[1]));
      y[2] = __fadd_rn(bf16_lo(r.y), __fmul_rn(p.resid_scale, y[2])), y[3] = __fadd_rn(bf16_hi(r.y), __fmul_rn(p.resid_scale, y[3]));
    } else {
      for (int j = 0; j < 4 && n + j < p.N; ++j)
        y[j] = __fadd_rn(bf16_to_f32(p.residual[off + j]), __fmul_rn(p.resid_scale, y[j]));
    }
  }
  if (full) {
    *reinterpret_cast<uint2*>(p.out_bf16 + off) = make_uint2(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]));
  } else {
    for (int j = 0; j < 4 && n + j < p.N; ++j) p.out_bf16[off + j] = uint16_t(f32_to_bf16_bits(y[j]));
  }
}

// Fused SwiGLU epilogue of one warp's 32 rows: gate from columns 0..127 and up from columns 128..255 of
// the accumulator, a = bf16(silu(g) u) (the arithmetic of the standalone kernel, g4_math.cuh swiglu) for
// output columns n0 .. n0 + 127, and the running max |a| of what was stored (packed bf16 pairs).
__device__ __forceinline__ uint32_t store_accumulator_swiglu(const GemmParams& p, uint32_t taddr, int row, int n0,
                                                             float a_scale) {
  uint32_t amax = 0u;
  const int I = p.swiglu_i;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    const int n = n0 + c * 32;
    if (n >= I) break;  // uniform over the warp
    uint32_t gv[32], uv[32];
    __syncwarp();
    tmem_ld32(taddr + c * 32, gv);
    tmem_ld32(taddr + 128 + c * 32, uv);
    tmem_ld_wait();
    if (row >= p.M) continue;
    const bool one_scale = (n >= p.seg1 || n + 32 <= p.seg1) && (n >= p.seg2 || n + 32 <= p.seg2) &&
                           (I + n >= p.seg1 || I + n + 32 <= p.seg1) && (I + n >= p.seg2 || I + n + 32 <= p.seg2);
    const float sg0 = a_scale * seg_scale(p, n), su0 = a_scale * seg_scale(p, I + n);
    uint32_t w[16];
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const float sg_a = one_scale ? sg0 : a_scale * seg_scale(p, n + j), sg_b = one_scale ? sg0 : a_scale * seg_scale(p, n + j + 1);
      const float su_a = one_scale ? su0 : a_scale * seg_scale(p, I + n + j), su_b = one_scale ? su0 : a_scale * seg_scale(p, I + n + j + 1);
      const float a0 = swiglu(__fmul_rn(sg_a, __uint_as_float(gv[j])), __fmul_rn(su_a, __uint_as_float(uv[j])));
      const float a1 = swiglu(__fmul_rn(sg_b, __uint_as_float(gv[j + 1])), __fmul_rn(su_b, __uint_as_float(uv[j + 1])));
      w[j / 2] = pack_bf16x2(a0, a1);
    }
    const size_t off = size_t(row) * p.ldc + n;
    if (p.vec != 0 && n + 32 <= I) {
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        *reinterpret_cast<uint4*>(p.out_bf16 + off + 2 * j) = make_uint4(w[j], w[j + 1], w[j + 2], w[j + 3]);
        amax = amax_acc(amax, make_uint4(w[j], w[j + 1], w[j + 2], w[j + 3]));
      }
    } else {
      for (int j = 0; j < 32 && n + j < I; ++j) {
        const uint32_t bits = (j & 1) ? (w[j / 2] >> 16) : (w[j / 2] & 0xffffu);
        p.out_bf16[off + j] = uint16_t(bits);
        amax = amax_acc(amax, bits);
      }
    }
  }
  return amax;
}

// One warp's 32 rows x 256 columns of a finished accumulator: tensor memory -> epilogue -> global,
// or (partial != NULL, split K) tensor memory -> this unit's f32 partial rows [.][256].
// Every lane executes the tensor-memory loads; lanes past row M skip the stores.
__device__ __forceinline__ void store_accumulator(const GemmParams& p, uint32_t taddr, int row, int n0, float a_scale,
                                                  float* partial_row) {
#pragma unroll 1
  for (int c = 0; c < kBN / 32; ++c) {
    const int n = n0 + c * 32;
    if (n >= p.N) break;  // uniform over the warp
    uint32_t v[32];
    __syncwarp();  // the load below is a warp-wide instruction: rejoin lanes that skipped the stores
    tmem_ld32(taddr + c * 32, v);
    tmem_ld_wait();
    if (row >= p.M) continue;
    if (partial_row != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        __stcg(reinterpret_cast<uint4*>(partial_row + c * 32 + j), make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]));
    } else {
      float f[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
      store_chunk(p, f, row, n, a_scale, p.N);
    }
  }
}

template <class C>
__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                const GemmParams p) {
  constexpr bool kPair = C::kTileM == 2 * kBM;
  constexpr uint32_t kABytes = C::kABytes;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw + 1023u) & ~1023u;  // swizzled tiles sit on 1024-byte boundaries
  uint8_t* tiles_ptr = smem_raw + (tiles_addr - raw);
  Ring* ring = reinterpret_cast<Ring*>(tiles_ptr + size_t(C::kStages) * C::kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = kPair ? cluster_rank() : 0u;  // CTA of the pair; 0 leads
  const bool leader = rank == 0u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) mbar_init(&ring->full[s], 1), mbar_init(&ring->empty[s], 1);
    // a finished accumulator is released by the four epilogue warps of every CTA that reads it;
    // in the pair form only the leader's barriers of this kind are waited on
    for (int a = 0; a < kAccs; ++a) mbar_init(&ring->acc_full[a], 1), mbar_init(&ring->acc_empty[a], kPair ? 8 : 4);
    ring->abort = 0;
    mbar_init_fence();
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc<kPair>(smem_u32(&ring->tmem_base), kTmemCols);
  tc_fence_before();
  __syncwarp();  // the cluster barrier is a warp-wide instruction
  if constexpr (kPair) cluster_sync(); else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ring->tmem_base;

  // Programmatic dependent launch. Everything above touches no global memory. The weights are
  // constants of the model, not products of the kernel before this one on the stream, so the
  // loader thread of the decode-size forms (p.early) fetches the first stages' W blocks before it
  // waits for that kernel; whatever reads activations, residuals, scales or the workspace, and
  // everything that writes, comes after the wait. Those forms also let the kernel after them
  // start as soon as CTAs of this one retire: with a few microseconds of work per launch, the
  // ramps of consecutive GEMMs are most of the time otherwise.
  const bool loader = warp == 0 && lane == 0;
  if (p.early) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!(loader && p.early)) pdl_begin();

  const int tile_cols = p.swiglu_i ? kBN / 2 : kBN;  // output columns of a tile
  const int mt = (p.M + C::kTileM - 1) / C::kTileM, nt = ((p.swiglu_i ? p.swiglu_i : p.N) + tile_cols - 1) / tile_cols;
  const int tiles = mt * nt, kblocks = (p.K + kBK - 1) / kBK;
  const int units = tiles * p.splits;  // splits == 1 unless K is split
  const int first = kPair ? int(blockIdx.x >> 1) : int(blockIdx.x);
  const int step = kPair ? int(gridDim.x >> 1) : int(gridDim.x);

  if (warp == 0) {
    if (lane == 0) {
      // Pair form: both CTAs load their own halves; every completion is counted on the leader's
      // `full` barrier, which the leader arms for both halves. The peer may refill a stage when
      // the leader has seen the MMAs that read it complete, which the leader passes on.
      const uint32_t full0 = kPair ? cluster_addr(smem_u32(&ring->full[0]), 0) : smem_u32(&ring->full[0]);
      uint32_t it = 0, ahead = 0;  // ahead: stages whose W block was fetched before the dependency wait
      if (!kPair && p.early) {
        for (int u = first; u < units && ahead < uint32_t(C::kStages); u += step) {
          const int t = u / p.splits, kb0 = (u % p.splits) * p.kb_per, kb1 = min(kblocks, kb0 + p.kb_per);
          for (int kb = kb0; kb < kb1 && ahead < uint32_t(C::kStages); ++kb, ++ahead) {
            mbar_arrive_expect_tx(&ring->full[ahead], C::kStageBytes);  // first use of every stage: it is empty
            const uint32_t wdst = tiles_addr + ahead * C::kStageBytes + kABytes;
            if (p.swiglu_i) {  // two boxes of 128 rows: gate rows, then up rows
              tma_load_2d<kPair>(wdst, &map_w, kb * kBK, (t / mt) * tile_cols, smem_u32(&ring->full[ahead]));
              tma_load_2d<kPair>(wdst + C::kWBytes / 2, &map_w, kb * kBK, p.swiglu_i + (t / mt) * tile_cols,
                                 smem_u32(&ring->full[ahead]));
            } else {
              tma_load_2d<kPair>(wdst, &map_w, kb * kBK, (t / mt) * kBN, smem_u32(&ring->full[ahead]));
            }
          }
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
      }
      bool ok = true;
      for (int u = first; u < units && ok; u += step) {
        const int t = u / p.splits, kb0 = (u % p.splits) * p.kb_per, kb1 = min(kblocks, kb0 + p.kb_per);
        const int m0 = (t % mt) * C::kTileM + int(rank) * kBM;
        // W rows of this CTA's block: its half (pair) or all (single) of the tile's 256 columns; with the
        // fused SwiGLU, columns 0..127 are gate rows n0.. and columns 128..255 are up rows I + n0..
        const int n0 = p.swiglu_i ? (t / mt) * tile_cols + (kPair && rank ? p.swiglu_i : 0)
                                  : (t / mt) * kBN + int(rank) * C::kWRows;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
          const uint32_t dst = tiles_addr + s * C::kStageBytes, bar = full0 + s * uint32_t(sizeof(uint64_t));
          if (it < ahead) {  // armed and half loaded above
            tma_load_2d<kPair>(dst, &map_a, kb * kBK, m0, bar);
            continue;
          }
          if (!(ok = wait_or_abort(&ring->empty[s], (kPair && !leader) ? ph : (ph ^ 1u), ring, p.status))) break;
          if (leader) {
            mbar_arrive_expect_tx(&ring->full[s], (kPair ? 2u : 1u) * C::kStageBytes);
            if constexpr (kPair) mbar_arrive_remote(smem_u32(&ring->empty[s]), 1);
          }
          tma_load_2d<kPair>(dst, &map_a, kb * kBK, m0, bar);
          tma_load_2d<kPair>(dst + kABytes, &map_w, kb * kBK, n0, bar);
          if (!kPair && p.swiglu_i)
            tma_load_2d<kPair>(dst + kABytes + C::kWBytes / 2, &map_w, kb * kBK, p.swiglu_i + n0, bar);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int u = first; u < units && ok; u += step, ++local) {
        const int kb0 = (u % p.splits) * p.kb_per, kb1 = min(kblocks, kb0 + p.kb_per);
        const uint32_t acc = local & 1u, aph = (local >> 1) & 1u;
        if (!(ok = wait_or_abort(&ring->acc_empty[acc], aph ^ 1u, ring, p.status))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % C::kStages, ph = (it / C::kStages) & 1u;
          if (!(ok = wait_or_abort(&ring->full[s], ph, ring, p.status))) break;
          tc_fence_after();
          const uint32_t a_addr = tiles_addr + s * C::kStageBytes;
          const uint64_t a_desc = smem_desc_k128(a_addr), w_desc = smem_desc_k128(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < kBK / 32; ++k)  // 32 bytes of K per instruction: +2 in 16-byte units
            mma_f8<kPair>(d_tmem, a_desc + uint64_t(2 * k), w_desc + uint64_t(2 * k), C::kIdesc, (kb > kb0) || k != 0);
          mma_commit<kPair>(smem_u32(&ring->empty[s]));
        }
        if (ok) mma_commit<kPair>(smem_u32(&ring->acc_full[acc]));
      }
    }
  } else {
    const int q = warp & 3;  // the 32 tensor-memory lanes this warp may read
    const float a_scale = p.a_scale != nullptr ? __ldg(p.a_scale) : 1.0f;
    const int et = int(threadIdx.x) - 64;  // 0..127 among the epilogue threads
    uint32_t local = 0;
    bool ok = true;
    for (int u = first; u < units && ok; u += step, ++local) {
      const int t = u / p.splits, sl = u % p.splits;
      const uint32_t acc = local & 1u, aph = (local >> 1) & 1u;
      const int m0 = (t % mt) * C::kTileM + int(rank) * kBM, n0 = (t / mt) * tile_cols;
      ok = wait_or_abort(&ring->acc_full[acc], aph, ring, p.status);
      if (p.splits > 1) ok = epilogue_all(ok);  // the split path below has barriers: leave it together or not at all
      if (!ok) break;
      // the leader learns from its own barrier that both halves of the accumulator are complete
      // and tells the peer
      if (kPair && leader && warp == 2 && lane == 0) mbar_arrive_remote(smem_u32(&ring->acc_full[acc]), 1);
      tc_fence_after();
      float* partial = p.splits > 1 ? p.ws + (size_t(t) * p.splits + sl) * p.ws_rows * kBN : nullptr;
      if (p.swiglu_i) {
        if (m0 + q * 32 < p.M) {
          const uint32_t amax = amax_warp(store_accumulator_swiglu(p, tmem_base + (uint32_t(q * 32) << 16) + acc * kBN,
                                                                   m0 + q * 32 + lane, n0, a_scale));
          if (lane == 0 && amax != 0u) atomic_amax(p.amax_slot + 1, amax_value(amax));
        }
      } else if (m0 + q * 32 < p.M)  // uniform over the warp: a warp whose rows are all past M has nothing to read
        store_accumulator(p, tmem_base + (uint32_t(q * 32) << 16) + acc * kBN, m0 + q * 32 + lane, n0, a_scale,
                          partial != nullptr ? partial + size_t(q * 32 + lane) * kBN : nullptr);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (kPair && !leader) mbar_arrive_remote(smem_u32(&ring->acc_empty[acc]), 0);
        else mbar_arrive(smem_u32(&ring->acc_empty[acc]));
      }
      if (partial != nullptr) {
        // Deterministic split-K sum: every unit publishes its partial, then counts itself in; the
        // unit that completes the count adds the partials in split order. Nobody waits.
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) ring->last = atomicAdd(p.counters + t, 1u) == unsigned(p.splits - 1);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (ring->last) {
          __threadfence();
          const int rows = min(p.ws_rows, p.M - m0);
          const float* base = p.ws + size_t(t) * p.splits * p.ws_rows * kBN;
          // four columns per thread and step: the loads of all splits are in flight together (one
          // round trip to L2), the additions then run in split order
          for (int g = et; g < rows * (kBN / 4); g += 128) {
            const int r = g / (kBN / 4), c = (g % (kBN / 4)) * 4;
            if (n0 + c >= p.N) continue;
            float4 x[kMaxSplits];
#pragma unroll
            for (int s2 = 0; s2 < kMaxSplits; ++s2)
              if (s2 < p.splits) x[s2] = __ldcg(reinterpret_cast<const float4*>(base + (size_t(s2) * p.ws_rows + r) * kBN + c));
            float4 v = x[0];
#pragma unroll
            for (int s2 = 1; s2 < kMaxSplits; ++s2)
              if (s2 < p.splits)
                v.x = __fadd_rn(v.x, x[s2].x), v.y = __fadd_rn(v.y, x[s2].y), v.z = __fadd_rn(v.z, x[s2].z),
                v.w = __fadd_rn(v.w, x[s2].w);
            store4(p, v, m0 + r, n0 + c, a_scale);
          }
          if (et == 0) p.counters[t] = 0u;  // the workspace is ready for the next call
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // ring->last is rewritten by the next unit
      }
    }
  }

  // Wind down. On the normal path the epilogue has seen the last accumulator
  // complete, so no MMA and no copy is in flight. After an abort, give copies
  // and MMAs already issued a bounded time to land before the tensor memory and
  // the shared memory go away. In the pair form neither CTA leaves (or frees
  // tensor memory) before both are here: each reads or signals the other's
  // shared memory until then.
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (ring->abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
  }
  __syncwarp();
  if constexpr (kPair) cluster_sync(); else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<kPair>(tmem_base, kTmemCols);
  }
}

// ---- at most 128 rows: a stream of the weights ---------------------------------------------------
// With few rows the GEMM is one pass over W and the question is only how to keep every SM fetching.
// A tile is p.bn output columns (a multiple of 16, chosen by the host so that the tiles are about
// one per SM) times ALL of K: no split of K, no partial sums, no workspace. A stage of the ring holds
// p.kc k-blocks; lanes 0 .. kc - 1 of the loader warp each issue the two TMA loads of one k-block,
// because one thread gets through only about three loads per microsecond and a 32-column block is
// just 4 KB. The MMA thread issues 4 p.kc MMAs (M 128, N p.bn, K 32) per stage; an MMA of up to 32
// columns takes ~46 cycles (measured; 64 -> 48, 128 -> 64, 256 -> 128), so a 32-column tile
// consumes 22 weight bytes per cycle, just under an SM's share of HBM. p.a_rows = 16 fetches only
// 16 rows of A per block (the MMA reads 128 rows of shared memory wherever the 16 end: rows of D
// nobody reads). Roles, barriers and the bounded waits are those of gemm_fp8_kernel.
constexpr int kStreamMaxStages = 8;
struct StreamRing {
  uint64_t full[kStreamMaxStages], empty[kStreamMaxStages], acc_full[kAccs], acc_empty[kAccs];
  uint32_t tmem_base;
  int abort;
};
constexpr size_t kStreamTileBytes = 192 * 1024;  // the ring
constexpr size_t kStreamSmemBytes = 1024 + kStreamTileBytes + (kBM - 16) * kBK + 256;

__device__ __forceinline__ bool stream_wait(uint64_t* bar, uint32_t parity, StreamRing* ring, unsigned int* status) {
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

__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_stream_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                       const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw + 1023u) & ~1023u;
  StreamRing* ring = reinterpret_cast<StreamRing*>(smem_raw + (tiles_addr - raw) + kStreamTileBytes + (kBM - 16) * kBK);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t a_blk = uint32_t(p.a_rows) * kBK, w_blk = uint32_t(p.bn) * kBK;
  const uint32_t stage_bytes = uint32_t(p.kc) * (a_blk + w_blk);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) mbar_init(&ring->full[s], 1), mbar_init(&ring->empty[s], 1);
    for (int a = 0; a < kAccs; ++a) mbar_init(&ring->acc_full[a], 1), mbar_init(&ring->acc_empty[a], 4);
    ring->abort = 0;
    mbar_init_fence();
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc<false>(smem_u32(&ring->tmem_base), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ring->tmem_base;

  // Programmatic dependent launch as in the 16-row form of gemm_fp8_kernel: the loader warp fetches
  // W (a constant of the model) before it waits for the kernel ahead of it on the stream.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (warp != 0) pdl_begin();

  const int tiles = (p.N + p.bn - 1) / p.bn, kblocks = (p.K + kBK - 1) / kBK;
  const int stages_per_tile = (kblocks + p.kc - 1) / p.kc;

  if (warp == 0) {
    // stage it (counted over this CTA's tiles) covers k-blocks [kc (it % spt), ...) of tile
    // blockIdx.x + gridDim.x (it / spt); lane j loads block j of the stage
    const long long total = (long long)stages_per_tile * ((tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x));
    auto issue = [&](long long it, bool load_a, bool load_w) {
      const int t = int(blockIdx.x) + int(gridDim.x) * int(it / stages_per_tile);
      const int kb = int(it % stages_per_tile) * p.kc + (p.box3d ? 0 : lane), nblk = min(p.kc, kblocks - int(it % stages_per_tile) * p.kc);
      const uint32_t s = uint32_t(it % p.stages);
      const uint32_t dst = tiles_addr + s * stage_bytes, bar = smem_u32(&ring->full[s]);
      if (p.box3d) {  // one box per operand and stage; k-blocks past K are filled with zeros
        if (lane == 0) {
          if (load_a) tma_load_3d(dst, &map_a, 0, 0, kb, bar);
          if (load_w) tma_load_3d(dst + p.kc * a_blk, &map_w, 0, t * p.bn, kb, bar);
        }
      } else if (lane < nblk) {
        if (load_a) tma_load_2d<false>(dst + lane * a_blk, &map_a, kb * kBK, 0, bar);
        if (load_w) tma_load_2d<false>(dst + p.kc * a_blk + lane * w_blk, &map_w, kb * kBK, t * p.bn, bar);
      }
      return nblk;
    };
    long long ahead = 0;
    for (; ahead < total && ahead < p.stages; ++ahead) {  // first use of every stage: it is empty
      const int nblk = p.box3d ? p.kc : min(p.kc, kblocks - int(ahead % stages_per_tile) * p.kc);
      if (lane == 0) mbar_arrive_expect_tx(&ring->full[ahead], uint32_t(nblk) * (a_blk + w_blk));
      __syncwarp();
      issue(ahead, false, true);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    bool ok = true;
    for (long long it = 0; it < total && ok; ++it) {
      if (it < ahead) {
        issue(it, true, false);
        continue;
      }
      const uint32_t s = uint32_t(it % p.stages), ph = uint32_t(it / p.stages) & 1u;
      if (lane == 0) ok = stream_wait(&ring->empty[s], ph ^ 1u, ring, p.status);
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      const int nblk = p.box3d ? p.kc : min(p.kc, kblocks - int(it % stages_per_tile) * p.kc);
      if (lane == 0) mbar_arrive_expect_tx(&ring->full[s], uint32_t(nblk) * (a_blk + w_blk));
      __syncwarp();
      issue(it, true, true);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (uint32_t(p.bn >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
      long long it = 0;
      uint32_t local = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++local) {
        const uint32_t acc = local & 1u, aph = (local >> 1) & 1u;
        if (!(ok = stream_wait(&ring->acc_empty[acc], aph ^ 1u, ring, p.status))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int st = 0; st < stages_per_tile; ++st, ++it) {
          const uint32_t s = uint32_t(it % p.stages), ph = uint32_t(it / p.stages) & 1u;
          if (!(ok = stream_wait(&ring->full[s], ph, ring, p.status))) break;
          tc_fence_after();
          const uint32_t base = tiles_addr + s * stage_bytes;
          const int nblk = min(p.kc, kblocks - st * p.kc);
          for (int j = 0; j < nblk; ++j) {
            const uint64_t a_desc = smem_desc_k128(base + j * a_blk), w_desc = smem_desc_k128(base + p.kc * a_blk + j * w_blk);
#pragma unroll
            for (int k = 0; k < kBK / 32; ++k)
              mma_f8<false>(d_tmem, a_desc + uint64_t(2 * k), w_desc + uint64_t(2 * k), idesc, (st | j | k) != 0);
          }
          mma_commit<false>(smem_u32(&ring->empty[s]));
        }
        if (ok) mma_commit<false>(smem_u32(&ring->acc_full[acc]));
      }
    }
  } else {
    const int q = warp & 3;
    const float a_scale = p.a_scale != nullptr ? __ldg(p.a_scale) : 1.0f;
    uint32_t local = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++local) {
      const uint32_t acc = local & 1u, aph = (local >> 1) & 1u;
      const int n0 = t * p.bn, n_end = min(p.N, n0 + p.bn), row = q * 32 + lane;
      if (!(ok = stream_wait(&ring->acc_full[acc], aph, ring, p.status))) break;
      tc_fence_after();
      if (q * 32 < p.M) {  // uniform over the warp
        const uint32_t taddr = tmem_base + (uint32_t(q * 32) << 16) + acc * kBN;
#pragma unroll 1
        for (int c = 0; n0 + c * 32 < n_end; ++c) {
          uint32_t v[32];
          __syncwarp();
          tmem_ld32(taddr + c * 32, v);
          tmem_ld_wait();
          if (row >= p.M) continue;
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          store_chunk(p, f, row, n0 + c * 32, a_scale, n_end);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ring->acc_empty[acc]));
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (ring->abort) {  // give copies and MMAs already issued a bounded time to land
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<false>(tmem_base, kTmemCols);
  }
}

// ---- at most 16 rows: the weights as the M operand ---------------------------------------------------
// A decode or verify step multiplies 1 .. 16 rows by every weight matrix: the GEMM is one pass over W,
// and an MMA whose M side is the (mostly empty) activation tile gets through too few weight bytes per
// instruction to keep up with an SM's share of HBM. Here the operands change sides: D^T = W A^T, so
// one MMA (M 128 weight rows, N 16 activation rows, K 32) consumes 4 KB of weights, and the
// accumulator is 128 tensor-memory lanes (output columns) by 16 columns (output rows).
//
// A unit is 128 weight rows times a slice of K; the grid is one CTA per unit and is not persistent.
// The CTA is small (a 90 KB ring, 32 columns of tensor memory) so that two are resident per SM: while
// one drains its accumulator the other streams, and under programmatic dependent launch the CTAs of
// the next GEMM on the stream move in and fetch their first weight blocks while this one finishes.
//
// The slices of one tile are the CTAs of one thread-block cluster, and their partial sums meet in
// distributed shared memory as a reduce-scatter: rank o owns a chunk of the tile's 128 columns; the
// epilogue thread of every other rank that holds one of those columns stores its partial sums into
// rank o's receive buffer and arrives (release, cluster scope) on rank o's mbarrier; the owner's
// thread for the column waits for that barrier (acquire), adds the partials in rank order - its own
// from registers in its place - and runs the epilogue. No workspace in global memory, no atomics,
// the same order of additions every time, and no cluster-wide barrier on the way out: the only one
// is at the start (every CTA is running and its barriers exist before anyone writes to it), where
// it overlaps the first loads.
//
// Roles: warp 0, lanes 0 .. 4: lane s owns ring stage s (k-blocks s, s + 5, ...): arms its barrier and
// issues the two TMA loads, the first W block before the wait on the kernel ahead of this one on the
// stream; warp 1: tensor-memory allocation, one thread issues the MMAs; warps 2-5: accumulator ->
// registers, exchange, epilogue. Every mbarrier wait is bounded as in the other forms.
constexpr int kDecStages = 5, kDecRows = 16;
constexpr uint32_t kDecWBytes = kBM * kBK, kDecABytes = kDecRows * kBK, kDecStageBytes = kDecWBytes + kDecABytes;
constexpr uint32_t kDecTmemCols = 32;
constexpr int kDecMaxSplits = 8;  // the portable cluster size
constexpr uint32_t kDecRecvBytes = 10240;
constexpr size_t kDecSmemBytes = 1024 + size_t(kDecStages) * kDecStageBytes + kDecRecvBytes + 256;
struct DecRing {
  uint64_t full[kDecStages], empty[kDecStages], acc_full, red_full;
  uint32_t tmem_base;
  int abort;
};

// Columns of a tile owned by one rank of a cluster of `splits`: a multiple of 8, so that an owner's
// bf16 row segment starts on a 16-byte boundary. (splits - 1) * 4 row groups * chunk * 16 bytes fit
// in kDecRecvBytes for every splits <= 8.
__host__ __device__ constexpr int dec_chunk(int splits) { return ((kBM + splits - 1) / splits + 7) / 8 * 8; }
static_assert(7 * 4 * dec_chunk(8) * 16 <= int(kDecRecvBytes) && 5 * 4 * dec_chunk(6) * 16 <= int(kDecRecvBytes) &&
                  4 * 4 * dec_chunk(5) * 16 <= int(kDecRecvBytes) && 3 * 4 * dec_chunk(4) * 16 <= int(kDecRecvBytes) &&
                  2 * 4 * dec_chunk(3) * 16 <= int(kDecRecvBytes) && 6 * 4 * dec_chunk(7) * 16 <= int(kDecRecvBytes) &&
                  1 * 4 * dec_chunk(2) * 16 <= int(kDecRecvBytes),
              "the receive buffer holds every rank's partial sums of the owned columns");

__device__ __forceinline__ bool dec_wait(uint64_t* bar, uint32_t parity, DecRing* ring, unsigned int* status) {
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
// The same wait with acquire semantics at cluster scope: what the arriving threads of other CTAs
// stored into this CTA's shared memory before their arrival is visible after it.
__device__ __forceinline__ bool dec_wait_cluster(uint64_t* bar, uint32_t parity, DecRing* ring, unsigned int* status) {
  volatile int* ab = &ring->abort;
  for (uint32_t i = 0; i < kMbarWaitLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (done) return true;
    if (*ab) return false;
    if (i > 256) __nanosleep(64);
  }
  *ab = 1;
  if (status != nullptr) atomicOr(status, kStatusGemmWaitTimeout);
  return false;
}

// 32 lanes x 16 consecutive 32-bit columns of tensor memory: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

__global__ void __launch_bounds__(kThreads, 2)
gemm_fp8_decode_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                       const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_addr = (raw + 1023u) & ~1023u;
  uint8_t* tiles_ptr = smem_raw + (tiles_addr - raw);
  uint8_t* recv_ptr = tiles_ptr + size_t(kDecStages) * kDecStageBytes;
  DecRing* ring = reinterpret_cast<DecRing*>(recv_ptr + kDecRecvBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int splits = p.splits;
  const uint32_t rank = splits > 1 ? cluster_rank() : 0u;  // the slice of K
  const int tile = int(blockIdx.x) / splits;
  const int kblocks = (p.K + kBK - 1) / kBK;
  const int kb0 = int(rank) * p.kb_per, kb1 = min(kblocks, kb0 + p.kb_per);
  const int chunk = dec_chunk(splits);
  const int owned = max(0, min(chunk, kBM - int(rank) * chunk));  // columns of the tile this rank finishes

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_a)) : "memory");
    for (int s = 0; s < kDecStages; ++s) mbar_init(&ring->full[s], 1), mbar_init(&ring->empty[s], 1);
    mbar_init(&ring->acc_full, 1);
    mbar_init(&ring->red_full, uint32_t(max(1, (splits - 1) * owned)));  // one arrival per partial column
    ring->abort = 0;
    mbar_init_fence();
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc<false>(smem_u32(&ring->tmem_base), kDecTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ring->tmem_base;
  // Split arrival on the cluster barrier: "this CTA runs and its barriers exist". Every thread waits
  // for it once, the epilogue threads just before they write to a peer, by when it is long complete.
  if (splits > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

  // The kernel after this one may move in as CTAs of this one retire. Only the threads that read
  // what the kernel ahead wrote (activations, their scale, the residual) or that write wait for it.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    if (lane < kDecStages) {
      const uint32_t dst = tiles_addr + uint32_t(lane) * kDecStageBytes, bar = smem_u32(&ring->full[lane]);
      int kb = kb0 + lane;
      const bool any = kb < kb1;
      if (any) {  // first use of the stage: it is empty; W is a constant of the model
        mbar_arrive_expect_tx(&ring->full[lane], kDecStageBytes);
        tma_load_2d<false>(dst, &map_w, kb * kBK, tile * kBM, bar);
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      if (any) tma_load_2d<false>(dst + kDecWBytes, &map_a, kb * kBK, 0, bar);
      uint32_t round = 1;
      for (kb += kDecStages; kb < kb1; kb += kDecStages, ++round) {
        if (!dec_wait(&ring->empty[lane], (round & 1u) ^ 1u, ring, p.status)) break;
        mbar_arrive_expect_tx(&ring->full[lane], kDecStageBytes);
        tma_load_2d<false>(dst, &map_w, kb * kBK, tile * kBM, bar);
        tma_load_2d<false>(dst + kDecWBytes, &map_a, kb * kBK, 0, bar);
      }
    }
    __syncwarp();
    if (splits > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  } else if (warp == 1) {
    if (lane == 0) {
      // f32 accumulator, e4m3 x e4m3, both operands K-major, N 16, M 128
      constexpr uint32_t idesc = (1u << 4) | (uint32_t(kDecRows >> 3) << 17) | (uint32_t(kBM >> 4) << 24);
      uint32_t it = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
        const uint32_t s = it % kDecStages, ph = (it / kDecStages) & 1u;
        if (!(ok = dec_wait(&ring->full[s], ph, ring, p.status))) break;
        tc_fence_after();
        const uint32_t w_addr = tiles_addr + s * kDecStageBytes;
        const uint64_t w_desc = smem_desc_k128(w_addr), a_desc = smem_desc_k128(w_addr + kDecWBytes);
#pragma unroll
        for (int k = 0; k < kBK / 32; ++k)
          mma_f8<false>(tmem_base, w_desc + uint64_t(2 * k), a_desc + uint64_t(2 * k), idesc, (it | uint32_t(k)) != 0u);
        mma_commit<false>(smem_u32(&ring->empty[s]));
      }
      if (ok) mma_commit<false>(smem_u32(&ring->acc_full));
    }
    __syncwarp();
    if (splits > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  } else {
    const int et = (warp & 3) * 32 + lane;  // the tensor-memory lane this thread reads = the tile's column
    const int n = tile * kBM + et;
    const int groups = (p.M + 3) / 4;       // float4 groups of rows that carry data
    const int owner = et / chunk;           // the rank that finishes this column
    const bool mine = owner == int(rank);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // what the epilogue needs from global memory, requested before the accumulator is complete
    float sc = 0.0f;
    uint16_t resid[kDecRows];
    if (mine && n < p.N) {
      sc = (p.a_scale != nullptr ? __ldg(p.a_scale) : 1.0f) * seg_scale(p, n);
      if (p.out_kind == GRANITE4_GEMM_OUT_RESIDUAL) {
#pragma unroll
        for (int j = 0; j < kDecRows; ++j)
          if (j < p.M) resid[j] = p.residual[size_t(j) * p.ldc + n];  // may alias the output: plain loads
      }
    }
    bool ok = dec_wait(&ring->acc_full, 0u, ring, p.status);
    tc_fence_after();
    __syncwarp();
    uint32_t v[kDecRows];
    tmem_ld16(tmem_base + (uint32_t((warp & 3) * 32) << 16), v);
    tmem_ld_wait();
    tc_fence_before();
    if (splits > 1) {
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // every CTA of the cluster runs
      const int local = et - owner * chunk;  // column within the owner's chunk
      if (!mine) {
        // slot of this rank among the owner's senders: ranks in order, the owner itself left out
        const uint32_t slot = rank < uint32_t(owner) ? rank : rank - 1u;
        const uint32_t base = cluster_addr(smem_u32(recv_ptr), uint32_t(owner));
#pragma unroll
        for (int g = 0; g < kDecRows / 4; ++g) {
          if (g < groups) {
            const uint32_t dst = base + (((slot * (kDecRows / 4) + uint32_t(g)) * uint32_t(chunk) + uint32_t(local)) << 4);
            asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(v[4 * g]),
                         "r"(v[4 * g + 1]), "r"(v[4 * g + 2]), "r"(v[4 * g + 3])
                         : "memory");
          }
        }
        asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(
                         cluster_addr(smem_u32(&ring->red_full), uint32_t(owner)))
                     : "memory");
      } else {
        ok = ok && dec_wait_cluster(&ring->red_full, 0u, ring, p.status);
        const float4* red = reinterpret_cast<const float4*>(recv_ptr);
        float acc[kDecRows];
#pragma unroll
        for (int j = 0; j < kDecRows; ++j) acc[j] = 0.0f;
        bool first = true;
        for (int r = 0; r < splits; ++r) {  // rank order; this rank's own partial comes from its registers
          const int slot = r < int(rank) ? r : r - 1;
#pragma unroll
          for (int g = 0; g < kDecRows / 4; ++g) {
            if (g < groups) {
              float4 x;
              if (r == int(rank))
                x = make_float4(__uint_as_float(v[4 * g]), __uint_as_float(v[4 * g + 1]), __uint_as_float(v[4 * g + 2]),
                                __uint_as_float(v[4 * g + 3]));
              else
                x = red[(size_t(slot) * (kDecRows / 4) + g) * chunk + local];
              if (first) {
                acc[4 * g] = x.x, acc[4 * g + 1] = x.y, acc[4 * g + 2] = x.z, acc[4 * g + 3] = x.w;
              } else {
                acc[4 * g] = __fadd_rn(acc[4 * g], x.x), acc[4 * g + 1] = __fadd_rn(acc[4 * g + 1], x.y);
                acc[4 * g + 2] = __fadd_rn(acc[4 * g + 2], x.z), acc[4 * g + 3] = __fadd_rn(acc[4 * g + 3], x.w);
              }
            }
          }
          first = false;
        }
#pragma unroll
        for (int j = 0; j < kDecRows; ++j) v[j] = __float_as_uint(acc[j]);
      }
    }
    if (mine && ok && n < p.N) {
#pragma unroll
      for (int j = 0; j < kDecRows; ++j) {
        if (j < p.M) {
          const size_t off = size_t(j) * p.ldc + n;
          float y = sc * __uint_as_float(v[j]);
          if (p.out_kind == GRANITE4_GEMM_OUT_F32) {
            p.out_f32[off] = y;
          } else {
            if (p.out_kind == GRANITE4_GEMM_OUT_RESIDUAL) y = __fadd_rn(bf16_to_f32(resid[j]), __fmul_rn(p.resid_scale, y));
            p.out_bf16[off] = uint16_t(f32_to_bf16_bits(y));
          }
        }
      }
    }
  }

  // A CTA leaves when its own part is done: senders have nothing more to receive (a rank that owns
  // no columns gets no stores), owners have seen every arrival on red_full.
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (ring->abort) {  // give copies and MMAs already issued a bounded time to land
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000) {
    }
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<false>(tmem_base, kDecTmemCols);
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


bool box3d_enabled() {
  const char* v = std::getenv("G4_GEMM_BOX3D");
  return !(v != nullptr && v[0] == '0');
}

bool stream_enabled() {
  const char* v = std::getenv("G4_GEMM_STREAM");  // G4_GEMM_STREAM=0: at most 128 rows take the tiled forms
  return !(v != nullptr && v[0] == '0');
}

bool pair_enabled() {
  const char* v = std::getenv("G4_GEMM_PAIR");  // read per call: tests compare the two forms
  return !(v != nullptr && v[0] == '0');
}

// The dynamic shared memory opt-in of one form, once per device (function attributes are per
// device); the error of that call.
template <class C>
cudaError_t smem_opt_in() {
  static std::mutex mu;
  static std::map<int, cudaError_t> done;
  int dev = 0;
  if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  const auto it = done.find(dev);
  if (it != done.end()) return it->second;
  const cudaError_t err =
      cudaFuncSetAttribute(gemm_fp8_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(C::kSmemBytes));
  done[dev] = err;
  return err;
}

cudaLaunchConfig_t pair_config(int clusters) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2u * unsigned(clusters));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = CfgPair::kSmemBytes;
  return cfg;
}

// How many two-CTA clusters of the pair kernel the current device runs at once (0: none, or the
// query failed); asked once per device.
int pair_clusters() {
  static std::mutex mu;
  static std::map<int, int> known;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  std::lock_guard<std::mutex> lock(mu);
  const auto it = known.find(dev);
  if (it != known.end()) return it->second;
  int fit = 0;
  if (smem_opt_in<CfgPair>() == cudaSuccess) {
    cudaLaunchConfig_t cfg = pair_config(sm_count() / 2);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaOccupancyMaxActiveClusters(&fit, gemm_fp8_kernel<CfgPair>, &cfg) != cudaSuccess) fit = 0;
  }
  (void)cudaGetLastError();
  known[dev] = fit;
  return fit;
}

// Split of K for at most 16 rows of A. With T = ceil(N / 256) tiles and S slices of K there are
// T * S units for `sms` persistent CTAs; the busiest CTA gets ceil(T S / sms) of them. The plan is
// the smallest S whose units keep the SMs at least 85 % busy, else the S that keeps them busiest;
// slices are whole 128-byte blocks of K, at least 4 of them. rows: rows of the partials kept (16
// or 128). Depends on the shape and the SM count only, so the workspace query and the launch agree.
struct SplitPlan {
  int splits, kb_per, rows;
  size_t counter_bytes, bytes;
};
SplitPlan plan_split(int M, int N, int K, int sms) {
  SplitPlan pl{1, (K + kBK - 1) / kBK, M <= 16 ? 16 : kBM, 0, 0};
  if (M > 16 || sms <= 0) return pl;  // the last unit of a tile adds the partials alone: worth it for few rows only
  const int tiles = (N + kBN - 1) / kBN, kblocks = pl.kb_per;
  double best = 0.0;
  for (int s = 1; s <= kMaxSplits && (s == 1 || kblocks / s >= 4); ++s) {
    const int per = (kblocks + s - 1) / s, real = (kblocks + per - 1) / per;
    const long long units = 1ll * tiles * real;
    const double busy = double(units) / double(((units + sms - 1) / sms) * sms);
    if (busy > best + 1e-9) best = busy, pl.splits = real, pl.kb_per = per;
    if (busy >= 0.85) break;
  }
  if (pl.splits > 1) {
    pl.counter_bytes = (size_t(tiles) * sizeof(unsigned int) + 255) / 256 * 256;
    pl.bytes = pl.counter_bytes + size_t(tiles) * pl.splits * pl.rows * kBN * sizeof(float);
  }
  return pl;
}

// Tile width and ring shape of the stream form. A round of tiles over `sms` CTAs costs what its
// slowest resource costs: the MMA thread (4 MMAs per k-block at ~max(46, bn / 2) cycles) or the SM's
// share of HBM (bn x K bytes at ~44 bytes per ns); the plan is the width with the cheapest total.
// Ties go to the wider tile (fewer A blocks and loader steps per weight byte).
struct StreamPlan {
  int bn, kc, stages;
};
StreamPlan plan_stream(int N, int K, int a_rows, int sms) {
  const int kblocks = (K + kBK - 1) / kBK;
  double best = 1e300;
  StreamPlan pl{kBN, 1, 4};
  for (int bn = 32; bn <= kBN; bn += 16) {
    const int tiles = (N + bn - 1) / bn, rounds = (tiles + sms - 1) / sms;
    const double mma_ns = 4.0 * kblocks * (bn / 2 > 46 ? bn / 2 : 46) / 1.85;
    const double hbm_ns = double(bn) * K / 44.0;
    const double cost = rounds * (mma_ns > hbm_ns ? mma_ns : hbm_ns) + 500.0 * rounds;
    if (cost <= best * 1.0001) best = cost, pl.bn = bn;
  }
  const int blk = (a_rows + pl.bn) * kBK;  // bytes of one k-block of a stage
  pl.kc = 48 * 1024 / blk;
  pl.kc = pl.kc < 1 ? 1 : (pl.kc > 8 ? 8 : pl.kc);
  if (pl.kc > kblocks) pl.kc = kblocks;
  pl.stages = int(kStreamTileBytes / (size_t(pl.kc) * blk));
  if (pl.stages > kStreamMaxStages) pl.stages = kStreamMaxStages;
  return pl;
}

// The same matrix as {128 bytes, rows, K / 128 k-blocks} with a box of kc k-blocks (K % 128 == 0).
bool make_map3d(CUtensorMap* map, const void* base, int rows, int K, long long ld, int box_rows, int kc) {
  EncodeTiledFn enc = encode_tiled();
  if (enc == nullptr) return false;
  const cuuint64_t dims[3] = {cuuint64_t(kBK), cuuint64_t(rows), cuuint64_t(K / kBK)};
  const cuuint64_t strides[2] = {cuuint64_t(ld), cuuint64_t(kBK)};
  const cuuint32_t box[3] = {cuuint32_t(kBK), cuuint32_t(box_rows), cuuint32_t(kc)};
  const cuuint32_t elem[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_stream(const char* fn, const uint8_t* d_a, long long lda, const uint8_t* d_w, GemmParams p) {
  p.a_rows = p.M <= 16 ? 16 : kBM;
  const StreamPlan pl = plan_stream(p.N, p.K, p.a_rows, sm_count());
  p.bn = pl.bn, p.kc = pl.kc, p.stages = pl.stages;
  CUtensorMap map_a, map_w;
  p.box3d = p.K % kBK == 0 && p.kc > 1 && box3d_enabled() && make_map3d(&map_a, d_a, p.M, p.K, lda, p.a_rows, p.kc) &&
            make_map3d(&map_w, d_w, p.N, p.K, p.K, p.bn, p.kc);
  if (!p.box3d && (!make_map(&map_a, d_a, p.M, p.K, lda, p.a_rows) || !make_map(&map_w, d_w, p.N, p.K, p.K, p.bn)))
    return fail(fn, "the tensor map could not be encoded");
  static std::mutex mu;
  static std::map<int, cudaError_t> done;
  int dev = 0;
  G4_CUDA_TRY(fn, cudaGetDevice(&dev));
  {
    std::lock_guard<std::mutex> lock(mu);
    if (done.find(dev) == done.end())
      done[dev] = cudaFuncSetAttribute(gemm_fp8_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       int(kStreamSmemBytes));
    G4_CUDA_TRY(fn, done[dev]);
  }
  const int tiles = (p.N + p.bn - 1) / p.bn;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  G4_LAUNCH_PDL(fn, gemm_fp8_stream_kernel, dim3(grid), dim3(kThreads), kStreamSmemBytes, current_stream(), map_a,
                map_w, p);
  return 0;
}

bool decode_form_enabled() {
  const char* v = std::getenv("G4_GEMM_DECODE");  // G4_GEMM_DECODE=0: at most 16 rows take the older forms
  return !(v != nullptr && v[0] == '0');
}

// Slices of K for the 16-row form. A unit costs about 4 us whatever its size (first bytes from HBM,
// the hand-over of the partial sums, the epilogue), and a CTA with a 90 KB ring streams ~45 B/ns, so
// few large units are better than many small ones as long as every SM has one: measured at one row,
// tiles x slices of about 1.3 per SM is the best plan for all five projection shapes of the model
// (1 slice for the gate|up and lm_head shapes, 4 for QKV, 6 for O and down; clusters of 7 or 8 lose
// to the scheduling of large clusters what they gain in balance). At least four k-blocks per slice.
// G4_GEMM_DECODE_SPLITS forces a count (measurements).
struct DecodePlan {
  int splits, kb_per;
};
DecodePlan plan_decode(int N, int K, int sms) {
  const int tiles = (N + kBM - 1) / kBM, kblocks = (K + kBK - 1) / kBK;
  int s = (13 * (sms > 0 ? sms : 1) / 10 + tiles - 1) / tiles;
  if (s > 6) s = 6;
  if (const char* v = std::getenv("G4_GEMM_DECODE_SPLITS"); v != nullptr && std::atoi(v) > 0) s = std::atoi(v);
  if (s > kblocks / 4) s = kblocks / 4;
  if (s > kDecMaxSplits) s = kDecMaxSplits;
  if (s < 1) s = 1;
  const int per = (kblocks + s - 1) / s;
  return DecodePlan{(kblocks + per - 1) / per, per};
}

// Launches the 16-row form; 1 when the device cannot co-schedule a cluster of the planned size (the
// caller then takes another form), 0 launched, -1 failed.
int launch_decode(const char* fn, const uint8_t* d_a, long long lda, const uint8_t* d_w, GemmParams p) {
  const DecodePlan pl = plan_decode(p.N, p.K, sm_count());
  p.splits = pl.splits, p.kb_per = pl.kb_per;
  static std::mutex mu;
  static std::map<int, cudaError_t> done;
  static std::map<std::pair<int, int>, bool> fits;
  int dev = 0;
  G4_CUDA_TRY(fn, cudaGetDevice(&dev));
  const int tiles = (p.N + kBM - 1) / kBM;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(tiles) * unsigned(p.splits));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kDecSmemBytes;
  cfg.stream = current_stream();
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = unsigned(p.splits), attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (done.find(dev) == done.end())
      done[dev] = cudaFuncSetAttribute(gemm_fp8_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       int(kDecSmemBytes));
    G4_CUDA_TRY(fn, done[dev]);
    const auto key = std::make_pair(dev, p.splits);
    if (fits.find(key) == fits.end()) {
      int n = 0;
      cfg.numAttrs = 1;
      fits[key] = cudaOccupancyMaxActiveClusters(&n, gemm_fp8_decode_kernel, &cfg) == cudaSuccess && n >= 1;
      (void)cudaGetLastError();
    }
    if (!fits[key]) return 1;
  }
  CUtensorMap map_a, map_w;
  if (!make_map(&map_a, d_a, p.M, p.K, lda, kDecRows) || !make_map(&map_w, d_w, p.N, p.K, p.K, kBM))
    return fail(fn, "the tensor map could not be encoded");
  cfg.numAttrs = pdl_enabled() ? 2u : 1u;
  G4_CUDA_TRY(fn, cudaLaunchKernelEx(&cfg, gemm_fp8_decode_kernel, map_a, map_w, p));
  return 0;
}

// Encodes the two tensor maps of form C and launches it over min(units, SMs) CTAs (CTA pairs).
template <class C>
int launch(const char* fn, const uint8_t* d_a, long long lda, const uint8_t* d_w, const GemmParams& p) {
  constexpr bool kPair = C::kTileM == 2 * kBM;
  CUtensorMap map_a, map_w;
  // the fused SwiGLU fetches a single CTA's 256 W rows as two boxes of 128 (gate rows, up rows)
  const int w_box = (p.swiglu_i && !kPair) ? kBN / 2 : C::kWRows;
  if (!make_map(&map_a, d_a, p.M, p.K, lda, C::kARows) || !make_map(&map_w, d_w, p.N, p.K, p.K, w_box))
    return fail(fn, "the tensor map could not be encoded");
  G4_CUDA_TRY(fn, smem_opt_in<C>());
  const int nt = p.swiglu_i ? (p.swiglu_i + kBN / 2 - 1) / (kBN / 2) : (p.N + kBN - 1) / kBN;
  const int units = ((p.M + C::kTileM - 1) / C::kTileM) * nt * p.splits;
  if constexpr (kPair) {
    const int clusters = units < pair_clusters() ? units : pair_clusters();
    cudaLaunchConfig_t cfg = pair_config(clusters);
    cfg.stream = current_stream();
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2u : 1u;
    G4_CUDA_TRY(fn, cudaLaunchKernelEx(&cfg, gemm_fp8_kernel<C>, map_a, map_w, p));
  } else {
    const int grid = units < sm_count() ? units : sm_count();
    G4_LAUNCH_PDL(fn, gemm_fp8_kernel<C>, dim3(grid), dim3(kThreads), C::kSmemBytes, current_stream(), map_a, map_w, p);
  }
  return 0;
}

}  // namespace

extern "C" long long granite4_gemm_fp8_workspace_bytes(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M <= kDecRows && decode_form_enabled()) return 0;  // partial sums go through a cluster's shared memory
  if (M > 2 && stream_enabled()) return 0;  // the stream form needs none
  return static_cast<long long>(plan_split(M, N, K, sm_count()).bytes);
}

extern "C" int granite4_kernel_gemm_fp8(int out_kind, const uint8_t* d_a, long long lda, const uint8_t* d_w, int M,
                                        int N, int K, const granite4_gemm_fp8_epilogue* ep, void* d_ws,
                                        long long ws_bytes) {
  static const char* fn = "granite4_kernel_gemm_fp8";
  // M == 0 (an empty shard) is valid: every check below still applies, then nothing is launched
  if (ep == nullptr || d_w == nullptr || (d_a == nullptr && M != 0)) return fail(fn, "null argument");
  if (M < 0 || N <= 0 || K <= 0 || K % 16 != 0 || lda < K || lda % 16 != 0 || !aligned16(d_a) || !aligned16(d_w))
    return fail(fn, "needs K % 16 == 0, lda % 16 == 0, lda >= K and 16-byte aligned A and W");
  if (out_kind != GRANITE4_GEMM_OUT_BF16 && out_kind != GRANITE4_GEMM_OUT_F32 && out_kind != GRANITE4_GEMM_OUT_RESIDUAL &&
      out_kind != GRANITE4_GEMM_OUT_SWIGLU)
    return fail(fn, "unknown output kind");
  const bool fused_swiglu = out_kind == GRANITE4_GEMM_OUT_SWIGLU;
  if (fused_swiglu && (N % 2 != 0 || ep->d_out_scale_amax == nullptr))
    return fail(fn, "the fused SwiGLU needs an even N (gate rows, then up rows) and d_out_scale_amax");
  if (ep->ldc < (fused_swiglu ? N / 2 : N)) return fail(fn, "ldc smaller than the output row");
  // (with no rows there is nothing to read or write: A, the output and the residual may be null)
  if (M != 0 && (out_kind == GRANITE4_GEMM_OUT_F32 ? ep->d_out_f32 == nullptr : ep->d_out_bf16 == nullptr))
    return fail(fn, "the output of the requested kind is null");
  if (M != 0 && out_kind == GRANITE4_GEMM_OUT_RESIDUAL && ep->d_residual == nullptr) return fail(fn, "null residual");
  if (d_ws != nullptr && !aligned16(d_ws)) return fail(fn, "the workspace must be 16-byte aligned");
  if (M == 0) {
    // no rows: the only effect is on the fused epilogue's {scale, amax} slot, which must not keep a
    // previous call's maximum for the encode step (or a GEMM reading the scale) that follows
    if (fused_swiglu && !amax_prezeroed())
      G4_CUDA_TRY(fn, cudaMemsetAsync(ep->d_out_scale_amax, 0, 2 * sizeof(float), current_stream()));
    return 0;
  }

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
  p.splits = 1, p.kb_per = (K + kBK - 1) / kBK;
  if (fused_swiglu) {
    p.swiglu_i = N / 2, p.amax_slot = ep->d_out_scale_amax;
    if (!amax_prezeroed()) G4_CUDA_TRY(fn, cudaMemsetAsync(p.amax_slot, 0, 2 * sizeof(float), current_stream()));
    if (M <= kBM) return launch<CfgWide>(fn, d_a, lda, d_w, p);  // no split of K under this epilogue
  }
  if (M <= kDecRows && decode_form_enabled()) {
    const int rc = launch_decode(fn, d_a, lda, d_w, p);
    if (rc <= 0) return rc;
  }
  if (M <= kBM) {
    // A stream of the weights. Measured per layer of four projections (one CUDA graph): the split of
    // K through the workspace wins at one and two rows (63 us against 70), the full-K stream form
    // from three rows on (70 us flat up to 16 rows against 74 - 126; 100 - 109 us for 32 - 128 rows
    // against 121 - 128).
    const SplitPlan pl = plan_split(M, N, K, sm_count());
    const bool can_split = pl.splits > 1 && d_ws != nullptr && ws_bytes >= static_cast<long long>(pl.bytes);
    if (stream_enabled() && !(M <= 2 && can_split)) return launch_stream(fn, d_a, lda, d_w, p);
    p.early = 1;
    if (can_split) {
      p.splits = pl.splits, p.kb_per = pl.kb_per, p.ws_rows = pl.rows;
      p.counters = static_cast<unsigned int*>(d_ws);
      p.ws = reinterpret_cast<float*>(static_cast<char*>(d_ws) + pl.counter_bytes);
    }
    return M <= 16 ? launch<CfgSkinny>(fn, d_a, lda, d_w, p) : launch<CfgWide>(fn, d_a, lda, d_w, p);
  }
  // 256-row tiles on CTA pairs where the device co-schedules two-CTA clusters of this size
  // (G4_GEMM_PAIR=0 keeps the single form)
  if (pair_enabled() && pair_clusters() > 0) return launch<CfgPair>(fn, d_a, lda, d_w, p);
  return launch<CfgWide>(fn, d_a, lda, d_w, p);
}
