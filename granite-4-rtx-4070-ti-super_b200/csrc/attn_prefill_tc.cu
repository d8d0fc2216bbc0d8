// Causal attention of a prefill chunk over the int8 paged pool on the 5th-generation tensor
// cores (tcgen05 + tensor memory): the large-chunk form of granite4_prefill_attention_int8.
//
// Contract: the reference's prefill_attention with the int8 cache (engine/src/prefill_gemm.h:86-101,
// kernel engine/src/prefill_gemm.cu:1018-1189): query rows at positions [base_pos, base_pos + rows)
// of ONE sequence attend to cache positions [0, position]; Hq = 4 Hk, d = 128
// (engine/src/attention_gpu.h:18-19).
//
// A CTA owns 64 consecutive query positions of one kv head as TWO row tiles of 128 MMA rows
// (32 positions x the 4 query heads of the group), and walks the cache in tiles of 64 positions.
// Both contractions of a tile are tcgen05.mma instructions with f16 operands and f32 accumulators
// in tensor memory:
//   S_t = Q_t K^T   M 128, N 64, K 128   (8 instructions of K 16; Q and K from shared memory),
//                   two S buffers per row tile
//   O_t += P_t V    M 128, N 128, K 64   (4 instructions; P from TENSOR MEMORY, where the softmax
//                   wrote it over the S buffer it came from; V from shared memory as an N-major
//                   operand)
// so that one K / V tile, converted from int8 ONCE, serves 256 query rows.
//
// Roles by warp (14 warps; every hand-over is an mbarrier, every wait on one is bounded):
//   warp 0      producer: looks the tile's 64 positions up in the page table and fetches their raw
//               K and V code rows with bulk asynchronous copies (TMA engine, cp.async.bulk into this
//               CTA's own shared memory, no multicast; one 2 KB copy per 16-token page where the
//               rows are consecutive, else 128 bytes per row) and their scales with 4-byte
//               cp.async, into a three-stage ring;
//   warp 1      allocates the tensor memory; one thread issues every MMA and commits them to the
//               barriers of whoever waits for the result: per tile, first S of the NEXT tile for both
//               row tiles (into the S buffer that tile j - 1 used), then P V of this tile for each
//               row tile as soon as its P is written. The tensor cores thus work on tile j + 1's
//               logits while the softmax of tile j runs; an S overwrites the buffer a P V of two
//               tiles ago read, and MMAs execute in issue order, so no barrier is needed between them;
//   warps 4-7   softmax of row tile 0, warps 8-11 of row tile 1: a thread owns one row (its
//               tensor-memory lane): reads its 64 logits (tcgen05.ld), applies the column factor
//               (K scale x softmax scale) and the causal mask, keeps the running maximum and sum,
//               and writes the probabilities as f16 pairs back over the logits (tcgen05.st). The
//               accumulator O is rescaled in tensor memory only when a tile's maximum exceeds the
//               running one by more than 2^12 (the final division uses the same maximum, so the
//               result does not depend on when the rescale happens), and only then does a tile
//               wait for the previous P V;
//   warps 2-3, 12-13  converters: int8 codes -> f16, written as 128-byte-swizzled tiles
//               ([position][64 dims] twice), three buffers: K as the exact codes, K-major for
//               S = Q K^T; V as code x scale and, the same byte layout, N-major for P V.
// The K scale multiplies the logit in f32, so K's operand holds the codes exactly; Q is scaled by
// one power of two per CTA into f16's range. Arithmetic against the reference's golden pipeline
// (engine/src/kernel_math.h:265-331): logits and the softmax in f32, probabilities and V rounded to
// f16 (bf16 there) - inside the reference's own 0.03 bar (engine/tests/test_kernels.cu:2055).
//
// Work: 4 d Hq n^2 / 2 flops for a chunk of n rows from position 0; the chunk's K / V stay in L2.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <climits>
#include <cmath>
#include <cstdint>
#include <cstdlib>

#include "g4_host.h"
#include "g4_math.cuh"
#include "g4_tcgen05.cuh"
#include "g4_tma.cuh"

namespace g4 {
namespace {

constexpr int kD = 128;      // head dim
constexpr int kQPos = 32;    // query positions per row tile (x 4 heads = 128 MMA rows)
constexpr int kRowTiles = 2;
constexpr int kCtaPos = kQPos * kRowTiles;  // 64 query positions per CTA
constexpr int kTN = 64;      // cache positions per tile
constexpr int kThreads = 448;  // 14 warps: four on two of the SM's sub-partitions, so 128 registers per thread
constexpr int kBufs = 3;  // converted K / V buffers
constexpr int kRaw = 3;   // raw stages

constexpr uint32_t kQTileBytes = 128 * kD * 2;     // 32768: two 64-dim halves of [128 rows][128 bytes]
constexpr uint32_t kKvTileBytes = kTN * kD * 2;    // 16384: two 64-dim halves of [64 positions][128 bytes]
constexpr uint32_t kPTileBytes = 128 * kTN * 2;    // 16384: [128 rows][128 bytes]
constexpr uint32_t kRawBytes = kTN * kD;           // 8192 per matrix and stage

struct TcSmem {
  // swizzled operand tiles first: each sits on a 1024-byte boundary
  uint8_t q16[kRowTiles][kQTileBytes];
  uint8_t k16[kBufs][kKvTileBytes];
  uint8_t v16[kBufs][kKvTileBytes];
  uint8_t raw_k[kRaw][kRawBytes];
  uint8_t raw_v[kRaw][kRawBytes];
  float raw_ks[kRaw][kTN], raw_vs[kRaw][kTN];  // scales of the raw stages
  float cs[kBufs][kTN];  // per converted K tile: K scale x softmax scale x log2(e) x the power of two taken out of Q
  uint64_t raw_full[kRaw], raw_empty[kRaw], kv_full[kBufs], kv_empty[kBufs];
  uint64_t s_full[kRowTiles][2], p_full[kRowTiles][2], pv_done[kRowTiles][2];
  uint64_t q_ready;
  uint32_t q_amax;  // max |q| over the CTA's rows, as float bits
  uint32_t tmem_base;
  int abort;
};
constexpr size_t kTcSmemBytes = sizeof(TcSmem) + 1024;
static_assert(kTcSmemBytes <= 227 * 1024, "shared memory of the tensor-core prefill attention");

struct TcParams {
  const uint16_t* q;
  const int8_t* ck;
  const int8_t* cv;
  const float* ks;
  const float* vs;
  const int* pt;
  uint16_t* out;
  unsigned int* status;
  int rows, base_pos, Hq, Hk;
  long long stride;
  float scale_log2;
};

// tensor-memory columns: S[t][buffer] 64 each, then O[t] 128 each
constexpr uint32_t kTmemCols = 512;
__device__ __forceinline__ uint32_t s_col(int t, int sb) { return uint32_t((t * 2 + sb) * kTN); }
__device__ __forceinline__ uint32_t o_col(int t) { return uint32_t(256 + t * kD); }

// Instruction descriptors (kind::f16): f32 accumulator, f16 x f16, M 128.
constexpr uint32_t kIdescS = (1u << 4) | (uint32_t(kTN >> 3) << 17) | (uint32_t(128 >> 4) << 24);             // N 64, both K-major
constexpr uint32_t kIdescPV = (1u << 4) | (1u << 16) | (uint32_t(kD >> 3) << 17) | (uint32_t(128 >> 4) << 24);  // N 128, B N-major

// P V with P in tensor memory: D (+)= A (tensor memory: lane = row, a 32-bit column = two
// consecutive f16 along K) x B (shared memory).
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Four MMAs of one accumulator in one statement: D (+)= A0 B0 + A1 B1 + A2 B2 + A3 B3; `accumulate` = 0
// makes the first of them overwrite D.
__device__ __forceinline__ void mma4_ss(uint32_t d_tmem, uint64_t a0, uint64_t b0, uint64_t a1, uint64_t b1, uint64_t a2,
                                        uint64_t b2, uint64_t a3, uint64_t b3, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %10, 0;\n\t"
      "setp.eq.b32 q, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %9, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %4, %9, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %6, %9, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %8, %9, q;\n\t}" ::"r"(d_tmem),
      "l"(a0), "l"(b0), "l"(a1), "l"(b1), "l"(a2), "l"(b2), "l"(a3), "l"(b3), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same with A in tensor memory: k-step i reads the 8 columns from a_tmem + 8 i.
__device__ __forceinline__ void mma4_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b0, uint64_t b1, uint64_t b2, uint64_t b3,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b32 a1, a2, a3;\n\t"
      "setp.ne.b32 p, %7, 0;\n\t"
      "setp.eq.b32 q, 0, 0;\n\t"
      "add.u32 a1, %1, 8;\n\tadd.u32 a2, %1, 16;\n\tadd.u32 a3, %1, 24;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %6, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], %3, %6, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], %4, %6, q;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], %5, %6, q;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b0), "l"(b1), "l"(b2), "l"(b3), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A shared-memory descriptor from its two words (g4_tcgen05.cuh smem_desc_sw128): the low one holds the
// address and the leading byte offset, both in 16-byte units, the high one is the same for every
// tile here (8-row groups 1024 bytes apart, version 1, 128-byte swizzle).
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint64_t desc_of(uint32_t lo) { return (uint64_t(kDescHi) << 32) | lo; }

__device__ __forceinline__ bool wait_tc(uint64_t* bar, uint32_t parity, TcSmem* sm, unsigned int* status) {
  volatile int* ab = &sm->abort;
  for (uint32_t i = 0; i < kMbarWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*ab) return false;
    if (i > 256) __nanosleep(32);
  }
  *ab = 1;
  if (status != nullptr) atomicOr(status, kStatusAttnWaitTimeout);
  return false;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
// One arrival on `bar` once this thread's earlier cp.async copies have landed (the arrival is part of
// the barrier's expected count).
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Byte offset of 16-byte chunk `chunk` (0..7) of 128-byte row `row` in a 128-byte-swizzled tile.
__device__ __forceinline__ uint32_t sw128(int row, int chunk) { return uint32_t(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// Sixteen int8 codes -> sixteen exact f16 values, as two 16-byte chunks.
__device__ __forceinline__ void codes16_to_half(const uint4 w, uint4& lo, uint4& hi) {
  const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
  auto four = [&](uint32_t x, uint32_t& a, uint32_t& b) {
    x ^= 0x80808080u;  // code + 128 in every byte; 0x6400 | byte is the f16 value 1024 + byte
    __half2 h0, h1;
    *reinterpret_cast<uint32_t*>(&h0) = __byte_perm(x, 0x64646464u, 0x4140);
    *reinterpret_cast<uint32_t*>(&h1) = __byte_perm(x, 0x64646464u, 0x4342);
    h0 = __hsub2(h0, bias), h1 = __hsub2(h1, bias);  // exact
    a = *reinterpret_cast<uint32_t*>(&h0), b = *reinterpret_cast<uint32_t*>(&h1);
  };
  four(w.x, lo.x, lo.y), four(w.y, lo.z, lo.w), four(w.z, hi.x, hi.y), four(w.w, hi.z, hi.w);
}

__device__ __forceinline__ void mul8(uint4& v, __half2 f) {
  __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __hmul2(h[i], f);
}

// The CTA's Q rows are scaled by 2^-e, e = exponent(max |q|) - 10, so that they sit in f16's range
// whatever their magnitude (bf16 reaches 3e38); 2^e goes into the logit factor.
__device__ __forceinline__ int q_exponent(uint32_t amax_bits) {
  const float a = __uint_as_float(amax_bits);
  if (!(a > 0.0f) || !(a < INFINITY)) return 0;
  return min(max(static_cast<int>((amax_bits >> 23) & 0xffu) - 127 - 10, -100), 100);
}
__device__ __forceinline__ float q_down_factor(uint32_t amax_bits) { return __int_as_float((127 - q_exponent(amax_bits)) << 23); }
__device__ __forceinline__ float q_up_factor(uint32_t amax_bits) { return __int_as_float((127 + q_exponent(amax_bits)) << 23); }

__global__ void __launch_bounds__(kThreads, 1) attn_prefill_tc_kernel(const TcParams p) {
  pdl_begin();
  extern __shared__ uint8_t smem_raw[];
  TcSmem* sm = reinterpret_cast<TcSmem*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hkv = blockIdx.y;
  // the longest prefixes first
  const int blk = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int row0 = blk * kCtaPos;                           // first chunk row of this CTA
  const int nrows = min(kCtaPos, p.rows - row0);            // its live rows
  const int kv_end = p.base_pos + row0 + nrows;             // cache positions [0, kv_end) are needed
  const int n_kv = (kv_end + kTN - 1) / kTN;
  const size_t head_row0 = static_cast<size_t>(hkv) * p.stride;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kRaw; ++i) {
      mbar_init(&sm->raw_full[i], 1 + 32);  // the arming arrival + one per producer lane (its scale copies)
      mbar_init(&sm->raw_empty[i], 4);
    }
    for (int i = 0; i < kBufs; ++i) {
      mbar_init(&sm->kv_full[i], 4);
      mbar_init(&sm->kv_empty[i], 1);
    }
    for (int t = 0; t < kRowTiles; ++t) {
      // one barrier of each kind per S buffer: the warps of a row tile may be a tile apart, never two
      for (int i = 0; i < 2; ++i)
        mbar_init(&sm->s_full[t][i], 1), mbar_init(&sm->pv_done[t][i], 1), mbar_init(&sm->p_full[t][i], 4);
    }
    mbar_init(&sm->q_ready, 8);
    sm->abort = 0;
    sm->q_amax = 0u;
    mbar_init_fence();
    fence_async_smem();
  }
  if (warp == 1) tmem_alloc<false>(smem_u32(&sm->tmem_base), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sm->tmem_base;

  if (warp == 0) {
    // ---- producer ---------------------------------------------------------------------------
    // lane l fetches positions l and l + 32 of every tile
    auto rows_of = [&](int j, int& a, int& b) {
      const int pa = min(j * kTN + lane, kv_end - 1), pb = min(j * kTN + 32 + lane, kv_end - 1);  // past the end: a row that is masked anyway
      a = p.pt != nullptr ? __ldg(p.pt + pa) : pa;
      b = p.pt != nullptr ? __ldg(p.pt + pb) : pb;
      a = min(max(a, 0), static_cast<int>(p.stride) - 1), b = min(max(b, 0), static_cast<int>(p.stride) - 1);
    };
    int ra, rb, na = 0, nb = 0;  // this tile's rows and the next tile's: a table entry is read two tiles ahead
    rows_of(0, ra, rb);
    if (n_kv > 1) rows_of(1, na, nb);
    for (int j = 0; j < n_kv; ++j) {
      const int s = j % kRaw;
      if (!wait_tc(&sm->raw_empty[s], ((j / kRaw) & 1) ^ 1, sm, p.status)) break;
      if (lane == 0) mbar_arrive_expect_tx(&sm->raw_full[s], 2u * kRawBytes);
      __syncwarp();
      // A group of 16 consecutive positions usually is one page of the pool, i.e. 16 consecutive pool
      // rows: one 2 KB copy per matrix then replaces 16 copies of 128 bytes (the copy engine takes a
      // few dozen cycles per request whatever its size). Lanes 0-15 / 16-31 hold groups 0 / 1 in ra and
      // groups 2 / 3 in rb.
      const int first_a = __shfl_sync(0xffffffffu, ra, lane & 16), first_b = __shfl_sync(0xffffffffu, rb, lane & 16);
      const unsigned run_a = __ballot_sync(0xffffffffu, ra == first_a + (lane & 15));
      const unsigned run_b = __ballot_sync(0xffffffffu, rb == first_b + (lane & 15));
      const unsigned mine = 0xffffu << (lane & 16);
      const bool page_a = (run_a & mine) == mine, page_b = (run_b & mine) == mine;
      const size_t oa = (head_row0 + ra) * kD, ob = (head_row0 + rb) * kD;
      if (page_a) {
        if ((lane & 15) == 0) {
          bulk_load(sm->raw_k[s] + lane * kD, p.ck + oa, 16 * kD, &sm->raw_full[s]);
          bulk_load(sm->raw_v[s] + lane * kD, p.cv + oa, 16 * kD, &sm->raw_full[s]);
        }
      } else {
        bulk_load(sm->raw_k[s] + lane * kD, p.ck + oa, kD, &sm->raw_full[s]);
        bulk_load(sm->raw_v[s] + lane * kD, p.cv + oa, kD, &sm->raw_full[s]);
      }
      if (page_b) {
        if ((lane & 15) == 0) {
          bulk_load(sm->raw_k[s] + (32 + lane) * kD, p.ck + ob, 16 * kD, &sm->raw_full[s]);
          bulk_load(sm->raw_v[s] + (32 + lane) * kD, p.cv + ob, 16 * kD, &sm->raw_full[s]);
        }
      } else {
        bulk_load(sm->raw_k[s] + (32 + lane) * kD, p.ck + ob, kD, &sm->raw_full[s]);
        bulk_load(sm->raw_v[s] + (32 + lane) * kD, p.cv + ob, kD, &sm->raw_full[s]);
      }
      cp_async4(&sm->raw_ks[s][lane], p.ks + head_row0 + ra);
      cp_async4(&sm->raw_ks[s][32 + lane], p.ks + head_row0 + rb);
      cp_async4(&sm->raw_vs[s][lane], p.vs + head_row0 + ra);
      cp_async4(&sm->raw_vs[s][32 + lane], p.vs + head_row0 + rb);
      cp_async_arrive_noinc(&sm->raw_full[s]);
      ra = na, rb = nb;
      if (j + 2 < n_kv) rows_of(j + 2, na, nb);
    }
  } else if (warp == 1) {
    // ---- MMA issue ----------------------------------------------------------------------------
    // One thread issues every MMA; it is the busiest thread of the CTA (29 MMAs and commits per
    // tile), so its instruction count per MMA is kept at the minimum: the descriptors of Q are
    // formed once, those of a tile's K and V once per tile (both row tiles use them), and four MMAs
    // go out per asm statement.
    if (lane == 0) {
      bool ok = wait_tc(&sm->q_ready, 0, sm, p.status);
      const uint32_t q_lo = (smem_u32(sm->q16[0]) >> 4) | (1u << 16), k_lo = (smem_u32(sm->k16[0]) >> 4) | (1u << 16);
      const uint32_t v_lo = (smem_u32(sm->v16[0]) >> 4) | ((kKvTileBytes / 2 >> 4) << 16);  // 64-dim halves 8 KB apart
      uint64_t qd[kRowTiles][8];
#pragma unroll
      for (int t = 0; t < kRowTiles; ++t)
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // 16 dims = 32 bytes per instruction; dims 64.. in the second half tile
          qd[t][kk] = desc_of(q_lo + ((t * kQTileBytes + (kk >> 2) * (kQTileBytes / 2) + (kk & 3) * 32) >> 4));
      auto issue_s = [&](int j) {
        const int b = j % kBufs, sb = j & 1;
        if (!(ok = ok && wait_tc(&sm->kv_full[b], (j / kBufs) & 1, sm, p.status))) return;
        tc_fence_after();
        uint64_t kd[8];
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          kd[kk] = desc_of(k_lo + ((b * kKvTileBytes + (kk >> 2) * (kKvTileBytes / 2) + (kk & 3) * 32) >> 4));
#pragma unroll
        for (int t = 0; t < kRowTiles; ++t) {
          mma4_ss(tmem_base + s_col(t, sb), qd[t][0], kd[0], qd[t][1], kd[1], qd[t][2], kd[2], qd[t][3], kd[3], kIdescS, 0u);
          mma4_ss(tmem_base + s_col(t, sb), qd[t][4], kd[4], qd[t][5], kd[5], qd[t][6], kd[6], qd[t][7], kd[7], kIdescS, 1u);
          mma_commit<false>(smem_u32(&sm->s_full[t][sb]));
        }
      };
      if (ok) issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) issue_s(j + 1);
        const int b = j % kBufs, sb = j & 1;
        uint64_t vd[4];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)  // 16 positions per instruction: 8 columns of P, two 8-row groups of V
          vd[kk] = desc_of(v_lo + ((b * kKvTileBytes + kk * 2048) >> 4));
        for (int t = 0; t < kRowTiles && ok; ++t) {
          if (!(ok = wait_tc(&sm->p_full[t][sb], (j >> 1) & 1, sm, p.status))) break;
          tc_fence_after();
          mma4_ts(tmem_base + o_col(t), tmem_base + s_col(t, sb), vd[0], vd[1], vd[2], vd[3], kIdescPV, j > 0 ? 1u : 0u);
          mma_commit<false>(smem_u32(&sm->pv_done[t][sb]));
        }
        if (ok) mma_commit<false>(smem_u32(&sm->kv_empty[b]));
      }
    }
  } else if (warp < 4 || warp >= 12) {
    // ---- converters -----------------------------------------------------------------------------
    const int c = (warp < 4 ? warp - 2 : warp - 10) * 32 + lane;  // 0..127
    // the logit factor of a column: its K scale x (softmax scale x log2 e x 2^qexp); the last two are
    // known once the Q rows have been scaled
    bool okc = wait_tc(&sm->q_ready, 0, sm, p.status);
    const float col_scale = p.scale_log2 * q_up_factor(sm->q_amax);
    for (int j = 0; j < n_kv && okc; ++j) {
      const int s = j % kRaw, b = j % kBufs;
      if (!wait_tc(&sm->raw_full[s], (j / kRaw) & 1, sm, p.status)) break;
      if (!wait_tc(&sm->kv_empty[b], ((j / kBufs) & 1) ^ 1, sm, p.status)) break;
      // unit u = (row, piece of 16 codes): a quarter warp reads one whole raw row; its stores land in
      // eight different 16-byte columns (the lanes of the second half tile write their two chunks in
      // the other order)
      uint4 raw[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) raw[i] = *reinterpret_cast<const uint4*>(sm->raw_k[s] + (i * 128 + c) * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int u = i * 128 + c, row = u >> 3, piece = u & 7;
        const int half = piece >> 2, ch = (piece & 3) * 2, flip = half;
        uint4 lo, hi;
        codes16_to_half(raw[i], lo, hi);
        uint8_t* kt = sm->k16[b] + half * (kKvTileBytes / 2);
        *reinterpret_cast<uint4*>(kt + sw128(row, ch + flip)) = flip ? hi : lo;
        *reinterpret_cast<uint4*>(kt + sw128(row, ch + 1 - flip)) = flip ? lo : hi;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) raw[i] = *reinterpret_cast<const uint4*>(sm->raw_v[s] + (i * 128 + c) * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int u = i * 128 + c, row = u >> 3, piece = u & 7;
        const int half = piece >> 2, ch = (piece & 3) * 2, flip = half;
        uint4 lo, hi;
        codes16_to_half(raw[i], lo, hi);
        const __half2 sv = __float2half2_rn(sm->raw_vs[s][row]);  // V = code x scale, rounded to f16
        mul8(lo, sv), mul8(hi, sv);
        uint8_t* vt = sm->v16[b] + half * (kKvTileBytes / 2);
        *reinterpret_cast<uint4*>(vt + sw128(row, ch + flip)) = flip ? hi : lo;
        *reinterpret_cast<uint4*>(vt + sw128(row, ch + 1 - flip)) = flip ? lo : hi;
      }
      if (c < kTN) sm->cs[b][c] = sm->raw_ks[s][c] * col_scale;
      fence_async_smem();  // the tiles are read by the tensor cores (async proxy)
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&sm->kv_full[b]));
        mbar_arrive(smem_u32(&sm->raw_empty[s]));
      }
    }
  } else {
    // ---- softmax (warps 4-11): row tile t, tensor-memory lane = MMA row = (head hl, position pl) -----------------
    const int t = (warp - 4) >> 2, hl = warp & 3, pl = lane;
    const int r = hl * 32 + pl;                        // MMA row
    const int crow = row0 + t * kQPos + pl;            // row of the chunk
    const bool live = crow < p.rows;
    const int pos = live ? p.base_pos + crow : -1;
    const uint32_t lane_addr = tmem_base + (uint32_t(hl * 32) << 16);
    // Q rows -> f16, scaled by one power of two per CTA into f16's range, into the swizzled Q tile
    {
      const uint4* src = reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(live ? crow : 0) * p.Hq + hkv * 4 + hl) * kD);
      float qmax = 0.0f;
#pragma unroll 4
      for (int i = 0; i < 16; ++i) {
        float f[8];
        unpack8(live ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) qmax = fmaxf(qmax, fabsf(f[e]));
      }
      qmax = warp_max(qmax);
      if (lane == 0 && qmax < INFINITY) atomicMax(&sm->q_amax, __float_as_uint(qmax));  // non-negative floats order as integers
      asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight softmax warps
      const float down = q_down_factor(sm->q_amax);
#pragma unroll 4
      for (int i = 0; i < 16; ++i) {  // the row again (it is in L1 now)
        float f[8];
        unpack8(live ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u), f);
        uint4 h;
        __half2 h2;
        h2 = __floats2half2_rn(f[0] * down, f[1] * down), h.x = *reinterpret_cast<uint32_t*>(&h2);
        h2 = __floats2half2_rn(f[2] * down, f[3] * down), h.y = *reinterpret_cast<uint32_t*>(&h2);
        h2 = __floats2half2_rn(f[4] * down, f[5] * down), h.z = *reinterpret_cast<uint32_t*>(&h2);
        h2 = __floats2half2_rn(f[6] * down, f[7] * down), h.w = *reinterpret_cast<uint32_t*>(&h2);
        *reinterpret_cast<uint4*>(sm->q16[t] + (i >> 3) * (kQTileBytes / 2) + sw128(r, i & 7)) = h;
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm->q_ready));
    }
    const int pos_first = __shfl_sync(0xffffffffu, pos, 0);  // lane 0 has the warp's earliest position
    const bool all_live = __all_sync(0xffffffffu, live);
    // Running maximum and sum of the row. A row without a position (past the chunk's end) starts at a
    // finite maximum: all its logits are masked and it never looks for one.
    float m_run = live ? -INFINITY : 0.0f, l_run = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int sb = j & 1, b = j % kBufs;
      if (!(ok = wait_tc(&sm->s_full[t][sb], (j >> 1) & 1, sm, p.status))) break;
      tc_fence_after();
      const int kv0 = j * kTN;
      const uint32_t s_addr = lane_addr + s_col(t, sb);
      // only a tile that reaches past the warp's first position needs the causal mask (warp-uniform)
      const bool masked = !all_live || kv0 + kTN - 1 > pos_first;
      const float4* cs4 = reinterpret_cast<const float4*>(sm->cs[b]);
      // One sweep over the row's 64 logits computes the probabilities against the maximum the row has
      // had so far, and the tile's own maximum on the side. The running maximum is replaced only when
      // a tile exceeds it by more than 2^12 (always so in the first tile): then O and the sum are
      // rescaled and the sweep is repeated against the new maximum. Probabilities therefore stay below
      // 2^12, inside f16, and the final division uses the same maximum as every sum, so the result
      // does not depend on when the maximum moved.
      uint32_t pk[32];
      float l_tile = 0.0f;
#pragma unroll 1
      for (int attempt = 0; attempt < 2; ++attempt) {
        const float base = m_run == -INFINITY ? 0.0f : m_run;
        float m_tile = -INFINITY;
        l_tile = 0.0f;
        uint32_t v2[2][32];  // both halves of the row are requested before the first is waited for
        tmem_ld32(s_addr, v2[0]);
        tmem_ld32(s_addr + 32, v2[1]);
        tmem_ld_wait();
#pragma unroll
        for (int hc = 0; hc < 2; ++hc) {
          const uint32_t(&v)[32] = v2[hc];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 c4 = cs4[hc * 8 + (i >> 2)];
            float y[4] = {__uint_as_float(v[i]) * c4.x, __uint_as_float(v[i + 1]) * c4.y, __uint_as_float(v[i + 2]) * c4.z,
                          __uint_as_float(v[i + 3]) * c4.w};
            if (masked) {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (kv0 + hc * 32 + i + e > pos) y[e] = -INFINITY;
            }
            m_tile = fmaxf(fmaxf(m_tile, fmaxf(y[0], y[1])), fmaxf(y[2], y[3]));
            const float p0 = ex2_approx(y[0] - base), p1 = ex2_approx(y[1] - base), p2 = ex2_approx(y[2] - base),
                        p3 = ex2_approx(y[3] - base);
            l_tile += (p0 + p1) + (p2 + p3);
            const __half2 h01 = __floats2half2_rn(p0, p1), h23 = __floats2half2_rn(p2, p3);
            pk[hc * 16 + (i >> 1)] = *reinterpret_cast<const uint32_t*>(&h01);
            pk[hc * 16 + (i >> 1) + 1] = *reinterpret_cast<const uint32_t*>(&h23);
          }
        }
        const bool grow = m_tile > m_run + 12.0f;  // also true for the first live logits (m_run = -inf)
        if (attempt == 1 || !__any_sync(0xffffffffu, grow)) break;
        const float m_new = grow ? m_tile : m_run;
        const float corr = (grow && m_run > -INFINITY) ? ex2_approx(m_run - m_new) : 1.0f;
        l_run *= corr;
        m_run = m_new;
        if (j > 0) {
          // O has to shrink: it is complete (and nobody adds to it) once the previous tile's P V is done
          if (!(ok = wait_tc(&sm->pv_done[t][(j - 1) & 1], ((j - 1) >> 1) & 1, sm, p.status))) break;
          tc_fence_after();
#pragma unroll 1
          for (int oc = 0; oc < 4; ++oc) {
            uint32_t v[32];
            tmem_ld32(lane_addr + o_col(t) + oc * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
            tmem_st32(lane_addr + o_col(t) + oc * 32, v);
          }
        }
      }
      if (!ok) break;
      l_run += l_tile;
      // The probabilities go over the first 32 columns of the logits they came from. That buffer last
      // held P of tile j - 2, and S of tile j, issued after that tile's P V, has completed: MMAs
      // complete in issue order, so nothing reads the old P any more and no wait is needed here.
      // (P V completions of even and odd tiles are counted on two barriers, so that a thread which
      // has not looked at them for a tile or two still reads the right phase when it has to.)
      tmem_st32(s_addr, pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm->p_full[t][sb]));
    }
    // ---- the finished row: O / l -> bf16
    if (ok && n_kv > 0) ok = wait_tc(&sm->pv_done[t][(n_kv - 1) & 1], ((n_kv - 1) >> 1) & 1, sm, p.status);
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.0f ? 1.0f / l_run : 0.0f;
      uint16_t* dst = p.out + (static_cast<size_t>(live ? crow : 0) * p.Hq + hkv * 4 + hl) * kD;
#pragma unroll 1
      for (int oc = 0; oc < 4; ++oc) {
        uint32_t v[32];
        tmem_ld32(lane_addr + o_col(t) + oc * 32, v);
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + oc * 32 + i) = w;
          }
        }
      }
    }
  }

  // Wind down. On the normal path every softmax thread has seen the last P V complete and every
  // raw stage has been consumed: no MMA and no copy is in flight. After an abort, MMAs and copies
  // already issued get a bounded time to land before the tensor memory and the shared memory go.
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (sm->abort) {
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

}  // namespace

// Launch for a chunk of at least 64 rows; arguments as granite4_prefill_attention_int8 (validated
// there). Returns 1 when the device status word cannot be resolved (the caller then takes the
// mma.sync form), 0 on success, -1 on a launch error.
int attn_prefill_tc(const char* fn, const uint16_t* d_q, float scale, int Hq, int Hk, int base_pos, int rows,
                    int stride, uint16_t* d_out, const int8_t* d_ck, const int8_t* d_cv, const float* d_ks,
                    const float* d_vs, const int* d_pt) {
  unsigned int* status = device_status_ptr();
  if (status == nullptr) return 1;
  static std::atomic<bool> attr_set[64];
  int dev = -1;
  G4_CUDA_TRY(fn, cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_relaxed)) {
    G4_CUDA_TRY(fn, cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kTcSmemBytes)));
    attr_set[dev].store(true, std::memory_order_relaxed);
  }
  TcParams p{};
  p.q = d_q, p.ck = d_ck, p.cv = d_cv, p.ks = d_ks, p.vs = d_vs, p.pt = d_pt, p.out = d_out, p.status = status;
  p.rows = rows, p.base_pos = base_pos, p.Hq = Hq, p.Hk = Hk, p.stride = stride;
  p.scale_log2 = scale * 1.4426950408889634f;
  const dim3 grid(static_cast<unsigned>((rows + kCtaPos - 1) / kCtaPos), static_cast<unsigned>(Hk));
  G4_LAUNCH_PDL(fn, attn_prefill_tc_kernel, grid, dim3(kThreads), kTcSmemBytes, current_stream(), p);
  return 0;
}

}  // namespace g4
