// RoPE on Q/K with the rotated K and the raw V quantised into the int8 paged KV
// cache; RoPE table build; the plain RoPE and int8 append primitives.
//
// Formulation (reference: prefill kernel engine/src/prefill_gemm.cu:356-428,
// decode / verify kernel engine/src/forward_gpu.cu:598-665, scalar math
// engine/src/device_math.cuh:105-134, host twins engine/src/kernel_math.h:71-86,
// :191-219):
//   tables  cos/sin(pos * theta^(-2i/d)) in double, stored f32 [max_pos][d/2]
//   rotate  (a, b) = (x[i], x[i + d/2]): lo = a c - b s, hi = b c + a s (f32)
//   q_rot   = bf16(rotated q)
//   K row   k' = rotated k (f32 in the prefill form, rounded to bf16 in the
//           decode form); amax = max |k'|, s = amax / 127,
//           code = clamp(round_half_away(k' / s), +-127); V the same on raw v
//   paging  code row (hkv * stride + kv_row) * d, scale (hkv * stride + kv_row);
//           kv_row = d_pt[pos] (16-token pages: page_id * 16 + pos % 16)
//
// Kernel layout (d = 128): eight lanes own one head. Lane j holds columns
// [8j, 8j+8) and [64+8j, 64+8j+8), i.e. both halves of its eight rotation
// pairs, so the rotation needs no exchange and the row amax is three xor
// shuffles. A 128-thread CTA covers one token row: thread (g, j) owns lane j of
// the heads g, g + 16, g + 32 (all 48 heads of a Granite row), so the cos / sin
// values of lane j are loaded once per row and reused for every head. Loads are
// 128-bit (a warp reads four whole heads = 1 KB) and all issued before the first
// is used, q_rot stores are 128-bit, code stores are two 8-byte pieces per lane
// that together fill the head's 128-byte cache row.
//
// Algorithmic bytes per token row (Hq 32, Hk 8): q 8192 + k 2048 + v 2048 +
// cos/sin 512 + ids 8 read; q_rot 8192 + codes 2048 + scales 64 written =
// 23 108 B.
#include "g4_host.h"
#include "g4_math.cuh"
#include "g4_tma.cuh"

#include "../../include/granite4_b200.h"
#include "../../include/granite4_b200.hpp"

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <vector>

namespace g4 {
namespace {

enum RowMode { kRunOfPositions = 0, kPerRowArrays = 1, kDescriptor = 2 };

struct RopeKvParams {
  const uint16_t* q;  // row pitch pitch_q elements; NULL when there is no q
  const uint16_t* k;
  const uint16_t* v;
  long long pitch_q, pitch_k, pitch_v;
  const float* cos_tbl;
  const float* sin_tbl;
  uint16_t* q_rot;  // [rows][Hq * 128]
  int8_t* cache_k;
  int8_t* cache_v;
  float* k_scale;
  float* v_scale;
  // where row r sits
  int mode;
  int base_pos;
  const int* pos_rows;
  const int* kv_rows;
  const int* d_pt;
  const granite4_multi_rows* mr;
  int max_pos;  // bound for pos_rows (kPerRowArrays)
  int rows, Hq, Hk;
  long long stride;
  int rotate_k;     // 0: K rows are appended as they are (plain append)
  int k_from_bf16;  // quantise the bf16-rounded rotated K
};

constexpr int kD = 128;
constexpr int kHeadsPerCta = 16;

// One 128-thread CTA handles kRows token rows, all heads: thread (g, j) = (tid / 8, tid % 8) owns
// lane j of the heads g, g + 16, g + 32, ... of each row. The cos / sin values of lane j depend
// only on the row, so they are loaded once per row and reused for every head of the thread.
// All the activation loads of a row are issued before the first is used.
constexpr int kMaxHeadsPerThread = 4;  // (Hq + 2 Hk) <= 64 heads per row in this kernel

template <int kRows>
__global__ void __launch_bounds__(kHeadsPerCta * 8) rope_kv_int8_kernel(const RopeKvParams p) {
  pdl_begin();
  const int g = threadIdx.x >> 3;
  const int j = threadIdx.x & 7;
  const int heads_total = p.Hq + 2 * p.Hk;
  const unsigned gmask = 0xffu << (threadIdx.x & 24);  // the 8 lanes that share this thread's heads
#pragma unroll
  for (int i = 0; i < kRows; ++i) {
    const int r = blockIdx.x * kRows + i;
    if (r >= p.rows) return;  // uniform over the CTA
    int pos, kv_row;
    if (p.mode == kRunOfPositions) {
      pos = p.base_pos + r;
      kv_row = p.d_pt != nullptr ? __ldg(p.d_pt + pos) : pos;
    } else if (p.mode == kPerRowArrays) {
      pos = __ldg(p.pos_rows + r);
      kv_row = __ldg(p.kv_rows + r);
      // a bad index skips the row instead of touching memory outside the tables or the pool
      if (pos < 0 || pos >= p.max_pos || kv_row < 0 || kv_row >= p.stride) continue;
    } else {
      pos = p.mr->pos[r];
      const int slot = p.mr->tree ? p.mr->slot[r] : pos;
      kv_row = p.mr->pt[r][slot];
    }
    // activations of every head this thread owns in this row
    uint4 xlo[kMaxHeadsPerThread], xhi[kMaxHeadsPerThread];
#pragma unroll
    for (int k = 0; k < kMaxHeadsPerThread; ++k) {
      const int head = g + k * kHeadsPerCta;
      if (head >= heads_total) break;
      const uint16_t* src;
      if (head < p.Hq) src = p.q + static_cast<size_t>(r) * p.pitch_q + static_cast<size_t>(head) * kD;
      else if (head < p.Hq + p.Hk) src = p.k + static_cast<size_t>(r) * p.pitch_k + static_cast<size_t>(head - p.Hq) * kD;
      else src = p.v + static_cast<size_t>(r) * p.pitch_v + static_cast<size_t>(head - p.Hq - p.Hk) * kD;
      xlo[k] = ld_stream(reinterpret_cast<const uint4*>(src) + j);
      xhi[k] = ld_stream(reinterpret_cast<const uint4*>(src) + 8 + j);
    }
    float c[8], s[8];
    if (p.cos_tbl != nullptr) {
      const float4* cp = reinterpret_cast<const float4*>(p.cos_tbl + static_cast<size_t>(pos) * (kD / 2)) + 2 * j;
      const float4* sp = reinterpret_cast<const float4*>(p.sin_tbl + static_cast<size_t>(pos) * (kD / 2)) + 2 * j;
      const float4 c0 = __ldg(cp), c1 = __ldg(cp + 1), s0 = __ldg(sp), s1 = __ldg(sp + 1);
      c[0] = c0.x, c[1] = c0.y, c[2] = c0.z, c[3] = c0.w, c[4] = c1.x, c[5] = c1.y, c[6] = c1.z, c[7] = c1.w;
      s[0] = s0.x, s[1] = s0.y, s[2] = s0.z, s[3] = s0.w, s[4] = s1.x, s[5] = s1.y, s[6] = s1.z, s[7] = s1.w;
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) c[e] = 1.0f, s[e] = 0.0f;
    }
#pragma unroll
    for (int k = 0; k < kMaxHeadsPerThread; ++k) {
      const int head = g + k * kHeadsPerCta;
      if (head >= heads_total) break;
      const bool is_q = head < p.Hq;
      const bool is_k = !is_q && head < p.Hq + p.Hk;
      float lo[8], hi[8];
      unpack8(xlo[k], lo);
      unpack8(xhi[k], hi);
      if (is_q || (is_k && p.rotate_k)) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float a, b;
          rope_pair(lo[e], hi[e], c[e], s[e], a, b);
          lo[e] = a, hi[e] = b;
        }
      }
      if (is_q) {
        uint4* dst = reinterpret_cast<uint4*>(p.q_rot + (static_cast<size_t>(r) * p.Hq + head) * kD);
        st_stream(dst + j, pack8(lo));
        st_stream(dst + 8 + j, pack8(hi));
        continue;
      }
      if (is_k && p.rotate_k && p.k_from_bf16) {
#pragma unroll
        for (int e = 0; e < 8; ++e) lo[e] = round_bf16(lo[e]), hi[e] = round_bf16(hi[e]);
      }
      float amax = 0.0f;
#pragma unroll
      for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fmaxf(fabsf(lo[e]), fabsf(hi[e])));
      // is_q / is_k depend on g only, so the 8 lanes of a head take the same path here
      amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 4));
      const Kv8Scale sc = kv8_scale(amax);
      const int hkv = is_k ? head - p.Hq : head - p.Hq - p.Hk;
      const size_t srow = static_cast<size_t>(hkv) * p.stride + kv_row;
      int8_t* cache = (is_k ? p.cache_k : p.cache_v) + srow * kD;
      if (j == 0) (is_k ? p.k_scale : p.v_scale)[srow] = sc.s;
      const uint2 cl = kv8_quant8(lo, sc), ch = kv8_quant8(hi, sc);
      st_stream(reinterpret_cast<uint2*>(cache) + j, cl);
      st_stream(reinterpret_cast<uint2*>(cache) + 8 + j, ch);
    }
  }
}

// ---- the same op with the inputs staged by bulk asynchronous copies ------------------------------
// The per-row work above is short and every CTA starts with a dependent chain (row index ->
// position -> table row), so at one CTA per row the kernel is latency-bound. Here persistent CTAs
// stream their rows through a ring of shared-memory stages instead. A producer warp (one elected
// thread) reads each row's position and pool row - one row ahead of the one it is issuing, so that
// the load's latency never sits between two issues - and issues bulk asynchronous copies (TMA engine,
// cp.async.bulk + mbarrier, no multicast) of the row's activations (one 12 KB copy for token-major
// qkv, three for separate q / k / v) and of its cos and sin table rows (256 B each) up to kBulkStages
// rows ahead; four consumer warps compute row i out of shared memory while the copies of the next
// rows are in flight, and store results straight to global memory. Stages go back to the producer
// through a second set of mbarriers (one arrival per consumer warp), so the loop has no CTA-wide
// barrier and the consumers never wait for anything but data. Bytes in flight per SM are bounded by
// shared memory (4 CTAs x 4 stages x 12.8 KB), not by registers or occupancy. The consumers' thread
// layout is the one of rope_kv_int8_kernel (every thread gets two query heads and one key or value
// head of a Granite row). The arithmetic, and so every output bit, is that of rope_kv_int8_kernel.
constexpr int kBulkStages = 4;
constexpr int kBulkConsumers = 128;                    // 16 heads per pass, 8 lanes each
constexpr int kBulkThreads = kBulkConsumers + 32;      // + the producer warp
constexpr int kBulkHeadsPerPass = kBulkConsumers / 8;  // thread (g, j) owns heads g, g + 16, g + 32, ...

struct RowMeta {
  int pos, kv_row, ok, pad;
};

// Bounded wait that also gives up when another thread of the CTA already has.
__device__ __forceinline__ bool mbar_wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kMbarWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (i > 64) __nanosleep(64);
  }
  *abort_flag = 1;
  return false;
}

__global__ void __launch_bounds__(kBulkThreads, 4) rope_kv_bulk_kernel(const RopeKvParams p,
                                                                    unsigned int* status) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int heads_total = p.Hq + 2 * p.Hk;
  const uint32_t act_bytes = static_cast<uint32_t>(heads_total) * kD * 2u;
  const uint32_t tbl_bytes = (kD / 2) * 4u;  // one table row
  const uint32_t stage_bytes = act_bytes + 2u * tbl_bytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + static_cast<size_t>(kBulkStages) * stage_bytes);
  uint64_t* empty = full + kBulkStages;
  RowMeta* meta = reinterpret_cast<RowMeta*>(empty + kBulkStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(meta + kBulkStages);
  const int t = threadIdx.x;
  const long long n_local = (p.rows - static_cast<long long>(blockIdx.x) + gridDim.x - 1) / gridDim.x;

  // the barriers live in shared memory: they are set up while the kernel before this one drains
  if (t == 0) {
    for (int s = 0; s < kBulkStages; ++s) mbar_init(full + s, 1), mbar_init(empty + s, kBulkConsumers / 32);
    *abort_flag = 0;
    mbar_init_fence();
  }
  pdl_begin();
  __syncthreads();

  if (t >= kBulkConsumers) {
    // ---- producer ----------------------------------------------------------------------------
    if (t != kBulkConsumers) return;
    auto where = [&](long long i, int& pos, int& kv_row, int& ok) {
      const int r = static_cast<int>(blockIdx.x + i * static_cast<long long>(gridDim.x));
      ok = 1;
      if (p.mode == kRunOfPositions) {
        pos = p.base_pos + r;
        kv_row = p.d_pt != nullptr ? __ldg(p.d_pt + pos) : pos;
      } else if (p.mode == kPerRowArrays) {
        pos = __ldg(p.pos_rows + r);
        kv_row = __ldg(p.kv_rows + r);
      } else {
        pos = p.mr->pos[r];
        const int slot = p.mr->tree ? p.mr->slot[r] : pos;
        kv_row = p.mr->pt[r][slot];
      }
    };
    int pos = 0, kv_row = 0, ok = 1;
    if (n_local > 0) where(0, pos, kv_row, ok);
    long long issued = 0;
    bool good = true;
    for (long long i = 0; i < n_local; ++i) {
      const int s = static_cast<int>(i % kBulkStages);
      int npos = 0, nkv = 0, nok = 1;
      if (i + 1 < n_local) where(i + 1, npos, nkv, nok);  // in flight while this row is issued
      if (!(good = mbar_wait_or_abort(empty + s, static_cast<uint32_t>(((i / kBulkStages) & 1) ^ 1), abort_flag))) break;
      const int r = static_cast<int>(blockIdx.x + i * static_cast<long long>(gridDim.x));
      // a bad index skips the row instead of touching memory outside the tables or the pool
      if (p.mode == kPerRowArrays && (pos < 0 || pos >= p.max_pos || kv_row < 0 || kv_row >= p.stride)) ok = 0;
      meta[s].pos = pos, meta[s].kv_row = kv_row, meta[s].ok = ok;
      unsigned char* stage = smem + static_cast<size_t>(s) * stage_bytes;
      if (!ok) {  // nothing to copy: one plain arrival completes the phase
        mbar_arrive_expect_tx(full + s, 0);
      } else {
        const bool tables = p.cos_tbl != nullptr;
        mbar_arrive_expect_tx(full + s, act_bytes + (tables ? 2u * tbl_bytes : 0u));
        const uint32_t qb = static_cast<uint32_t>(p.Hq) * kD * 2u, kb = static_cast<uint32_t>(p.Hk) * kD * 2u;
        if (p.q != nullptr && p.k == p.q + static_cast<size_t>(p.Hq) * kD &&
            p.v == p.k + static_cast<size_t>(p.Hk) * kD && p.pitch_q == p.pitch_k && p.pitch_k == p.pitch_v) {
          bulk_load(stage, p.q + static_cast<size_t>(r) * p.pitch_q, act_bytes, full + s);  // token-major row
        } else {
          if (qb != 0u) bulk_load(stage, p.q + static_cast<size_t>(r) * p.pitch_q, qb, full + s);
          bulk_load(stage + qb, p.k + static_cast<size_t>(r) * p.pitch_k, kb, full + s);
          bulk_load(stage + qb + kb, p.v + static_cast<size_t>(r) * p.pitch_v, kb, full + s);
        }
        if (tables) {
          bulk_load(stage + act_bytes, p.cos_tbl + static_cast<size_t>(pos) * (kD / 2), tbl_bytes, full + s);
          bulk_load(stage + act_bytes + tbl_bytes, p.sin_tbl + static_cast<size_t>(pos) * (kD / 2), tbl_bytes,
                    full + s);
        }
      }
      issued = i + 1;
      pos = npos, kv_row = nkv, ok = nok;
    }
    if (!good) {
      // A stage never came back, or a consumer gave up. Record it and give every copy issued so far one
      // more bounded chance to land, so that none is in flight towards this CTA's shared memory at exit.
      atomicOr(status, kStatusRopeWaitTimeout);
      for (long long i = issued > kBulkStages ? issued - kBulkStages : 0; i < issued; ++i)
        (void)mbar_wait_bounded(full + (i % kBulkStages), static_cast<uint32_t>((i / kBulkStages) & 1));
    } else {
      // normal path: the consumers hand the last stages back only after reading them, i.e. after
      // their copies landed; wait for that so that no copy outlives the CTA's shared memory
      for (long long i = n_local > kBulkStages ? n_local - kBulkStages : 0; i < n_local; ++i)
        if (!mbar_wait_or_abort(empty + (i % kBulkStages), static_cast<uint32_t>((i / kBulkStages) & 1), abort_flag)) {
          atomicOr(status, kStatusRopeWaitTimeout);
          break;
        }
    }
    return;
  }

  // ---- consumers -------------------------------------------------------------------------------
  const int g = t >> 3, j = t & 7, lane = t & 31;
  const unsigned gmask = 0xffu << (t & 24);
  for (long long i = 0; i < n_local; ++i) {
    const int s = static_cast<int>(i % kBulkStages);
    if (!mbar_wait_or_abort(full + s, static_cast<uint32_t>((i / kBulkStages) & 1), abort_flag)) {
      if (lane == 0) atomicOr(status, kStatusRopeWaitTimeout);
      return;
    }
    const RowMeta m = meta[s];
    if (m.ok) {
      const int r = static_cast<int>(blockIdx.x + i * static_cast<long long>(gridDim.x));
      const unsigned char* stage = smem + static_cast<size_t>(s) * stage_bytes;
      float c[8], sn[8];
      if (p.cos_tbl != nullptr) {
        const float4* cp = reinterpret_cast<const float4*>(stage + act_bytes) + 2 * j;
        const float4* sp = reinterpret_cast<const float4*>(stage + act_bytes + tbl_bytes) + 2 * j;
        const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
        c[0] = c0.x, c[1] = c0.y, c[2] = c0.z, c[3] = c0.w, c[4] = c1.x, c[5] = c1.y, c[6] = c1.z, c[7] = c1.w;
        sn[0] = s0.x, sn[1] = s0.y, sn[2] = s0.z, sn[3] = s0.w, sn[4] = s1.x, sn[5] = s1.y, sn[6] = s1.z, sn[7] = s1.w;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) c[e] = 1.0f, sn[e] = 0.0f;
      }
#pragma unroll
      for (int k = 0; k < kMaxHeadsPerThread; ++k) {
        const int head = g + k * kBulkHeadsPerPass;
        if (head >= heads_total) break;
        const bool is_q = head < p.Hq;
        const bool is_k = !is_q && head < p.Hq + p.Hk;
        const uint4* src = reinterpret_cast<const uint4*>(stage + static_cast<size_t>(head) * kD * 2);
        float lo[8], hi[8];
        unpack8(src[j], lo);
        unpack8(src[8 + j], hi);
        if (is_q || (is_k && p.rotate_k)) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float a, b;
            rope_pair(lo[e], hi[e], c[e], sn[e], a, b);
            lo[e] = a, hi[e] = b;
          }
        }
        if (is_q) {
          uint4* dst = reinterpret_cast<uint4*>(p.q_rot + (static_cast<size_t>(r) * p.Hq + head) * kD);
          st_stream(dst + j, pack8(lo));
          st_stream(dst + 8 + j, pack8(hi));
          continue;
        }
        if (is_k && p.rotate_k && p.k_from_bf16) {
#pragma unroll
          for (int e = 0; e < 8; ++e) lo[e] = round_bf16(lo[e]), hi[e] = round_bf16(hi[e]);
        }
        float amax = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fmaxf(fabsf(lo[e]), fabsf(hi[e])));
        amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 4));
        const Kv8Scale sc = kv8_scale(amax);
        const int hkv = is_k ? head - p.Hq : head - p.Hq - p.Hk;
        const size_t srow = static_cast<size_t>(hkv) * p.stride + m.kv_row;
        int8_t* cache = (is_k ? p.cache_k : p.cache_v) + srow * kD;
        if (j == 0) (is_k ? p.k_scale : p.v_scale)[srow] = sc.s;
        const uint2 cl = kv8_quant8(lo, sc), ch = kv8_quant8(hi, sc);
        st_stream(reinterpret_cast<uint2*>(cache) + j, cl);
        st_stream(reinterpret_cast<uint2*>(cache) + 8 + j, ch);
      }
    }
    // the warp is done reading the stage: it goes back to the producer
    __syncwarp();
    if (lane == 0) mbar_arrive_local(empty + s);
  }
}

// Plain RoPE of [rows][d] with table row = row index; any even d. One thread
// per rotation pair (a test primitive in the reference, kept for its callers).
__global__ void __launch_bounds__(256)
    rope_rows_kernel(const uint16_t* x, const float* cos_tbl, const float* sin_tbl, int rows, int d,
                     uint16_t* out) {
  const int half = d / 2;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(rows) * half) return;
  const long long row = idx / half;
  const int i = static_cast<int>(idx % half);
  const float a = bf16_to_f32(x[row * d + i]), b = bf16_to_f32(x[row * d + i + half]);
  float lo, hi;
  rope_pair(a, b, cos_tbl[row * half + i], sin_tbl[row * half + i], lo, hi);
  out[row * d + i] = static_cast<uint16_t>(f32_to_bf16_bits(lo));
  out[row * d + i + half] = static_cast<uint16_t>(f32_to_bf16_bits(hi));
}

// int8 append of bf16 K/V rows for head dims other than 128: one CTA of d
// threads per (kv head, row), shared-memory amax.
__global__ void __launch_bounds__(1024)
    kv_append_int8_generic_kernel(const uint16_t* src_k, const uint16_t* src_v, int8_t* cache_k,
                                  int8_t* cache_v, float* k_scale, float* v_scale, int base_pos,
                                  int stride, int Hk, int d, const int* d_pt,
                                  const granite4_multi_rows* mr) {
  const int hkv = blockIdx.x, r = blockIdx.y, i = threadIdx.x;
  int row;
  if (mr != nullptr) {
    row = mr->pt[r][mr->tree ? mr->slot[r] : mr->pos[r]];
  } else {
    const int pos = base_pos + r;
    row = d_pt != nullptr ? d_pt[pos] : pos;
  }
  const bool act = i < d;  // the CTA is d rounded up to whole warps
  const size_t src = (static_cast<size_t>(r) * Hk + hkv) * d + i;
  const float x = act ? bf16_to_f32(src_k[src]) : 0.0f, y = act ? bf16_to_f32(src_v[src]) : 0.0f;
  float ax = warp_max(fabsf(x)), ay = warp_max(fabsf(y));
  __shared__ float wmax[2][32];
  if ((i & 31) == 0) wmax[0][i >> 5] = ax, wmax[1][i >> 5] = ay;
  __syncthreads();
  float mk = 0.0f, mv = 0.0f;
  for (int w = 0; w < (d + 31) / 32; ++w) mk = fmaxf(mk, wmax[0][w]), mv = fmaxf(mv, wmax[1][w]);
  const float sk = kv8_scale(mk).s, sv = kv8_scale(mv).s;
  const size_t srow = static_cast<size_t>(hkv) * stride + row;
  if (i == 0) k_scale[srow] = sk, v_scale[srow] = sv;
  if (!act) return;
  cache_k[srow * d + i] = static_cast<int8_t>(kv8_quant_exact(x, sk));
  cache_v[srow * d + i] = static_cast<int8_t>(kv8_quant_exact(y, sv));
}

int launch_rope_kv(const char* fn, RopeKvParams& p) {
  const int heads_total = p.Hq + 2 * p.Hk;
  if (heads_total > kMaxHeadsPerThread * kHeadsPerCta) return fail(fn, "more than 64 heads per row");
  cudaStream_t st = current_stream();
  // Bulk-copy path (default): needs 16-byte aligned sources and a status word to report to.
  const char* env = std::getenv("G4_ROPE_BULK");
  const bool want_bulk = !(env != nullptr && env[0] == '0');
  unsigned int* status = want_bulk ? device_status_ptr() : nullptr;
  const size_t stage_bytes = static_cast<size_t>(heads_total) * kD * 2 + 2 * (kD / 2) * 4;
  const size_t smem = kBulkStages * stage_bytes + kBulkStages * (2 * sizeof(uint64_t) + sizeof(RowMeta)) + 16;
  const bool aligned = aligned16(p.q) && aligned16(p.k) && aligned16(p.v) && aligned16(p.cos_tbl) &&
                       aligned16(p.sin_tbl) && (p.pitch_q * 2) % 16 == 0 && (p.pitch_k * 2) % 16 == 0 &&
                       (p.pitch_v * 2) % 16 == 0;
  if (status != nullptr && aligned && heads_total <= kMaxHeadsPerThread * kBulkHeadsPerPass && smem <= 100 * 1024) {
    static std::atomic<bool> attr_set[64];  // per device; relaxed: setting the attribute twice is harmless
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(fn, "cannot identify the current device");
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_relaxed)) {
      G4_CUDA_TRY(fn, cudaFuncSetAttribute(rope_kv_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           100 * 1024));
      attr_set[dev].store(true, std::memory_order_relaxed);
    }
    const int per_sm = static_cast<int>(std::max<size_t>(1, std::min<size_t>(4, (220 * 1024) / smem)));
    const unsigned grid = static_cast<unsigned>(std::min<long long>(p.rows, static_cast<long long>(sm_count()) * per_sm));
    G4_LAUNCH_PDL(fn, rope_kv_bulk_kernel, dim3(grid), dim3(kBulkThreads), smem, st, p, status);
  } else {
    G4_LAUNCH_PDL(fn, rope_kv_int8_kernel<1>, dim3(static_cast<unsigned>(p.rows)), dim3(kHeadsPerCta * 8), 0,
                  st, p);
  }
  return 0;
}

}  // namespace

// bf16-cache form (rope_bf16.cu).
int multi_rope_append_bf16(const char* fn, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                           const float* cos_tbl, const float* sin_tbl,
                           const granite4_multi_rows* d_rows, int rows, int Hq, int Hk, int d,
                           uint16_t* cache_k, uint16_t* cache_v, int stride, uint16_t* q_rot);

// The int8 append of the multi-row helpers: K and V rows as they are, row r into the pool row its
// descriptor names (engine/src/forward_gpu.cu:3919-3923, kv_append_int8_multi_kernel :427-452).
int multi_kv_append_int8(const char* fn, const uint16_t* k, const uint16_t* v, int8_t* cache_k,
                         int8_t* cache_v, float* k_scale, float* v_scale,
                         const granite4_multi_rows* d_rows, int rows, int stride, int Hk, int d) {
  if (k_scale == nullptr || v_scale == nullptr || d > 1024) return fail(fn, "invalid arguments");
  const bool fast = d == kD && aligned16(k) && aligned16(v) && aligned16(cache_k) && aligned16(cache_v);
  if (!fast) {
    kv_append_int8_generic_kernel<<<dim3(Hk, rows), (d + 31) / 32 * 32, 0, current_stream()>>>(
        k, v, cache_k, cache_v, k_scale, v_scale, 0, stride, Hk, d, nullptr, d_rows);
    G4_LAUNCH_CHECK(fn);
    return 0;
  }
  RopeKvParams p{};
  p.q = nullptr, p.k = k, p.v = v;
  p.pitch_k = p.pitch_v = static_cast<long long>(Hk) * d;
  p.cache_k = cache_k, p.cache_v = cache_v, p.k_scale = k_scale, p.v_scale = v_scale;
  p.mode = kDescriptor, p.mr = d_rows;
  p.rows = rows, p.Hq = 0, p.Hk = Hk, p.stride = stride, p.rotate_k = 0, p.k_from_bf16 = 0;
  return launch_rope_kv(fn, p);
}

}  // namespace g4

extern "C" {

int granite4_rope_tables_build(double theta, int head_dim, int max_pos, float** d_cos,
                               float** d_sin) {
  const char* fn = "granite4_rope_tables_build";
  if (d_cos == nullptr || d_sin == nullptr || !std::isfinite(theta) || theta <= 0.0 ||
      head_dim <= 0 || (head_dim & 1) != 0 || head_dim > 256 || max_pos <= 0)
    return g4::fail(fn, "invalid arguments");
  *d_cos = nullptr;
  *d_sin = nullptr;
  const int half = head_dim / 2;
  const size_t n = static_cast<size_t>(max_pos) * half;
  std::vector<float> h_cos(n), h_sin(n);
  // engine/src/kernel_math.h:191-206: everything in double, stored as f32.
  for (int i = 0; i < half; ++i) {
    const double inv_freq = 1.0 / std::pow(theta, 2.0 * static_cast<double>(i) / head_dim);
    for (int pos = 0; pos < max_pos; ++pos) {
      const double angle = static_cast<double>(pos) * inv_freq;
      h_cos[static_cast<size_t>(pos) * half + i] = static_cast<float>(std::cos(angle));
      h_sin[static_cast<size_t>(pos) * half + i] = static_cast<float>(std::sin(angle));
    }
  }
  float *c = nullptr, *s = nullptr;
  if (cudaMalloc(&c, n * sizeof(float)) != cudaSuccess) return g4::fail(fn, "cudaMalloc failed");
  if (cudaMalloc(&s, n * sizeof(float)) != cudaSuccess) {
    cudaFree(c);
    return g4::fail(fn, "cudaMalloc failed");
  }
  if (cudaMemcpy(c, h_cos.data(), n * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess ||
      cudaMemcpy(s, h_sin.data(), n * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaFree(c);
    cudaFree(s);
    return g4::fail(fn, "upload failed");
  }
  *d_cos = c;
  *d_sin = s;
  return 0;
}

int granite4_kernel_rope(const uint16_t* d_x, const float* d_cos, const float* d_sin, int rows,
                         int head_dim, uint16_t* d_out) {
  const char* fn = "granite4_kernel_rope";
  if (d_x == nullptr || d_cos == nullptr || d_sin == nullptr || d_out == nullptr || rows <= 0 ||
      head_dim <= 0 || (head_dim & 1) != 0 || static_cast<long long>(rows) * head_dim > INT_MAX ||
      head_dim > 256)
    return g4::fail(fn, "invalid arguments");
  const long long pairs = static_cast<long long>(rows) * (head_dim / 2);
  g4::rope_rows_kernel<<<static_cast<unsigned>((pairs + 255) / 256), 256, 0, g4::current_stream()>>>(
      d_x, d_cos, d_sin, rows, head_dim, d_out);
  G4_LAUNCH_CHECK(fn);
  return 0;
}

int granite4_kernel_kv_append_int8_batched(const uint16_t* d_src_k, const uint16_t* d_src_v,
                                           int8_t* d_cache_k, int8_t* d_cache_v,
                                           float* d_cache_k_scale, float* d_cache_v_scale,
                                           int base_pos, int rows, int stride, int Hk, int d,
                                           const int* d_pt) {
  const char* fn = "granite4_kernel_kv_append_int8_batched";
  if (d_src_k == nullptr || d_src_v == nullptr || d_cache_k == nullptr || d_cache_v == nullptr ||
      d_cache_k_scale == nullptr || d_cache_v_scale == nullptr || base_pos < 0 || rows <= 0 ||
      rows > GRANITE4_MAX_VERIFY_ROWS || Hk <= 0 || d <= 0 || d > 1024 ||
      base_pos > INT_MAX - rows || stride < base_pos + rows ||
      static_cast<long long>(Hk) * d > INT_MAX || stride > INT_MAX / (Hk > 1 ? Hk : 1))
    return g4::fail(fn, "invalid arguments");
  const bool fast = d == g4::kD && g4::aligned16(d_src_k) && g4::aligned16(d_src_v) &&
                    g4::aligned16(d_cache_k) && g4::aligned16(d_cache_v);
  if (!fast) {
    g4::kv_append_int8_generic_kernel<<<dim3(Hk, rows), (d + 31) / 32 * 32, 0,
                                        g4::current_stream()>>>(
        d_src_k, d_src_v, d_cache_k, d_cache_v, d_cache_k_scale, d_cache_v_scale, base_pos, stride,
        Hk, d, d_pt, nullptr);
    G4_LAUNCH_CHECK(fn);
    return 0;
  }
  g4::RopeKvParams p{};
  p.q = nullptr, p.k = d_src_k, p.v = d_src_v;
  p.pitch_k = p.pitch_v = static_cast<long long>(Hk) * d;
  p.cache_k = d_cache_k, p.cache_v = d_cache_v, p.k_scale = d_cache_k_scale,
  p.v_scale = d_cache_v_scale;
  p.mode = g4::kRunOfPositions, p.base_pos = base_pos, p.d_pt = d_pt;
  p.rows = rows, p.Hq = 0, p.Hk = Hk, p.stride = stride, p.rotate_k = 0, p.k_from_bf16 = 0;
  return g4::launch_rope_kv(fn, p);
}

int granite4_prefill_rope_split_append_int8(const uint16_t* qkv, const float* cos_tbl,
                                            const float* sin_tbl, int base_pos, int rows, int Hq,
                                            int Hk, int d, int stride, uint16_t* q_rot,
                                            int8_t* cache_k, int8_t* cache_v,
                                            float* cache_k_scale, float* cache_v_scale,
                                            const int* d_pt) {
  const char* fn = "prefill_rope_split_append_int8";
  // engine/src/prefill_gemm.cu:1335-1340 (qkv / table pointers are checked too here)
  if (rows <= 0 || rows > 65535 || base_pos < 0 || stride < base_pos + rows || d != g4::kD ||
      Hq <= 0 || Hk <= 0 || q_rot == nullptr || cache_k == nullptr || cache_v == nullptr ||
      cache_k_scale == nullptr || cache_v_scale == nullptr || qkv == nullptr ||
      cos_tbl == nullptr || sin_tbl == nullptr)
    return g4::fail(fn, "invalid arguments");
  if (!g4::aligned16(qkv) || !g4::aligned16(q_rot) || !g4::aligned16(cache_k) ||
      !g4::aligned16(cache_v) || !g4::aligned16(cos_tbl) || !g4::aligned16(sin_tbl))
    return g4::fail(fn, "pointers must be 16-byte aligned");
  g4::RopeKvParams p{};
  const long long pitch = static_cast<long long>(Hq + 2 * Hk) * d;
  p.q = qkv, p.k = qkv + static_cast<size_t>(Hq) * d, p.v = qkv + static_cast<size_t>(Hq + Hk) * d;
  p.pitch_q = p.pitch_k = p.pitch_v = pitch;
  p.cos_tbl = cos_tbl, p.sin_tbl = sin_tbl, p.q_rot = q_rot;
  p.cache_k = cache_k, p.cache_v = cache_v, p.k_scale = cache_k_scale, p.v_scale = cache_v_scale;
  p.mode = g4::kRunOfPositions, p.base_pos = base_pos, p.d_pt = d_pt;
  p.rows = rows, p.Hq = Hq, p.Hk = Hk, p.stride = stride, p.rotate_k = 1, p.k_from_bf16 = 0;
  return g4::launch_rope_kv(fn, p);
}

int granite4_gpu_multi_rope_append(const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                   const float* cos_tbl, const float* sin_tbl,
                                   const granite4_multi_rows* d_rows, int rows, int Hq, int Hk,
                                   int d, int bits, void* cache_k, void* cache_v, float* k_scale,
                                   float* v_scale, int stride, uint16_t* q_rot) {
  const char* fn = "gpu_multi_rope_append";
  // engine/src/forward_gpu.cu:3911 (-1 also tells the caller to take its unfused path)
  if (d_rows == nullptr || rows < 1 || rows > GRANITE4_MAX_VERIFY_ROWS) return -1;
  if (bits == 16)
    return g4::multi_rope_append_bf16(fn, q, k, v, cos_tbl, sin_tbl, d_rows, rows, Hq, Hk, d,
                                      static_cast<uint16_t*>(cache_k), static_cast<uint16_t*>(cache_v),
                                      stride, q_rot);
  if (bits != 8 || d != g4::kD) return -1;  // the 4- and 5-bit cache formats are not built here
  if (q == nullptr || k == nullptr || v == nullptr || cos_tbl == nullptr || sin_tbl == nullptr ||
      cache_k == nullptr || cache_v == nullptr || k_scale == nullptr || v_scale == nullptr ||
      q_rot == nullptr || Hq <= 0 || Hk <= 0 || stride <= 0)
    return g4::fail(fn, "invalid arguments");
  g4::RopeKvParams p{};
  p.q = q, p.k = k, p.v = v;
  p.pitch_q = static_cast<long long>(Hq) * d, p.pitch_k = p.pitch_v = static_cast<long long>(Hk) * d;
  p.cos_tbl = cos_tbl, p.sin_tbl = sin_tbl, p.q_rot = q_rot;
  p.cache_k = static_cast<int8_t*>(cache_k), p.cache_v = static_cast<int8_t*>(cache_v);
  p.k_scale = k_scale, p.v_scale = v_scale;
  p.mode = g4::kDescriptor, p.mr = d_rows;
  p.rows = rows, p.Hq = Hq, p.Hk = Hk, p.stride = stride, p.rotate_k = 1, p.k_from_bf16 = 1;
  return g4::launch_rope_kv(fn, p);
}

int granite4_kernel_rope_kv_int8_paged(const uint16_t* d_qkv, const float* d_cos,
                                       const float* d_sin, const int* d_pos_rows,
                                       const int* d_kv_rows, int rows, int Hq, int Hk, int d,
                                       int stride, int max_pos, int k_from_bf16,
                                       uint16_t* d_q_rot, int8_t* d_cache_k, int8_t* d_cache_v,
                                       float* d_k_scale, float* d_v_scale) {
  const char* fn = "granite4_kernel_rope_kv_int8_paged";
  if (d_qkv == nullptr || d_cos == nullptr || d_sin == nullptr || d_pos_rows == nullptr ||
      d_kv_rows == nullptr || rows <= 0 || Hq <= 0 || Hk <= 0 || d != g4::kD || stride <= 0 ||
      max_pos <= 0 || d_q_rot == nullptr || d_cache_k == nullptr || d_cache_v == nullptr ||
      d_k_scale == nullptr || d_v_scale == nullptr)
    return g4::fail(fn, "invalid arguments");
  if (!g4::aligned16(d_qkv) || !g4::aligned16(d_q_rot) || !g4::aligned16(d_cache_k) ||
      !g4::aligned16(d_cache_v) || !g4::aligned16(d_cos) || !g4::aligned16(d_sin))
    return g4::fail(fn, "pointers must be 16-byte aligned");
  g4::RopeKvParams p{};
  const long long pitch = static_cast<long long>(Hq + 2 * Hk) * d;
  p.q = d_qkv, p.k = d_qkv + static_cast<size_t>(Hq) * d,
  p.v = d_qkv + static_cast<size_t>(Hq + Hk) * d;
  p.pitch_q = p.pitch_k = p.pitch_v = pitch;
  p.cos_tbl = d_cos, p.sin_tbl = d_sin, p.q_rot = d_q_rot;
  p.cache_k = d_cache_k, p.cache_v = d_cache_v, p.k_scale = d_k_scale, p.v_scale = d_v_scale;
  p.mode = g4::kPerRowArrays, p.pos_rows = d_pos_rows, p.kv_rows = d_kv_rows, p.max_pos = max_pos;
  p.rows = rows, p.Hq = Hq, p.Hk = Hk, p.stride = stride, p.rotate_k = 1,
  p.k_from_bf16 = k_from_bf16 != 0;
  return g4::launch_rope_kv(fn, p);
}

}  // extern "C"

namespace granite4 {

int prefill_rope_split_append_int8(const std::uint16_t* qkv, const float* cos_tbl,
                                   const float* sin_tbl, int base_pos, int rows, int Hq, int Hk,
                                   int d, int stride, std::uint16_t* q_rot, std::int8_t* cache_k,
                                   std::int8_t* cache_v, float* cache_k_scale,
                                   float* cache_v_scale, const int* d_pt) {
  return granite4_prefill_rope_split_append_int8(qkv, cos_tbl, sin_tbl, base_pos, rows, Hq, Hk, d,
                                                 stride, q_rot, cache_k, cache_v, cache_k_scale,
                                                 cache_v_scale, d_pt);
}

int gpu_multi_rope_append(const std::uint16_t* q, const std::uint16_t* k, const std::uint16_t* v,
                          const float* cos_tbl, const float* sin_tbl, const GpuMultiRows* d_rows,
                          int rows, int Hq, int Hk, int d, int bits, void* cache_k, void* cache_v,
                          float* k_scale, float* v_scale, int stride, std::uint16_t* q_rot) {
  return granite4_gpu_multi_rope_append(q, k, v, cos_tbl, sin_tbl,
                                        reinterpret_cast<const granite4_multi_rows*>(d_rows), rows,
                                        Hq, Hk, d, bits, cache_k, cache_v, k_scale, v_scale, stride,
                                        q_rot);
}

}  // namespace granite4
