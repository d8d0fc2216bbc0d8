// Decode / verify attention over the int8 paged KV pool: the reader of what the
// RoPE + KV-write kernel stores.
//
// Formulation (reference: contract engine/src/attention_gpu.h:15-68, kernel
// engine/src/attention_split.cu; host golden form engine/src/kernel_math.h:265-331):
//   row r of q [rows][Hq d] sits at position pos[r] of its sequence and attends
//   to cache positions 0..pos[r]; cache position t lives in pool row pt[t];
//   k_t = code_k[hkv][pt[t]][:] * k_scale[hkv][pt[t]],  v_t likewise;
//   logits = scale * q . k_t,  p = softmax(logits),  out = sum_t p_t v_t
//   with q head h reading kv head h / 4 (Hq == 4 Hk, d == 128 only, as the
//   reference's split kernel).
// The reference dequantises every cache row to bf16 and rounds logits and
// probabilities to bf16 between its steps; its device tests accept 0.03 absolute
// against that form (engine/tests/test_kernels.cu:2055, :2282). Here the codes stay
// integers: they convert exactly to fp16, the row scale multiplies the logit
// (K) and the probability (V) instead of 128 elements, and nothing is rounded
// below fp16 / f32 on the way - inside the same tolerance, and closer to the
// exact result.
//
// This op is memory-bound: per cache position and kv head it reads 2 x 128 code
// bytes + 2 scales (264 B) for 1024 multiply-adds per query row, more than the
// f32 pipes deliver at HBM speed, so the two contractions run on the tensor
// cores (mma.sync m16n8k16, fp16 in, f32 accumulate).
//
// Decomposition: grid (split, kv head, row group). A CTA has 4 warps and owns a
// contiguous range of cache positions; each warp works alone on tiles of 16
// positions (gathers the 16 K and V code rows through the page table into its
// own shared-memory ring, S^T = K Q^T, online softmax, O^T += V^T P^T) with its
// own running (max, sum, O), so the main loop has no CTA barrier. The warps'
// states are merged in shared memory at the end, the splits' states by a second
// small kernel (flash-decoding).
//
// Algorithmic bytes per (row group, kv head): (pos + 1) * 264.
#include "g4_host.h"
#include "g4_math.cuh"

#include "../../include/granite4_b200.h"

#include <atomic>
#include <cuda_fp16.h>

#include <algorithm>

namespace g4 {
namespace {

constexpr int kAD = 128;       // head dim
constexpr int kTile = 16;      // cache positions per warp tile
constexpr int kWarps = 4;
constexpr int kGqa = 4;        // q heads per kv head
constexpr int kGroupRows = 4;  // query rows of one sequence per CTA (two column tiles of 2 rows x 4 heads)
constexpr int kSplitAlign = kTile * kWarps;
constexpr int kCtasPerSm = 3;  // register budget with two column tiles (groups of three or four rows)
constexpr int kTailStride = 8;  // engine/src/attention_gpu.h:52 (kAttnTailStride): a tree row has at most 8 ancestors

// Shared memory of one warp: kStagesT tiles of raw K and V code rows, filled by 16-byte asynchronous
// copies (cp.async), so the bytes in flight occupy no registers. Rows are padded to 144 bytes: the
// 32-bit K fragment loads of the 32 lanes (8 positions x 4 k-groups) and the eight 16-byte row
// pieces of an ldmatrix then hit different banks. Both mma operands are built from the raw bytes
// in registers; no converted copy of a tile is ever written back to shared memory.
constexpr int kPitch = kAD + 16;          // bytes per raw code row
constexpr int kRawTile = kTile * kPitch;  // 2304

struct AttnParams {
  const uint16_t* q;
  const int8_t* ck;
  const int8_t* cv;
  const float* ks;
  const float* vs;
  const int* row_pos;        // per-row positions, or NULL: row r is at position base + r
  int base_pos;              // base when d_pos is NULL
  const int* d_pos;          // base read on the device, or NULL
  const int* const* row_pt;  // per-row tables, or NULL
  const int* pt;             // one table for every row, or NULL (identity)
  const int* row_grp;        // per-group words r0 | nr << 8, or NULL: groups of group_rows consecutive rows
  const int* row_tbase;      // tree rows: positions above row_tbase[r0] are the row's own ancestors' slots ...
  const int* row_tail;       // ... row_tail[r * kTailStride + (position - tbase - 1)], both or neither
  int window;                // > 0: a row attends to its last `window` positions only
  float* part_o;             // [groups][Hk][splits][16][128]
  float* part_ml;            // [groups][Hk][splits][16][2]
  uint16_t* out;
  int rows, group_rows, Hq, Hk;
  long long stride;
  int splits, split_len, max_len;
  float scale_log2;  // scale * log2(e)
  int early;         // every CTA of the grid is resident at once: the kernel after this one may be staged right away
};

__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// Four int8 codes (one 32-bit word) -> four fp16 values code + 1152, exactly: bias each byte to
// unsigned (code + 128) and drop it into the mantissa of 1024.0 (0x6400). The constant 1152 is not
// subtracted per element (that would cost as much again): a contraction sum_k a_k (c_k + 1152)
// equals sum_k a_k c_k + 1152 sum_k a_k, and sum_k a_k is one number per tile row (the sum of
// the q row, computed once; the sum of the probabilities, which one extra mma against a column
// of ones accumulates). Products of two fp16 values are exact in the f32 accumulator and the
// offset term is ~30 times the signal, so the f32 sum loses under 1e-5 relative to it.
constexpr float kCodeBias = 1152.0f;
__device__ __forceinline__ void codes4_to_half(uint32_t w, uint32_t& lo, uint32_t& hi) {
  w ^= 0x80808080u;
  lo = __byte_perm(w, 0x64646464u, 0x4140);
  hi = __byte_perm(w, 0x64646464u, 0x4342);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, bool real) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  const int src_bytes = real ? 16 : 0;  // 0: nothing is read, the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Merge of the four warps' parked states ([16][128] O, then [16][2] (max, sum), at the start of each
// warp's shared-memory block) into the CTA's result: written out directly when there is one split,
// else as this split's partial state. Called by all 128 threads after a __syncthreads().
__device__ __forceinline__ void merge_warps(const AttnParams& p, const unsigned char* s_dyn, int warp_bytes,
                                            int grp, int hkv, int split, int r0, int nrows) {
  const size_t part = (static_cast<size_t>(grp) * p.Hk + hkv) * p.splits + split;
  for (int m = 0; m < 16; ++m) {
    const int j = m >> 2, hl = m & 3;
    if (j >= nrows) break;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w)
      mm = fmaxf(mm, reinterpret_cast<const float*>(s_dyn + static_cast<size_t>(w) * warp_bytes)[16 * kAD + m * 2]);
    float l = 0.0f, acc = 0.0f;
    const int dim = threadIdx.x;  // 128 threads = 128 dims
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float* base = reinterpret_cast<const float*>(s_dyn + static_cast<size_t>(w) * warp_bytes);
      const float mw = base[16 * kAD + m * 2];
      const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - mm);
      l += f * base[16 * kAD + m * 2 + 1];
      acc += f * base[m * kAD + dim];
    }
    if (p.splits == 1) {
      const float v = l > 0.0f ? acc / l : 0.0f;
      p.out[(static_cast<size_t>(r0 + j) * p.Hq + hkv * kGqa + hl) * kAD + dim] =
          static_cast<uint16_t>(f32_to_bf16_bits(v));
    } else {
      p.part_o[(part * 16 + m) * kAD + dim] = acc;
      if (dim == 0) p.part_ml[(part * 16 + m) * 2] = mm, p.part_ml[(part * 16 + m) * 2 + 1] = l;
    }
  }
}

// ---- the main kernel -----------------------------------------------------------------------------
// A decode step has few query rows per sequence (1 for plain decode, up to 4 for a verify group),
// so the cache positions take the 16-row side of the mma and the (query row, head) pairs the
// 8-column side: S^T = K Q^T (A = 16 positions x dims from the raw K codes, B = the columns of q) and
// O^T = V^T P^T (A = 16 dims x 16 positions from the raw V codes through ldmatrix.trans, B = P^T,
// which is the S^T accumulator transposed by movmatrix). The softmax of a column runs down the
// lanes (three xor shuffles over g). One column tile serves one or two query rows, two tiles
// three or four; the K and V operands are converted once and feed every tile.
// Rows [r0, r0 + nrows) of group `grp`: a row_grp word r0 | nr << 8 when the caller describes the
// groups (engine/src/attention_split.cu:108-113), else group_rows consecutive rows.
__device__ __forceinline__ void group_rows_of(const AttnParams& p, int grp, int cap, int& r0, int& nrows) {
  if (p.row_grp != nullptr) {
    const int w = __ldg(p.row_grp + grp);
    r0 = w & 0xff;
    nrows = max(0, min(min(w >> 8, cap), p.rows - r0));
  } else {
    r0 = grp * p.group_rows;
    nrows = min(p.group_rows, p.rows - r0);
  }
}

constexpr int kStagesT = 3;
constexpr int kWarpSmemT = kStagesT * 2 * kRawTile;  // 13824
constexpr size_t kAttnSmemBytesT = static_cast<size_t>(kWarps) * kWarpSmemT;
constexpr int kCtasPerSmT = 4;
static_assert(kWarpSmemT >= (16 * kAD + 32) * 4, "a warp parks its final state in its own block");

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

// NT column tiles of 8 columns: NT = 1 for groups of one or two query rows (4 CTAs per SM), NT = 2
// for three or four (3 CTAs per SM). Column c = 4 j + hl stands for (query row j, head hl).
// EXT: the launch has a window or tree rows; without it that code is compiled away.
template <int NT, bool EXT>
__global__ void __launch_bounds__(kWarps * 32, NT == 1 ? kCtasPerSmT : kCtasPerSm)
    attn_decode_t_kernel(const AttnParams p) {
  // (a decode-size grid fits the device in one wave, so CTAs of the next kernel that are staged early
  // take nothing from CTAs of this one that are still to start)
  if (p.early) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  pdl_begin();
  extern __shared__ __align__(128) unsigned char s_dyn[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, hkv = blockIdx.y, grp = blockIdx.z;
  int r0, nrows;
  group_rows_of(p, grp, 2 * NT, r0, nrows);
  unsigned char* wsm = s_dyn + static_cast<size_t>(warp) * kWarpSmemT;
  unsigned char* raw_k = wsm;
  unsigned char* raw_v = wsm + kStagesT * kRawTile;

  // As accumulator owner a thread has columns 8 nt + 2 t and 8 nt + 2 t + 1 of every tile nt (both of
  // query row 2 nt + t / 2); as B-operand owner it has column 8 nt + g.
  // A column attends to logical positions [lo_col, pos_col]. Those up to `shared_max` (all of them
  // unless the rows are tree rows) are the same pool rows for every row of the group and are walked
  // as shared tiles; a tree row's positions above its tbase are its own ancestors' slots and come
  // as one extra tile per row after the loop.
  const int base = p.d_pos != nullptr ? __ldg(p.d_pos) : p.base_pos;
  const int tb = (EXT && p.row_tbase != nullptr) ? __ldg(p.row_tbase + r0) : INT_MAX;
  int pos_col[NT], lo_col[NT], pos_max = -1, pos_min = INT_MAX, lo_min = INT_MAX, lo_max = 0;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) pos_col[nt] = -1, lo_col[nt] = 0;
  for (int j = 0; j < nrows; ++j) {
    int pj = p.row_pos != nullptr ? __ldg(p.row_pos + r0 + j) : base + r0 + j;
    pj = pj < 0 ? -1 : min(pj, p.max_len - 1);
    const int lj = (EXT && p.window > 0) ? max(0, pj + 1 - p.window) : 0;
    pos_max = max(pos_max, pj);
    pos_min = min(pos_min, pj);
    lo_min = min(lo_min, lj);
    lo_max = max(lo_max, lj);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
      if (j == 2 * nt + (t >> 1)) pos_col[nt] = pj, lo_col[nt] = lj;
  }
  const int shared_max = min(pos_max, tb);  // last logical position read through the shared tiles
  const int* pt = p.row_pt != nullptr ? p.row_pt[r0] : p.pt;
  // whole 64-position steps below every row's window are skipped
  const int t_begin = split * p.split_len +
                      (EXT ? max(0, (lo_min - split * p.split_len) / (kTile * kWarps)) * (kTile * kWarps) : 0);
  const int t_end = min(split * p.split_len + p.split_len, shared_max + 1);

  // ---- q as the B operand: (dims 16 kk + 4 t .. + 3 of column 8 nt + g), fp16, scaled by a power of two
  uint32_t qb[NT][8][2];
  float logit_scale;
  float q_off[NT][2];  // 1152 x the sum of q over the dims, for the accumulator's columns
  {
    float qf[NT][8][4];
    float qmax = 0.0f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int j = 2 * nt + (g >> 2), hl = g & 3;
      const bool live = j < nrows;
      const uint16_t* qrow = p.q + (static_cast<size_t>(r0 + (live ? j : 0)) * p.Hq + hkv * kGqa + hl) * kAD;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint2 w = live ? __ldg(reinterpret_cast<const uint2*>(qrow + kk * 16 + 4 * t)) : make_uint2(0u, 0u);
        qf[nt][kk][0] = bf16_to_f32(w.x & 0xffffu), qf[nt][kk][1] = bf16_to_f32(w.x >> 16);
        qf[nt][kk][2] = bf16_to_f32(w.y & 0xffffu), qf[nt][kk][3] = bf16_to_f32(w.y >> 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) qmax = fmaxf(qmax, fabsf(qf[nt][kk][i]));
      }
    }
    qmax = warp_max(qmax);
    int qexp = 0;
    if (qmax > 0.0f && qmax < INFINITY)
      qexp = min(max(((__float_as_int(qmax) >> 23) & 0xff) - 127 - 10, -100), 100);
    const float qdown = __int_as_float((127 - qexp) << 23);
    logit_scale = p.scale_log2 * __int_as_float((127 + qexp) << 23);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float sum = 0.0f;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        qb[nt][kk][0] = pack_half2(qf[nt][kk][0] * qdown, qf[nt][kk][1] * qdown);
        qb[nt][kk][1] = pack_half2(qf[nt][kk][2] * qdown, qf[nt][kk][3] * qdown);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&qb[nt][kk][0]));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&qb[nt][kk][1]));
        sum += (a.x + a.y) + (b.x + b.y);
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);  // the whole row of column 8 nt + g, in all four lanes of quad g
      q_off[nt][0] = kCodeBias * __shfl_sync(0xffffffffu, sum, (2 * t) * 4);
      q_off[nt][1] = kCodeBias * __shfl_sync(0xffffffffu, sum, (2 * t + 1) * 4);
    }
  }

  // O^T accumulators: tile nt, block b, rows g / g + 8 = dims 16 b + 2 g / 16 b + 2 g + 1, columns 2 t, 2 t + 1
  float o[NT][8][4];
  float osum[NT][4];
  float m_run[NT][2], l_run[NT][2];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int b = 0; b < 8; ++b) o[nt][b][0] = o[nt][b][1] = o[nt][b][2] = o[nt][b][3] = 0.0f;
    osum[nt][0] = osum[nt][1] = osum[nt][2] = osum[nt][3] = 0.0f;
    m_run[nt][0] = m_run[nt][1] = -INFINITY;
    l_run[nt][0] = l_run[nt][1] = 0.0f;
  }
  const size_t head_row0 = static_cast<size_t>(hkv) * p.stride;

  constexpr int kStep = kTile * kWarps;
  auto table_row = [&](int tile0) -> int {
    const int tpos = tile0 + (lane & 15);
    if (tpos >= t_end) return 0;
    const int prow = pt != nullptr ? __ldg(pt + tpos) : tpos;
    return min(max(prow, 0), static_cast<int>(p.stride) - 1);
  };
  auto gather = [&](int stage, int tile0, int prow, float& sk, float& sv) {
    const int piece = (lane & 7) * 16;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int n = 4 * i + (lane >> 3);
      const int pr = __shfl_sync(0xffffffffu, prow, n);
      const bool have = tile0 + n < t_end;
      const size_t off = (head_row0 + pr) * kAD + piece;
      cp_async16(raw_k + stage * kRawTile + n * kPitch + piece, p.ck + off, have);
      cp_async16(raw_v + stage * kRawTile + n * kPitch + piece, p.cv + off, have);
    }
    cp_async_commit();
    const bool mine = tile0 + (lane & 15) < t_end;
    sk = mine ? __ldg(p.ks + head_row0 + prow) : 0.0f;
    sv = mine ? __ldg(p.vs + head_row0 + prow) : 0.0f;
  };
  const int t_first = t_begin + warp * kTile;
  float sk_q[kStagesT], sv_q[kStagesT];
  {
    const int pr0 = table_row(t_first), pr1 = table_row(t_first + kStep);
    gather(0, t_first, pr0, sk_q[0], sv_q[0]);
    gather(1, t_first + kStep, pr1, sk_q[1], sv_q[1]);
  }
  int prow_next = table_row(t_first + 2 * kStep);
  int stage = 0;

  // One tile of 16 positions (raw code rows at kstage / vstage, their scales in lanes 0-15 of sk_cur /
  // sv_cur) against every column. ok_lo / ok_hi: whether position g / g + 8 of the tile counts for
  // the accumulator columns of tile nt this thread owns; unmasked: every position counts for every
  // column (warp-uniform).
  auto attend = [&](const unsigned char* kstage, const unsigned char* vstage, float sk_cur, float sv_cur,
                    bool unmasked, const bool (&okl)[NT], const bool (&okh)[NT]) {
    // ---- S^T = K Q^T: rows = positions g and g + 8; the K operand is converted once per k-step and
    // serves every column tile
    float sa[NT][4], sb[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) sa[nt][i] = sb[nt][i] = 0.0f;
    const unsigned char* k_lo = kstage + g * kPitch + 4 * t;
    const unsigned char* k_hi = k_lo + 8 * kPitch;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      uint32_t a[4];
      codes4_to_half(*reinterpret_cast<const uint32_t*>(k_lo + kk * 16), a[0], a[2]);
      codes4_to_half(*reinterpret_cast<const uint32_t*>(k_hi + kk * 16), a[1], a[3]);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) mma_f16((kk & 1) ? sb[nt] : sa[nt], a, qb[nt][kk][0], qb[nt][kk][1]);
    }
    // ---- scale, mask, online softmax down the lanes
    const float f_lo = __shfl_sync(0xffffffffu, sk_cur, g) * logit_scale;
    const float f_hi = __shfl_sync(0xffffffffu, sk_cur, g + 8) * logit_scale;
    const float sv_lo = __shfl_sync(0xffffffffu, sv_cur, g), sv_hi = __shfl_sync(0xffffffffu, sv_cur, g + 8);
    uint32_t b0[NT], b1[NT];
    bool rescale = false;
    float corr[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const bool ok_lo = unmasked || okl[nt];
      const bool ok_hi = unmasked || okh[nt];
      float pr[4];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float x_lo = ok_lo ? (sa[nt][e] + sb[nt][e] - q_off[nt][e]) * f_lo : -INFINITY;
        const float x_hi = ok_hi ? (sa[nt][2 + e] + sb[nt][2 + e] - q_off[nt][e]) * f_hi : -INFINITY;
        float mx = fmaxf(x_lo, x_hi);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
        const float m_new = fmaxf(m_run[nt][e], mx);
        corr[nt][e] = (m_new == -INFINITY) ? 1.0f : ex2_approx(m_run[nt][e] - m_new);
        const float base = (m_new == -INFINITY) ? 0.0f : m_new;
        pr[e] = ex2_approx(x_lo - base);      // position g
        pr[2 + e] = ex2_approx(x_hi - base);  // position g + 8
        l_run[nt][e] = l_run[nt][e] * corr[nt][e] + pr[e] + pr[2 + e];  // this lane's two positions
        m_run[nt][e] = m_new;
        rescale |= corr[nt][e] != 1.0f;
      }
      // P^T as the B operand: the accumulator fragments (position g: columns 2 t, 2 t + 1) transposed
      b0[nt] = movmatrix_trans(pack_half2(pr[0] * sv_lo, pr[1] * sv_lo));  // positions 0-7
      b1[nt] = movmatrix_trans(pack_half2(pr[2] * sv_hi, pr[3] * sv_hi));  // positions 8-15
    }
    if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          o[nt][b][0] *= corr[nt][0], o[nt][b][1] *= corr[nt][1];
          o[nt][b][2] *= corr[nt][0], o[nt][b][3] *= corr[nt][1];
        }
        osum[nt][0] *= corr[nt][0], osum[nt][1] *= corr[nt][1];
        osum[nt][2] *= corr[nt][0], osum[nt][3] *= corr[nt][1];
      }
    }
    // ---- O^T += V^T P^T. V operand straight from the raw bytes: the tile is read as 16-bit elements
    // (two adjacent dims of one position), transposed by ldmatrix; a register then holds positions
    // 2 t, 2 t + 1 for dims 2 g and 2 g + 1 of a 16-dim block, and one byte permute each picks the
    // (position pair, dim) halves, already in fp16 form (code + 1152). Converted once per block, used
    // by every column tile.
#pragma unroll
    for (int blk = 0; blk < 8; blk += 2) {
      // matrices: (pos 0-7, block blk), (pos 8-15, block blk), (pos 0-7, block blk + 1), (pos 8-15, ..)
      uint32_t r[4];
      ldmatrix_x4_trans(r, vstage + (lane & 15) * kPitch + (blk + (lane >> 4)) * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) r[i] ^= 0x80808080u;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t lo = r[2 * u], hi = r[2 * u + 1];
        // rows g / g + 8 = dims 2 g / 2 g + 1 of the block; k = positions 2 t, 2 t + 1 | 2 t + 8, 2 t + 9
        const uint32_t a[4] = {__byte_perm(lo, 0x64646464u, 0x4240), __byte_perm(lo, 0x64646464u, 0x4341),
                               __byte_perm(hi, 0x64646464u, 0x4240), __byte_perm(hi, 0x64646464u, 0x4341)};
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) mma_f16(o[nt][blk + u], a, b0[nt], b1[nt]);
      }
    }
    const uint32_t ones[4] = {0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_f16(osum[nt], ones, b0[nt], b1[nt]);  // sum over the positions of P^T's columns
  };

  for (int t0 = t_first; t0 < t_end; t0 += kStep) {
    cp_async_wait<kStagesT - 2>();
    __syncwarp();
    gather((stage + kStagesT - 1) % kStagesT, t0 + (kStagesT - 1) * kStep, prow_next, sk_q[kStagesT - 1],
           sv_q[kStagesT - 1]);
    prow_next = table_row(t0 + kStagesT * kStep);
    const float sk_cur = sk_q[0], sv_cur = sv_q[0];
#pragma unroll
    for (int i = 0; i + 1 < kStagesT; ++i) sk_q[i] = sk_q[i + 1], sv_q[i] = sv_q[i + 1];
    const unsigned char* kstage = raw_k + stage * kRawTile;
    const unsigned char* vstage = raw_v + stage * kRawTile;
    stage = (stage + 1) % kStagesT;
    const bool unmasked = t0 + kTile <= t_end && t0 + kTile - 1 <= pos_min && (!EXT || t0 >= lo_max);  // warp-uniform
    bool okl[NT], okh[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      okl[nt] = t0 + g <= pos_col[nt] && (!EXT || t0 + g >= lo_col[nt]) && t0 + g < t_end;
      okh[nt] = t0 + g + 8 <= pos_col[nt] && (!EXT || t0 + g + 8 >= lo_col[nt]) && t0 + g + 8 < t_end;
    }
    attend(kstage, vstage, sk_cur, sv_cur, unmasked, okl, okh);
  }

  cp_async_wait<0>();
  __syncwarp();
  // Tree rows: row j's positions tbase + 1 .. pos_j are the slots of its own ancestors (at most
  // kTailStride of them). They form one more tile that only row j's columns attend to; warp j of
  // the first split's CTA takes it (a group has at most four rows, a CTA four warps).
  if (EXT && p.row_tail != nullptr && split == 0 && warp < nrows) {
    const int j = warp;
    int pj = __ldg(p.row_pos + r0 + j);
    pj = pj < 0 ? -1 : min(pj, p.max_len - 1);
    const int cnt = min(max(pj - tb, 0), kTailStride);
    if (cnt > 0) {
      const int n = lane & 15;
      int prow = 0;
      if (n < cnt) {
        const int slot = __ldg(p.row_tail + static_cast<size_t>(r0 + j) * kTailStride + n);
        prow = pt != nullptr ? __ldg(pt + slot) : slot;
        prow = min(max(prow, 0), static_cast<int>(p.stride) - 1);
      }
      const int piece = (lane & 7) * 16;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int nn = 4 * i + (lane >> 3);
        const int pr = __shfl_sync(0xffffffffu, prow, nn);
        const size_t off = (head_row0 + pr) * kAD + piece;
        cp_async16(raw_k + nn * kPitch + piece, p.ck + off, nn < cnt);
        cp_async16(raw_v + nn * kPitch + piece, p.cv + off, nn < cnt);
      }
      cp_async_commit();
      const float sk_t = n < cnt ? __ldg(p.ks + head_row0 + prow) : 0.0f;
      const float sv_t = n < cnt ? __ldg(p.vs + head_row0 + prow) : 0.0f;
      cp_async_wait<0>();
      __syncwarp();
      bool okl[NT], okh[NT];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        okl[nt] = j == 2 * nt + (t >> 1) && g < cnt && (EXT ? tb : 0) + 1 + g >= lo_col[nt];
        okh[nt] = false;
      }
      attend(raw_k, raw_v, sk_t, sv_t, false, okl, okh);
      __syncwarp();
    }
  }
  float* wo = reinterpret_cast<float*>(wsm);  // [16][128]; only the rows of live columns are read
  float* wml = wo + 16 * kAD;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      l_run[nt][e] += __shfl_xor_sync(0xffffffffu, l_run[nt][e], 4);
      l_run[nt][e] += __shfl_xor_sync(0xffffffffu, l_run[nt][e], 8);
      l_run[nt][e] += __shfl_xor_sync(0xffffffffu, l_run[nt][e], 16);
    }
    const int c0 = 8 * nt + 2 * t;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      // take the code offset out: O = O_mma - 1152 * sum(p)
      *reinterpret_cast<float2*>(wo + c0 * kAD + b * 16 + 2 * g) =
          make_float2(o[nt][b][0] - kCodeBias * osum[nt][0], o[nt][b][2] - kCodeBias * osum[nt][0]);
      *reinterpret_cast<float2*>(wo + (c0 + 1) * kAD + b * 16 + 2 * g) =
          make_float2(o[nt][b][1] - kCodeBias * osum[nt][1], o[nt][b][3] - kCodeBias * osum[nt][1]);
    }
    if (g == 0) {
      wml[c0 * 2] = m_run[nt][0], wml[c0 * 2 + 1] = l_run[nt][0];
      wml[(c0 + 1) * 2] = m_run[nt][1], wml[(c0 + 1) * 2 + 1] = l_run[nt][1];
    }
  }
  __syncthreads();
  merge_warps(p, s_dyn, kWarpSmemT, grp, hkv, split, r0, nrows);
}

// Merge of the splits: one CTA per (kv head, row group, tile row), thread = dim. The splits'
// weights exp2(m_s - M) are computed once into shared memory, then every thread sums its dim.
constexpr int kMaxSplits = 512;
__global__ void __launch_bounds__(kAD) attn_combine_kernel(const AttnParams p) {
  pdl_begin();
  const int hkv = blockIdx.x, grp = blockIdx.y, m = blockIdx.z, dim = threadIdx.x;
  int r0, nrows;
  group_rows_of(p, grp, kGroupRows, r0, nrows);
  if (m >= 4 * nrows) return;
  const int j = m >> 2, hl = m & 3;
  const size_t part0 = (static_cast<size_t>(grp) * p.Hk + hkv) * p.splits;
  __shared__ float s_w[kMaxSplits];
  __shared__ float s_red[2][kAD / 32];
  float mm = -INFINITY;
  for (int s = dim; s < p.splits; s += kAD) mm = fmaxf(mm, __ldcg(p.part_ml + ((part0 + s) * 16 + m) * 2));
  mm = warp_max(mm);
  if ((dim & 31) == 0) s_red[0][dim >> 5] = mm;
  __syncthreads();
  mm = fmaxf(fmaxf(s_red[0][0], s_red[0][1]), fmaxf(s_red[0][2], s_red[0][3]));
  float l = 0.0f;
  for (int s = dim; s < p.splits; s += kAD) {
    const float ms = __ldcg(p.part_ml + ((part0 + s) * 16 + m) * 2);
    const float f = (ms == -INFINITY) ? 0.0f : exp2f(ms - mm);
    s_w[s] = f;
    l += f * __ldcg(p.part_ml + ((part0 + s) * 16 + m) * 2 + 1);
  }
  l = warp_sum(l);
  if ((dim & 31) == 0) s_red[1][dim >> 5] = l;
  __syncthreads();
  l = (s_red[1][0] + s_red[1][1]) + (s_red[1][2] + s_red[1][3]);
  // each warp sums a quarter of the splits for all 128 dims (lane = four dims), eight loads in
  // flight per lane; the four partial sums meet in shared memory
  __shared__ float4 s_acc[kAD / 32][32];
  const int warp = dim >> 5, lane = dim & 31;
  const float4* po = reinterpret_cast<const float4*>(p.part_o + (part0 * 16 + m) * kAD) + lane;
  const size_t split_pitch4 = static_cast<size_t>(16) * kAD / 4;
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  int s = warp;
  for (; s + 7 * (kAD / 32) < p.splits; s += 8 * (kAD / 32)) {
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = __ldcg(po + (s + u * (kAD / 32)) * split_pitch4);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const float w = s_w[s + u * (kAD / 32)];
      acc.x += w * v[u].x, acc.y += w * v[u].y, acc.z += w * v[u].z, acc.w += w * v[u].w;
    }
  }
  for (; s < p.splits; s += kAD / 32) {
    const float4 v = __ldcg(po + s * split_pitch4);
    const float w = s_w[s];
    acc.x += w * v.x, acc.y += w * v.y, acc.z += w * v.z, acc.w += w * v.w;
  }
  s_acc[warp][lane] = acc;
  __syncthreads();
  if (warp == 0) {
    float4 t = s_acc[0][lane];
#pragma unroll
    for (int w = 1; w < kAD / 32; ++w) {
      const float4 o = s_acc[w][lane];
      t.x += o.x, t.y += o.y, t.z += o.z, t.w += o.w;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    uint16_t* dst = p.out + (static_cast<size_t>(r0 + j) * p.Hq + hkv * kGqa + hl) * kAD + lane * 4;
    const uint32_t lo = f32_to_bf16_bits(t.x * inv) | (f32_to_bf16_bits(t.y * inv) << 16);
    const uint32_t hi = f32_to_bf16_bits(t.z * inv) | (f32_to_bf16_bits(t.w * inv) << 16);
    *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
  }
}

struct SplitPlan {
  int groups, splits, split_len;
};

SplitPlan plan_splits_for_groups(int groups, int group_rows, int Hk, int max_len) {
  const int ctas_per_sm = group_rows <= 2 ? kCtasPerSmT : kCtasPerSm;
  SplitPlan s{};
  s.groups = groups;
  const int tiles = (max_len + kSplitAlign - 1) / kSplitAlign;  // units of 64 positions
  // aim at one resident wave over the whole launch, at least 64 positions per split
  const long long ctas_wanted = static_cast<long long>(ctas_per_sm) * sm_count();
  // rounded down: the launch is then at most one resident wave (a second, nearly empty wave would
  // double the time)
  long long splits = ctas_wanted / (static_cast<long long>(s.groups) * Hk);
  splits = std::max<long long>(1, std::min<long long>(std::min<long long>(splits, tiles), kMaxSplits));
  const int tiles_per_split = static_cast<int>((tiles + splits - 1) / splits);
  s.split_len = tiles_per_split * kSplitAlign;
  s.splits = (tiles + tiles_per_split - 1) / tiles_per_split;
  return s;
}

SplitPlan plan_splits(int rows, int group_rows, int Hk, int max_len) {
  return plan_splits_for_groups((rows + group_rows - 1) / group_rows, group_rows, Hk, max_len);
}

// Partial states of every (group, kv head, split): [16][128] O and [16][2] (max, sum), f32.
long long scratch_bytes_of(const SplitPlan& s, int Hk) {
  return static_cast<long long>(s.groups) * Hk * s.splits * 16 * (kAD + 2) * static_cast<long long>(sizeof(float));
}

}  // namespace
}  // namespace g4

extern "C" long long granite4_attn_decode_scratch_bytes(int rows, int rows_per_group, int Hk, int max_len);

namespace g4 {
// csrc/attn_prefill.cu
int attn_prefill_flash(const char* fn, const uint16_t* d_q, float scale, int Hq, int Hk, int base_pos, int rows,
                       int stride, uint16_t* d_out, const int8_t* d_ck, const int8_t* d_cv, const float* d_ks,
                       const float* d_vs, const int* d_pt);
}  // namespace g4

namespace g4 {
// Everything the launch needs beyond the caches: the reference's attn_split arguments
// (engine/src/attention_gpu.h:39-68) that select where each row sits and what it may see.
struct AttnRows {
  const int* d_row_pos = nullptr;        // per-row positions; NULL: row r is at base + r
  int base_pos = 0;                      // base when d_pos is NULL
  const int* d_pos = nullptr;            // base read on the device
  const int* const* d_row_pt = nullptr;  // per-row (per-group) tables
  const int* d_pt = nullptr;             // one table for every row
  const int* d_row_grp = nullptr;        // group words r0 | nr << 8 ...
  int ngroups = 0;                       // ... and how many
  const int* d_row_tbase = nullptr;      // tree rows
  const int* d_row_tail = nullptr;
  int window = 0;
};

// Validation, split plan and launches shared by the entry points.
// single_split_without_scratch: a caller that has no scratch to give (the reference's
// prefill signature) gets one split over the whole range instead of an error.
int attn_launch(const char* fn, const uint16_t* d_q, const int8_t* d_cache_k, const int8_t* d_cache_v,
                const float* d_k_scale, const float* d_v_scale, const AttnRows& r, int rows, int rows_per_group,
                int Hq, int Hk, int d, int stride, int max_len, float scale, void* d_scratch, long long scratch_bytes,
                uint16_t* d_out, bool single_split_without_scratch) {
  if (d_q == nullptr || d_cache_k == nullptr || d_cache_v == nullptr || d_k_scale == nullptr ||
      d_v_scale == nullptr || d_out == nullptr || rows <= 0 ||
      rows_per_group <= 0 || rows_per_group > kGroupRows || stride <= 0 || max_len <= 0 ||
      max_len > stride || !std::isfinite(scale) || r.window < 0)
    return fail(fn, "invalid arguments");
  // the reference's own argument rules (engine/src/attention_split.cu:1098-1105)
  if ((r.d_row_grp != nullptr && (r.d_row_pos == nullptr || r.ngroups <= 0 || r.ngroups > rows || rows > 256)) ||
      ((r.d_row_tbase != nullptr) != (r.d_row_tail != nullptr)) || (r.d_row_tbase != nullptr && r.d_row_pos == nullptr))
    return fail(fn, "row groups and tree rows need per-row positions; tbase and tail come together");
  if (d != kAD || Hk <= 0 || Hq != kGqa * Hk) return -1;  // engine/src/attention_gpu.h:18-19
  if (!aligned16(d_cache_k) || !aligned16(d_cache_v) || !aligned16(d_q))
    return fail(fn, "q and the caches must be 16-byte aligned");
  SplitPlan s = plan_splits(rows, rows_per_group, Hk, max_len);
  if (r.d_row_grp != nullptr) s = plan_splits_for_groups(r.ngroups, rows_per_group, Hk, max_len);
  const long long need = scratch_bytes_of(s, Hk);
  if (s.splits > 1 && single_split_without_scratch && (d_scratch == nullptr || scratch_bytes < need)) {
    s.splits = 1;
    s.split_len = (max_len + kSplitAlign - 1) / kSplitAlign * kSplitAlign;
  }
  if (s.groups > 65535) return fail(fn, "too many row groups");
  AttnParams p{};
  p.q = d_q, p.ck = d_cache_k, p.cv = d_cache_v, p.ks = d_k_scale, p.vs = d_v_scale;
  p.row_pos = r.d_row_pos, p.base_pos = r.base_pos, p.d_pos = r.d_pos, p.row_pt = r.d_row_pt, p.pt = r.d_pt;
  p.row_grp = r.d_row_grp, p.row_tbase = r.d_row_tbase, p.row_tail = r.d_row_tail, p.window = r.window;
  p.out = d_out;
  p.rows = rows, p.group_rows = rows_per_group, p.Hq = Hq, p.Hk = Hk, p.stride = stride;
  p.splits = s.splits, p.split_len = s.split_len, p.max_len = max_len;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (s.splits > 1) {
    if (d_scratch == nullptr || scratch_bytes < need || !aligned16(d_scratch))
      return fail(fn, "scratch missing or smaller than the size the scratch query returns");
    p.part_o = static_cast<float*>(d_scratch);
    p.part_ml = p.part_o + static_cast<size_t>(s.groups) * Hk * s.splits * 16 * kAD;
  }
  cudaStream_t st = current_stream();
  {
    static std::atomic<bool> attr_set[64];  // per device; relaxed: setting the attribute twice is harmless
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(fn, "cannot identify the current device");
    if (dev >= 0 && dev < 64 && !attr_set[dev].load(std::memory_order_relaxed)) {
      const int bytes = static_cast<int>(kAttnSmemBytesT);
      G4_CUDA_TRY(fn, cudaFuncSetAttribute(attn_decode_t_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
      G4_CUDA_TRY(fn, cudaFuncSetAttribute(attn_decode_t_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
      G4_CUDA_TRY(fn, cudaFuncSetAttribute(attn_decode_t_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
      G4_CUDA_TRY(fn, cudaFuncSetAttribute(attn_decode_t_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
      attr_set[dev].store(true, std::memory_order_relaxed);
    }
  }
  const dim3 grid(static_cast<unsigned>(s.splits), static_cast<unsigned>(Hk), static_cast<unsigned>(s.groups));
  p.early = static_cast<long long>(s.splits) * Hk * s.groups <= 3ll * sm_count() ? 1 : 0;
  const bool ext = r.window > 0 || r.d_row_tail != nullptr;
  if (rows_per_group <= 2) {
    if (ext) G4_LAUNCH_PDL(fn, (attn_decode_t_kernel<1, true>), grid, dim3(kWarps * 32), kAttnSmemBytesT, st, p);
    else G4_LAUNCH_PDL(fn, (attn_decode_t_kernel<1, false>), grid, dim3(kWarps * 32), kAttnSmemBytesT, st, p);
  } else {
    if (ext) G4_LAUNCH_PDL(fn, (attn_decode_t_kernel<2, true>), grid, dim3(kWarps * 32), kAttnSmemBytesT, st, p);
    else G4_LAUNCH_PDL(fn, (attn_decode_t_kernel<2, false>), grid, dim3(kWarps * 32), kAttnSmemBytesT, st, p);
  }
  if (s.splits > 1)
    G4_LAUNCH_PDL(fn, attn_combine_kernel,
                  dim3(static_cast<unsigned>(Hk), static_cast<unsigned>(s.groups), 4u * rows_per_group),
                  dim3(kAD), 0, st, p);
  return 0;
}

}  // namespace g4

extern "C" {

long long granite4_attn_decode_scratch_bytes(int rows, int rows_per_group, int Hk, int max_len) {
  if (rows <= 0 || rows_per_group <= 0 || rows_per_group > g4::kGroupRows || Hk <= 0 || max_len <= 0)
    return -1;
  return g4::scratch_bytes_of(g4::plan_splits(rows, rows_per_group, Hk, max_len), Hk);
}

int granite4_kernel_attn_decode_int8_paged(const uint16_t* d_q, const int8_t* d_cache_k,
                                           const int8_t* d_cache_v, const float* d_k_scale,
                                           const float* d_v_scale, const int* d_row_pos,
                                           const int* const* d_row_pt, const int* d_pt, int rows,
                                           int rows_per_group, int Hq, int Hk, int d, int stride,
                                           int max_len, float scale, void* d_scratch,
                                           long long scratch_bytes, uint16_t* d_out) {
  const char* fn = "granite4_kernel_attn_decode_int8_paged";
  if (d_row_pos == nullptr) return g4::fail(fn, "invalid arguments");
  g4::AttnRows r;
  r.d_row_pos = d_row_pos, r.d_row_pt = d_row_pt, r.d_pt = d_pt;
  return g4::attn_launch(fn, d_q, d_cache_k, d_cache_v, d_k_scale, d_v_scale, r, rows, rows_per_group, Hq, Hk, d,
                         stride, max_len, scale, d_scratch, scratch_bytes, d_out, false);
}

// Upper bound over every way the rows may be grouped (one group of up to four consecutive rows
// per sequence, or one group per row), so that a caller can size the scratch before it knows the
// grouping, as with the reference's attn_split_scratch_bytes(Hq, rows, stride).
long long granite4_attn_split_scratch_bytes(int Hq, int rows, int max_len) {
  if (Hq <= 0 || Hq % g4::kGqa != 0 || rows <= 0 || max_len <= 0) return -1;
  const int Hk = Hq / g4::kGqa;
  long long need = 0;
  for (int groups = 1; groups <= rows; ++groups)
    for (int per = 1; per <= g4::kGroupRows; per += 2)  // the two kernel forms plan differently
      need = std::max(need, g4::scratch_bytes_of(g4::plan_splits_for_groups(groups, per == 1 ? 1 : g4::kGroupRows, Hk, max_len), Hk));
  return need;
}

int granite4_attn_split_int8(const uint16_t* d_q, const int8_t* d_cache_k8, const int8_t* d_cache_v8,
                             const float* d_k_scale, const float* d_v_scale, float scale, int Hq, int Hk, int d,
                             int kv_base, const int* d_pos, int rows, int stride, void* d_scratch,
                             long long scratch_bytes, uint16_t* d_out, const int* d_pt, int max_len,
                             const int* d_row_pos, const int* const* d_row_pt, const int* d_row_grp, int ngroups,
                             const int* d_row_tbase, const int* d_row_tail, int window) {
  const char* fn = "granite4_attn_split_int8";
  const int ml = max_len > 0 ? max_len : stride;
  // engine/src/attention_split.cu:1096-1105
  if (rows <= 0 || rows > GRANITE4_MAX_VERIFY_ROWS || stride <= 0 || ml > stride ||
      (d_pos == nullptr && d_row_pos == nullptr && (kv_base < 0 || kv_base + rows > ml)) ||
      ((d_row_pos == nullptr) != (d_row_pt == nullptr)))
    return g4::fail(fn, "invalid arguments");
  g4::AttnRows r;
  r.d_row_pos = d_row_pos, r.base_pos = kv_base, r.d_pos = d_pos, r.d_row_pt = d_row_pt, r.d_pt = d_pt;
  r.d_row_grp = d_row_grp, r.ngroups = ngroups, r.d_row_tbase = d_row_tbase, r.d_row_tail = d_row_tail;
  r.window = window;
  // rows of one sequence at consecutive positions share tiles in groups of four; rows that are
  // sequences of their own are one group each unless the caller's group words say otherwise
  const int per_group = (d_row_pos == nullptr || d_row_grp != nullptr) ? g4::kGroupRows : 1;
  return g4::attn_launch(fn, d_q, d_cache_k8, d_cache_v8, d_k_scale, d_v_scale, r, rows, per_group, Hq, Hk, d, stride,
                         ml, scale, d_scratch, scratch_bytes, d_out, false);
}

int granite4_prefill_attention_int8(const uint16_t* d_q_rot, float scale, int Hq, int Hk, int d, int base_pos,
                                    int rows, int stride, uint16_t* d_out, const int8_t* d_cache_k8,
                                    const int8_t* d_cache_v8, const float* d_k_scale, const float* d_v_scale,
                                    const int* d_pt, void* d_scratch, long long scratch_bytes) {
  const char* fn = "granite4_prefill_attention_int8";
  if (base_pos < 0 || rows <= 0 || base_pos > INT_MAX - rows) return g4::fail(fn, "invalid arguments");
  // A chunk of 32 rows or more takes the flash form (one K / V tile serves 16 positions x 4 heads);
  // shorter ones the decode kernel as groups of four rows, which can also split a long context
  // over CTAs. G4_PREFILL_FLASH=0 keeps every chunk on the decode kernel.
  const char* flash_env = std::getenv("G4_PREFILL_FLASH");
  if (rows >= 32 && !(flash_env != nullptr && flash_env[0] == '0')) {
    if (d_q_rot == nullptr || d_cache_k8 == nullptr || d_cache_v8 == nullptr || d_k_scale == nullptr ||
        d_v_scale == nullptr || d_out == nullptr || stride <= 0 || base_pos + rows > stride || !std::isfinite(scale))
      return g4::fail(fn, "invalid arguments");
    if (d != g4::kAD || Hk <= 0 || Hq != g4::kGqa * Hk) return -1;  // engine/src/attention_gpu.h:18-19
    if (!g4::aligned16(d_cache_k8) || !g4::aligned16(d_cache_v8) || !g4::aligned16(d_q_rot))
      return g4::fail(fn, "q and the caches must be 16-byte aligned");
    return g4::attn_prefill_flash(fn, d_q_rot, scale, Hq, Hk, base_pos, rows, stride, d_out, d_cache_k8, d_cache_v8,
                                  d_k_scale, d_v_scale, d_pt);
  }
  g4::AttnRows r;
  r.base_pos = base_pos, r.d_pt = d_pt;
  return g4::attn_launch(fn, d_q_rot, d_cache_k8, d_cache_v8, d_k_scale, d_v_scale, r, rows, g4::kGroupRows, Hq, Hk, d,
                         stride, base_pos + rows, scale, d_scratch, scratch_bytes, d_out, true);
}

}  // extern "C"

// The reference's C++ entry point (engine/src/prefill_gemm.h:86-101), same mangled name. Only the
// int8 cache is built; the other formats and the sliding window return -1, which the reference's
// caller treats as "take the other attention path" (engine/src/forward_gpu.cu:2800-2830).
namespace granite4 {
int prefill_attention(const std::uint16_t* q_rot, const std::uint16_t* cache_k, const std::uint16_t* cache_v,
                      float scale, int Hq, int Hk, int d, int base_pos, int rows, int stride, std::uint16_t* out,
                      const std::int8_t* cache_k8, const std::int8_t* cache_v8, const float* k_scale,
                      const float* v_scale, bool int8, const std::uint8_t* cache_k4, const std::uint8_t* cache_v4,
                      bool int4, const int* d_pt, bool k5, int window) {
  (void)cache_k, (void)cache_v, (void)cache_k4, (void)cache_v4;
  if (!int8 || int4 || k5 || window > 0) return -1;
  return granite4_prefill_attention_int8(q_rot, scale, Hq, Hk, d, base_pos, rows, stride, out, cache_k8, cache_v8,
                                         k_scale, v_scale, d_pt, nullptr, 0);
}
}  // namespace granite4

// The reference's split-KV entry points (engine/src/attention_gpu.h:13, :53-66), same mangled names.
// Only the int8 cache is built: the bf16, int4 and K5 forms return -1, which the reference's callers
// treat as "take the other attention path".
namespace granite4 {
std::size_t attn_split_scratch_bytes(int Hq, int rows, int stride) {
  const long long n = granite4_attn_split_scratch_bytes(Hq, rows, stride);
  return n < 0 ? 0 : static_cast<std::size_t>(n);
}
int attn_split(const std::uint16_t* q, const std::uint16_t* cache_k, const std::uint16_t* cache_v, float scale, int Hq,
               int Hk, int d, int kv_base, const int* d_pos, int rows, int stride, void* scratch, std::uint16_t* out,
               const std::int8_t* cache_k8, const std::int8_t* cache_v8, const float* cache_k_scale,
               const float* cache_v_scale, bool int8, const std::uint8_t* cache_k4, const std::uint8_t* cache_v4,
               bool int4, const int* d_pt, int max_len, const int* row_pos, const int* const* row_pt,
               const int* row_grp, int ngroups, const int* row_tbase, const int* row_tail, int kv_hint, bool k5,
               int window) {
  (void)cache_k, (void)cache_v, (void)cache_k4, (void)cache_v4, (void)kv_hint;
  if (!int8 || int4 || k5 || scratch == nullptr) return -1;
  // the reference's callers size the scratch with attn_split_scratch_bytes(Hq, rows, stride)
  const long long have = granite4_attn_split_scratch_bytes(Hq, rows, stride);
  return granite4_attn_split_int8(q, cache_k8, cache_v8, cache_k_scale, cache_v_scale, scale, Hq, Hk, d, kv_base, d_pos,
                                  rows, stride, scratch, have, out, d_pt, max_len, row_pos, row_pt, row_grp, ngroups,
                                  row_tbase, row_tail, window);
}
}  // namespace granite4
