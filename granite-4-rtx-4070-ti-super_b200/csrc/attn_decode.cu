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
// bytes + 2 scales (264 B) for 1024 multiply-adds, more than the f32 pipes
// deliver at HBM speed, so the two contractions run on the tensor cores
// (mma.sync m16n8k16, fp16 in, f32 accumulate; the 16 rows of the tile are the 4
// q heads of the kv head x up to 4 query rows of one sequence).
//
// Decomposition: grid (split, kv head, row group). A CTA has 4 warps and owns a
// contiguous range of cache positions; each warp works alone on tiles of 16
// positions (gathers the 16 K and V code rows through the page table, converts
// them into its own shared-memory tile, S = Q K^T, online softmax, O += P V) with
// its own running (max, sum, O), so the main loop has no CTA barrier. The warps'
// states are merged in shared memory at the end, the splits' states by a second
// small kernel (flash-decoding).
//
// Algorithmic bytes per (row group, kv head): (pos + 1) * 264.
#include "g4_host.h"
#include "g4_math.cuh"

#include "../../include/granite4_b200.h"

#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

namespace g4 {
namespace {

constexpr int kAD = 128;       // head dim
constexpr int kTile = 16;      // cache positions per warp tile
constexpr int kWarps = 4;
constexpr int kGqa = 4;        // q heads per kv head
constexpr int kGroupRows = 4;  // query rows per CTA (4 x 4 = the 16 rows of the mma tile)
constexpr int kSplitAlign = kTile * kWarps;
constexpr int kCtasPerSm = 3;  // register and shared-memory budget of the main kernel

// Shared memory of one warp: kStages tiles of raw K and V code rows, filled by 16-byte asynchronous
// copies (cp.async), so the bytes in flight occupy no registers. Rows are padded to 144 bytes: the
// 32-bit K fragment loads of the 32 lanes (8 positions x 4 k-groups) and the eight 16-byte row
// pieces of an ldmatrix then hit different banks. Both mma operands are built from the raw bytes
// in registers; no converted copy of a tile is ever written back to shared memory.
constexpr int kStages = 4;
constexpr int kPitch = kAD + 16;          // bytes per raw code row
constexpr int kRawTile = kTile * kPitch;  // 2304
constexpr int kWarpSmem = kStages * 2 * kRawTile;  // 18432
constexpr size_t kAttnSmemBytes = static_cast<size_t>(kWarps) * kWarpSmem;
static_assert(kWarpSmem >= (16 * kAD + 32) * 4, "a warp parks its final state in its own block");

struct AttnParams {
  const uint16_t* q;
  const int8_t* ck;
  const int8_t* cv;
  const float* ks;
  const float* vs;
  const int* row_pos;
  const int* const* row_pt;  // per-row tables, or NULL
  const int* pt;             // one table for every row, or NULL (identity)
  float* part_o;             // [groups][Hk][splits][16][128]
  float* part_ml;            // [groups][Hk][splits][16][2]
  uint16_t* out;
  int rows, group_rows, Hq, Hk;
  long long stride;
  int splits, split_len, max_len;
  float scale_log2;  // scale * log2(e)
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

__global__ void __launch_bounds__(kWarps * 32, kCtasPerSm) attn_decode_kernel(const AttnParams p) {
  pdl_begin();
  extern __shared__ __align__(128) unsigned char s_dyn[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, hkv = blockIdx.y, grp = blockIdx.z;
  const int r0 = grp * p.group_rows;
  const int nrows = min(p.group_rows, p.rows - r0);
  unsigned char* wsm = s_dyn + static_cast<size_t>(warp) * kWarpSmem;
  unsigned char* raw_k = wsm;                       // [kStages][16][144]
  unsigned char* raw_v = wsm + kStages * kRawTile;  // [kStages][16][144]

  // positions of the group's rows; the mma rows g and g + 8 belong to query rows g / 4 and 2 + g / 4
  int pos_lo = -1, pos_hi = -1, pos_max = -1;
  for (int j = 0; j < nrows; ++j) {
    int pj = __ldg(p.row_pos + r0 + j);
    pj = pj < 0 ? -1 : min(pj, p.max_len - 1);
    pos_max = max(pos_max, pj);
    if (j == (g >> 2)) pos_lo = pj;
    if (j == 2 + (g >> 2)) pos_hi = pj;
  }
  const int* pt = p.row_pt != nullptr ? p.row_pt[r0] : p.pt;
  const int t_begin = split * p.split_len;
  const int t_end = min(t_begin + p.split_len, pos_max + 1);

  // ---- Q fragments: 16 rows (query row j = m / 4, head hl = m % 4) x 128 dims, as fp16 scaled by
  // a power of two so that the largest magnitude sits near 2^10. Within each 16-wide k-step the
  // contraction index is permuted: lane group t takes dims 4 t .. 4 t + 3 (first operand register
  // 4 t, 4 t + 1, second 4 t + 2, 4 t + 3) instead of 2 t, 2 t + 1 and 2 t + 8, 2 t + 9. A dot product
  // does not care about the order, and the matching K operand is then four consecutive code
  // bytes: one 32-bit shared-memory load per mma.
  uint32_t qa[8][4];
  float logit_scale;
  float q_off[2];  // rows g and g + 8
  {
    float qf[8][8];  // per k-step: row g dims 4t, 4t+1 | row g+8 same | row g dims 4t+2, 4t+3 | row g+8 same
    float qmax = 0.0f;
#pragma unroll
    for (int half_rows = 0; half_rows < 2; ++half_rows) {
      const int m = g + 8 * half_rows;
      const int j = m >> 2, hl = m & 3;
      const bool live = j < nrows;
      const uint16_t* qrow = p.q + (static_cast<size_t>(r0 + (live ? j : 0)) * p.Hq + hkv * kGqa + hl) * kAD;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint2 w = live ? __ldg(reinterpret_cast<const uint2*>(qrow + kk * 16 + 4 * t)) : make_uint2(0u, 0u);
        const float d0 = bf16_to_f32(w.x & 0xffffu), d1 = bf16_to_f32(w.x >> 16);
        const float d2 = bf16_to_f32(w.y & 0xffffu), d3 = bf16_to_f32(w.y >> 16);
        qf[kk][half_rows * 2 + 0] = d0, qf[kk][half_rows * 2 + 1] = d1;
        qf[kk][4 + half_rows * 2 + 0] = d2, qf[kk][4 + half_rows * 2 + 1] = d3;
        qmax = fmaxf(qmax, fmaxf(fmaxf(fabsf(d0), fabsf(d1)), fmaxf(fabsf(d2), fabsf(d3))));
      }
    }
    qmax = warp_max(qmax);
    int qexp = 0;
    if (qmax > 0.0f && qmax < INFINITY)
      qexp = min(max(((__float_as_int(qmax) >> 23) & 0xff) - 127 - 10, -100), 100);
    const float qdown = __int_as_float((127 - qexp) << 23);  // 2^-qexp
    logit_scale = p.scale_log2 * __int_as_float((127 + qexp) << 23);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      // operand registers: (row g, k lo), (row g + 8, k lo), (row g, k hi), (row g + 8, k hi)
      qa[kk][0] = pack_half2(qf[kk][0] * qdown, qf[kk][1] * qdown);
      qa[kk][1] = pack_half2(qf[kk][2] * qdown, qf[kk][3] * qdown);
      qa[kk][2] = pack_half2(qf[kk][4] * qdown, qf[kk][5] * qdown);
      qa[kk][3] = pack_half2(qf[kk][6] * qdown, qf[kk][7] * qdown);
    }
    // 1152 x the sum of each q row as the mma sees it (the fp16 values), for the code offset
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      float sum = 0.0f;
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&qa[kk][hr]));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&qa[kk][2 + hr]));
        sum += (a.x + a.y) + (b.x + b.y);
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      q_off[hr] = kCodeBias * sum;
    }
  }

  // O accumulators: o[2 b + par] is the n-tile of 16-dim block b whose column c stands for dim
  // 16 b + 2 c + par (see the V operand below); a thread's four values of a block (par 0 / 1,
  // columns 2 t / 2 t + 1) are therefore the four consecutive dims 16 b + 4 t .. + 3.
  float o[16][4];
#pragma unroll
  for (int nd = 0; nd < 16; ++nd) o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.0f;
  float osum[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // P against a column of ones: sum of the fp16 probabilities
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
  // the lowest position among the group's rows: tiles entirely below it need no causal mask
  int pos_min = pos_max;
  for (int j = 0; j < nrows; ++j) {
    const int pj = __ldg(p.row_pos + r0 + j);
    pos_min = min(pos_min, pj < 0 ? -1 : min(pj, p.max_len - 1));
  }
  const size_t head_row0 = static_cast<size_t>(hkv) * p.stride;

  // ---- gather. Lane l (and l + 16) looks up the pool row of tile position l and fetches that
  // position's two scales. The code rows are copied four rows per instruction: in copy i lane l
  // moves 16-byte piece l % 8 of row 4 i + l / 8, so one instruction covers four whole 128-byte
  // rows (every 32-byte sector requested once). While tile i is computed, the raw codes of tiles
  // i + 1 and i + 2 are in flight into this warp's stages and the table entries of tile i + 3 are
  // being looked up, so neither of the two dependent global latencies (table -> row address ->
  // codes) is exposed.
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
  float sk_q[kStages], sv_q[kStages];  // scales of the tiles in flight, oldest first (lane n: position n)
  {
    const int pr0 = table_row(t_first), pr1 = table_row(t_first + kStep), pr2 = table_row(t_first + 2 * kStep);
    gather(0, t_first, pr0, sk_q[0], sv_q[0]);
    gather(1, t_first + kStep, pr1, sk_q[1], sv_q[1]);
    gather(2, t_first + 2 * kStep, pr2, sk_q[2], sv_q[2]);
  }
  int prow_next = table_row(t_first + 3 * kStep);
  int stage = 0;

  for (int t0 = t_first; t0 < t_end; t0 += kStep) {
    cp_async_wait<kStages - 2>();  // all but the newest two groups have landed: tile i is in shared memory
    __syncwarp();                  // ... for every lane, and every lane is done with tile i - 1
    // tile i + 3 goes into the stage tile i - 1 was read out of
    gather((stage + kStages - 1) % kStages, t0 + (kStages - 1) * kStep, prow_next, sk_q[kStages - 1],
           sv_q[kStages - 1]);
    prow_next = table_row(t0 + kStages * kStep);
    const float sk_cur = sk_q[0], sv_cur = sv_q[0];
#pragma unroll
    for (int i = 0; i + 1 < kStages; ++i) sk_q[i] = sk_q[i + 1], sv_q[i] = sv_q[i + 1];

    // ---- S = Q K^T over the tile: two 8-position column blocks, K operands straight from the
    // raw codes (two accumulators per block halve the dependent mma chain)
    float s[2][4];
    const unsigned char* kstage = raw_k + stage * kRawTile;
    const unsigned char* vstage = raw_v + stage * kRawTile;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      float sa[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sb[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      const unsigned char* krow = kstage + (nt * 8 + g) * kPitch + 4 * t;
#pragma unroll
      for (int kk = 0; kk < 8; kk += 2) {
        uint32_t b0, b1, c0, c1;
        codes4_to_half(*reinterpret_cast<const uint32_t*>(krow + kk * 16), b0, b1);
        codes4_to_half(*reinterpret_cast<const uint32_t*>(krow + kk * 16 + 16), c0, c1);
        mma_f16(sa, qa[kk], b0, b1);
        mma_f16(sb, qa[kk + 1], c0, c1);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) s[nt][i] = sa[i] + sb[i];
    }
    stage = (stage + 1) % kStages;

    // ---- scale, mask, online softmax; thread holds columns n = nt * 8 + 2 t + {0, 1} of rows g, g + 8
    float pr[2][4];
    float tile_max[2] = {-INFINITY, -INFINITY};
    float svn[2][2];
    const bool unmasked = t0 + kTile <= t_end && t0 + kTile - 1 <= pos_min;  // warp-uniform
    const bool upper = nrows > 2;  // tile rows 8..15 carry query rows 2 and 3; a decode row leaves them empty
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int n = nt * 8 + 2 * t + e;
        const float f = __shfl_sync(0xffffffffu, sk_cur, n) * logit_scale;
        svn[nt][e] = __shfl_sync(0xffffffffu, sv_cur, n);
        float a = (s[nt][e] - q_off[0]) * f;
        float b = upper ? (s[nt][2 + e] - q_off[1]) * f : -INFINITY;
        if (!unmasked) {
          const int tp = t0 + n;
          if (tp > pos_lo || tp >= t_end) a = -INFINITY;
          if (tp > pos_hi || tp >= t_end) b = -INFINITY;
        }
        s[nt][e] = a, s[nt][2 + e] = b;
        tile_max[0] = fmaxf(tile_max[0], a);
        tile_max[1] = fmaxf(tile_max[1], b);
      }
    }
    float corr[2];
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      if (hr == 1 && !upper) {
        corr[1] = 1.0f;
        pr[0][2] = pr[0][3] = pr[1][2] = pr[1][3] = 0.0f;
        continue;
      }
      float mx = tile_max[hr];
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[hr], mx);
      corr[hr] = (m_new == -INFINITY) ? 1.0f : ex2_approx(m_run[hr] - m_new);  // 2^-inf = 0
      const float base = (m_new == -INFINITY) ? 0.0f : m_new;
      float sum = 0.0f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pv = ex2_approx(s[nt][2 * hr + e] - base);  // masked: 2^-inf = 0
          pr[nt][2 * hr + e] = pv;
          sum += pv;
        }
      l_run[hr] = l_run[hr] * corr[hr] + sum;  // this thread's columns only; quads are summed at the end
      m_run[hr] = m_new;
    }
    // the running maximum settles after a few tiles; most tiles need no rescaling at all
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
      for (int nd = 0; nd < 16; ++nd) {
        o[nd][0] *= corr[0], o[nd][1] *= corr[0];
        o[nd][2] *= corr[1], o[nd][3] *= corr[1];
      }
      osum[0] *= corr[0], osum[1] *= corr[0], osum[2] *= corr[1], osum[3] *= corr[1];
    }
    // ---- O += (P diag(v_scale)) V: P's accumulator layout is the A-operand layout ------------------
    uint32_t pa[4];
    pa[0] = pack_half2(pr[0][0] * svn[0][0], pr[0][1] * svn[0][1]);
    pa[1] = pack_half2(pr[0][2] * svn[0][0], pr[0][3] * svn[0][1]);
    pa[2] = pack_half2(pr[1][0] * svn[1][0], pr[1][1] * svn[1][1]);
    pa[3] = pack_half2(pr[1][2] * svn[1][0], pr[1][3] * svn[1][1]);
    // V operand straight from the raw bytes: the tile is read as 16-bit elements (two adjacent
    // dims of one position), transposed by ldmatrix; a register then holds positions 2 t, 2 t + 1 for
    // dims 2 g and 2 g + 1 of a 16-dim block, and one byte permute each picks the (position pair,
    // dim) halves of the even-dim and of the odd-dim n-tile, already in fp16 form (code + 1152).
#pragma unroll
    for (int blk = 0; blk < 8; blk += 2) {
      // matrices: (pos 0-7, block blk), (pos 8-15, block blk), (pos 0-7, block blk + 1), (pos 8-15, ..)
      uint32_t r[4];
      ldmatrix_x4_trans(r, vstage + (lane & 15) * kPitch + (blk + (lane >> 4)) * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) r[i] ^= 0x80808080u;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const uint32_t lo = r[2 * u], hi = r[2 * u + 1];  // positions 0-7 / 8-15 of block blk + u
        mma_f16(o[2 * (blk + u)], pa, __byte_perm(lo, 0x64646464u, 0x4240), __byte_perm(hi, 0x64646464u, 0x4240));
        mma_f16(o[2 * (blk + u) + 1], pa, __byte_perm(lo, 0x64646464u, 0x4341), __byte_perm(hi, 0x64646464u, 0x4341));
      }
    }
    mma_f16(osum, pa, 0x3c003c00u, 0x3c003c00u);  // the column of ones
  }
  // take the code offset out of the accumulators: O = O_mma - 1152 * sum(p)
#pragma unroll
  for (int nd = 0; nd < 16; ++nd) {
    o[nd][0] -= kCodeBias * osum[0], o[nd][1] -= kCodeBias * osum[0];
    o[nd][2] -= kCodeBias * osum[2], o[nd][3] -= kCodeBias * osum[2];
  }

  cp_async_wait<0>();  // nothing of this thread's may still be landing when the memory is reused
  // ---- merge the four warps' states (each warp parks its state at the start of its own block) ----
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    l_run[hr] += __shfl_xor_sync(0xffffffffu, l_run[hr], 1);
    l_run[hr] += __shfl_xor_sync(0xffffffffu, l_run[hr], 2);
  }
  __syncwarp();
  float* wo = reinterpret_cast<float*>(wsm);  // [16][128] floats
  float* wml = wo + 16 * kAD;                 // [16][2]
#pragma unroll
  for (int blk = 0; blk < 8; ++blk) {
    // dims 16 blk + 4 t + {0, 1, 2, 3} = (even tile col 2t, odd tile col 2t, even col 2t+1, odd col 2t+1)
    *reinterpret_cast<float4*>(wo + g * kAD + blk * 16 + 4 * t) =
        make_float4(o[2 * blk][0], o[2 * blk + 1][0], o[2 * blk][1], o[2 * blk + 1][1]);
    *reinterpret_cast<float4*>(wo + (g + 8) * kAD + blk * 16 + 4 * t) =
        make_float4(o[2 * blk][2], o[2 * blk + 1][2], o[2 * blk][3], o[2 * blk + 1][3]);
  }
  if (t == 0) {
    wml[g * 2] = m_run[0], wml[g * 2 + 1] = l_run[0];
    wml[(g + 8) * 2] = m_run[1], wml[(g + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  merge_warps(p, s_dyn, kWarpSmem, grp, hkv, split, r0, nrows);
}

// ---- groups of one or two query rows (plain decode), transposed ------------------------------------
// With 4 or 8 live rows the 16-row mma tile of the kernel above is mostly padding. Here the cache
// positions take the 16-row side instead: S^T = K Q^T (A = 16 positions x dims from the raw K
// codes, B = the 8 columns (query row, head) of q) and O^T = V^T P^T (A = 16 dims x 16 positions
// from the raw V codes through ldmatrix.trans, B = P^T, which is the S^T accumulator transposed by
// movmatrix). Half the mma instructions per tile, half the O accumulators (so four CTAs per SM),
// and the softmax of a column runs down the lanes (three xor shuffles over g).
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

__global__ void __launch_bounds__(kWarps * 32, kCtasPerSmT) attn_decode_t_kernel(const AttnParams p) {
  pdl_begin();
  extern __shared__ __align__(128) unsigned char s_dyn[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, hkv = blockIdx.y, grp = blockIdx.z;
  const int r0 = grp * p.group_rows;
  const int nrows = min(p.group_rows, p.rows - r0);  // 1 or 2
  unsigned char* wsm = s_dyn + static_cast<size_t>(warp) * kWarpSmemT;
  unsigned char* raw_k = wsm;
  unsigned char* raw_v = wsm + kStagesT * kRawTile;

  // column c = 4 j + hl stands for (query row j, head hl). As accumulator owner a thread has columns
  // 2 t and 2 t + 1 (both of query row t / 2); as B-operand owner it has column g.
  int pos_col = -1, pos_max = -1, pos_min = INT_MAX;
  for (int j = 0; j < nrows; ++j) {
    int pj = __ldg(p.row_pos + r0 + j);
    pj = pj < 0 ? -1 : min(pj, p.max_len - 1);
    pos_max = max(pos_max, pj);
    pos_min = min(pos_min, pj);
    if (j == (t >> 1)) pos_col = pj;
  }
  const int* pt = p.row_pt != nullptr ? p.row_pt[r0] : p.pt;
  const int t_begin = split * p.split_len;
  const int t_end = min(t_begin + p.split_len, pos_max + 1);

  // ---- q as the B operand: (dims 16 kk + 4 t .. + 3 of column g), fp16, scaled by a power of two
  uint32_t qb[8][2];
  float logit_scale;
  float q_off[2];  // 1152 x the sum of q over the dims, for the accumulator's columns 2 t, 2 t + 1
  {
    const int j = g >> 2, hl = g & 3;
    const bool live = j < nrows;
    const uint16_t* qrow = p.q + (static_cast<size_t>(r0 + (live ? j : 0)) * p.Hq + hkv * kGqa + hl) * kAD;
    float qf[8][4];
    float qmax = 0.0f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint2 w = live ? __ldg(reinterpret_cast<const uint2*>(qrow + kk * 16 + 4 * t)) : make_uint2(0u, 0u);
      qf[kk][0] = bf16_to_f32(w.x & 0xffffu), qf[kk][1] = bf16_to_f32(w.x >> 16);
      qf[kk][2] = bf16_to_f32(w.y & 0xffffu), qf[kk][3] = bf16_to_f32(w.y >> 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) qmax = fmaxf(qmax, fabsf(qf[kk][i]));
    }
    qmax = warp_max(qmax);
    int qexp = 0;
    if (qmax > 0.0f && qmax < INFINITY)
      qexp = min(max(((__float_as_int(qmax) >> 23) & 0xff) - 127 - 10, -100), 100);
    const float qdown = __int_as_float((127 - qexp) << 23);
    logit_scale = p.scale_log2 * __int_as_float((127 + qexp) << 23);
    float sum = 0.0f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      qb[kk][0] = pack_half2(qf[kk][0] * qdown, qf[kk][1] * qdown);
      qb[kk][1] = pack_half2(qf[kk][2] * qdown, qf[kk][3] * qdown);
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&qb[kk][0]));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&qb[kk][1]));
      sum += (a.x + a.y) + (b.x + b.y);
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);  // the whole row of column g, in all four lanes of quad g
    q_off[0] = kCodeBias * __shfl_sync(0xffffffffu, sum, (2 * t) * 4);
    q_off[1] = kCodeBias * __shfl_sync(0xffffffffu, sum, (2 * t + 1) * 4);
  }

  // O^T accumulators: block b, rows g / g + 8 = dims 16 b + 2 g / 16 b + 2 g + 1, columns 2 t, 2 t + 1
  float o[8][4];
#pragma unroll
  for (int b = 0; b < 8; ++b) o[b][0] = o[b][1] = o[b][2] = o[b][3] = 0.0f;
  float osum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
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

    // ---- S^T = K Q^T: rows = positions g and g + 8, columns 2 t, 2 t + 1
    float sa[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sb[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const unsigned char* k_lo = kstage + g * kPitch + 4 * t;
    const unsigned char* k_hi = k_lo + 8 * kPitch;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      uint32_t a[4];
      codes4_to_half(*reinterpret_cast<const uint32_t*>(k_lo + kk * 16), a[0], a[2]);
      codes4_to_half(*reinterpret_cast<const uint32_t*>(k_hi + kk * 16), a[1], a[3]);
      mma_f16((kk & 1) ? sb : sa, a, qb[kk][0], qb[kk][1]);
    }
    // ---- scale, mask, online softmax down the lanes
    const float f_lo = __shfl_sync(0xffffffffu, sk_cur, g) * logit_scale;
    const float f_hi = __shfl_sync(0xffffffffu, sk_cur, g + 8) * logit_scale;
    const float sv_lo = __shfl_sync(0xffffffffu, sv_cur, g), sv_hi = __shfl_sync(0xffffffffu, sv_cur, g + 8);
    const bool unmasked = t0 + kTile <= t_end && t0 + kTile - 1 <= pos_min;  // warp-uniform
    const bool ok_lo = unmasked || (t0 + g <= pos_col && t0 + g < t_end);
    const bool ok_hi = unmasked || (t0 + g + 8 <= pos_col && t0 + g + 8 < t_end);
    float pr[4], corr[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float x_lo = ok_lo ? (sa[e] + sb[e] - q_off[e]) * f_lo : -INFINITY;
      const float x_hi = ok_hi ? (sa[2 + e] + sb[2 + e] - q_off[e]) * f_hi : -INFINITY;
      float mx = fmaxf(x_lo, x_hi);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
      const float m_new = fmaxf(m_run[e], mx);
      corr[e] = (m_new == -INFINITY) ? 1.0f : ex2_approx(m_run[e] - m_new);
      const float base = (m_new == -INFINITY) ? 0.0f : m_new;
      pr[e] = ex2_approx(x_lo - base);      // position g
      pr[2 + e] = ex2_approx(x_hi - base);  // position g + 8
      l_run[e] = l_run[e] * corr[e] + pr[e] + pr[2 + e];  // this lane's two positions; lanes are summed at the end
      m_run[e] = m_new;
    }
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        o[b][0] *= corr[0], o[b][1] *= corr[1];
        o[b][2] *= corr[0], o[b][3] *= corr[1];
      }
      osum[0] *= corr[0], osum[1] *= corr[1], osum[2] *= corr[0], osum[3] *= corr[1];
    }
    // ---- P^T as the B operand: the accumulator fragments (position g: columns 2 t, 2 t + 1) transposed
    const uint32_t b0 = movmatrix_trans(pack_half2(pr[0] * sv_lo, pr[1] * sv_lo));  // positions 0-7
    const uint32_t b1 = movmatrix_trans(pack_half2(pr[2] * sv_hi, pr[3] * sv_hi));  // positions 8-15
    // ---- O^T += V^T P^T, V operand from the raw bytes (see the kernel above)
#pragma unroll
    for (int blk = 0; blk < 8; blk += 2) {
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
        mma_f16(o[blk + u], a, b0, b1);
      }
    }
    const uint32_t ones[4] = {0x3c003c00u, 0x3c003c00u, 0x3c003c00u, 0x3c003c00u};
    mma_f16(osum, ones, b0, b1);  // every row: the sum over the positions of P^T's columns
  }
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    o[b][0] -= kCodeBias * osum[0], o[b][1] -= kCodeBias * osum[1];
    o[b][2] -= kCodeBias * osum[0], o[b][3] -= kCodeBias * osum[1];
  }

  cp_async_wait<0>();
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 4);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 8);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 16);
  }
  __syncwarp();
  float* wo = reinterpret_cast<float*>(wsm);  // [16][128]; only the rows of live columns are read
  float* wml = wo + 16 * kAD;
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    *reinterpret_cast<float2*>(wo + (2 * t) * kAD + b * 16 + 2 * g) = make_float2(o[b][0], o[b][2]);
    *reinterpret_cast<float2*>(wo + (2 * t + 1) * kAD + b * 16 + 2 * g) = make_float2(o[b][1], o[b][3]);
  }
  if (g == 0) {
    wml[(2 * t) * 2] = m_run[0], wml[(2 * t) * 2 + 1] = l_run[0];
    wml[(2 * t + 1) * 2] = m_run[1], wml[(2 * t + 1) * 2 + 1] = l_run[1];
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
  const int r0 = grp * p.group_rows;
  const int nrows = min(p.group_rows, p.rows - r0);
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

SplitPlan plan_splits(int rows, int group_rows, int Hk, int max_len) {
  const int ctas_per_sm = group_rows <= 2 ? kCtasPerSmT : kCtasPerSm;
  SplitPlan s{};
  s.groups = (rows + group_rows - 1) / group_rows;
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

}  // namespace
}  // namespace g4

extern "C" {

long long granite4_attn_decode_scratch_bytes(int rows, int rows_per_group, int Hk, int max_len) {
  if (rows <= 0 || rows_per_group <= 0 || rows_per_group > g4::kGroupRows || Hk <= 0 || max_len <= 0)
    return -1;
  const g4::SplitPlan s = g4::plan_splits(rows, rows_per_group, Hk, max_len);
  return static_cast<long long>(s.groups) * Hk * s.splits * 16 * (g4::kAD + 2) * static_cast<long long>(sizeof(float));
}

int granite4_kernel_attn_decode_int8_paged(const uint16_t* d_q, const int8_t* d_cache_k,
                                           const int8_t* d_cache_v, const float* d_k_scale,
                                           const float* d_v_scale, const int* d_row_pos,
                                           const int* const* d_row_pt, const int* d_pt, int rows,
                                           int rows_per_group, int Hq, int Hk, int d, int stride,
                                           int max_len, float scale, void* d_scratch,
                                           long long scratch_bytes, uint16_t* d_out) {
  const char* fn = "granite4_kernel_attn_decode_int8_paged";
  if (d_q == nullptr || d_cache_k == nullptr || d_cache_v == nullptr || d_k_scale == nullptr ||
      d_v_scale == nullptr || d_row_pos == nullptr || d_out == nullptr || rows <= 0 ||
      rows_per_group <= 0 || rows_per_group > g4::kGroupRows || stride <= 0 || max_len <= 0 ||
      max_len > stride || !std::isfinite(scale))
    return g4::fail(fn, "invalid arguments");
  if (d != g4::kAD || Hk <= 0 || Hq != g4::kGqa * Hk) return -1;  // engine/src/attention_gpu.h:18-19
  if (!g4::aligned16(d_cache_k) || !g4::aligned16(d_cache_v) || !g4::aligned16(d_q))
    return g4::fail(fn, "q and the caches must be 16-byte aligned");
  const g4::SplitPlan s = g4::plan_splits(rows, rows_per_group, Hk, max_len);
  if (s.groups > 65535) return g4::fail(fn, "too many row groups");
  g4::AttnParams p{};
  p.q = d_q, p.ck = d_cache_k, p.cv = d_cache_v, p.ks = d_k_scale, p.vs = d_v_scale;
  p.row_pos = d_row_pos, p.row_pt = d_row_pt, p.pt = d_pt, p.out = d_out;
  p.rows = rows, p.group_rows = rows_per_group, p.Hq = Hq, p.Hk = Hk, p.stride = stride;
  p.splits = s.splits, p.split_len = s.split_len, p.max_len = max_len;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (s.splits > 1) {
    const long long need = granite4_attn_decode_scratch_bytes(rows, rows_per_group, Hk, max_len);
    if (d_scratch == nullptr || scratch_bytes < need || !g4::aligned16(d_scratch))
      return g4::fail(fn, "scratch missing or smaller than granite4_attn_decode_scratch_bytes()");
    p.part_o = static_cast<float*>(d_scratch);
    p.part_ml = p.part_o + static_cast<size_t>(s.groups) * Hk * s.splits * 16 * g4::kAD;
  }
  cudaStream_t st = g4::current_stream();
  {
    static bool attr_set[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
      G4_CUDA_TRY(fn, cudaFuncSetAttribute(g4::attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(g4::kAttnSmemBytes)));
      G4_CUDA_TRY(fn, cudaFuncSetAttribute(g4::attn_decode_t_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(g4::kAttnSmemBytesT)));
      attr_set[dev] = true;
    }
  }
  const dim3 grid(static_cast<unsigned>(s.splits), static_cast<unsigned>(Hk), static_cast<unsigned>(s.groups));
  const char* force = std::getenv("G4_ATTN_TRANSPOSED");  // 0: the 16-row kernel for every group size (A/B runs)
  if (rows_per_group <= 2 && !(force != nullptr && force[0] == '0'))
    G4_LAUNCH_PDL(fn, g4::attn_decode_t_kernel, grid, dim3(g4::kWarps * 32), g4::kAttnSmemBytesT, st, p);
  else
    G4_LAUNCH_PDL(fn, g4::attn_decode_kernel, grid, dim3(g4::kWarps * 32), g4::kAttnSmemBytes, st, p);
  if (s.splits > 1)
    G4_LAUNCH_PDL(fn, g4::attn_combine_kernel,
                  dim3(static_cast<unsigned>(Hk), static_cast<unsigned>(s.groups), 4u * rows_per_group),
                  dim3(g4::kAD), 0, st, p);
  return 0;
}

}  // extern "C"
