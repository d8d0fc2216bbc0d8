// Causal attention of a prefill chunk over the int8 paged pool (flash form).
//
// The reference's prefill_attention with the int8 cache (contract engine/src/prefill_gemm.h:86-101,
// kernel engine/src/prefill_gemm.cu:1018-1020 prefill_attention_q_kernel): query rows at positions
// [base_pos, base_pos + rows) of ONE sequence attend to cache positions [0, position].
//
// A CTA owns 16 consecutive query positions of one kv head: its four warps are the four query
// heads of the GQA group (engine/src/attention_gpu.h:18-19: Hq = 4 Hk, d = 128), so one K / V tile
// serves 64 query rows. Per tile of 64 cache positions:
//   1. the raw int8 rows and their scales arrive by cp.async (two stages; gathered through the page
//      table, 128 bytes per row);
//   2. all 128 threads turn them ONCE into fp16 tiles in shared memory: K as the codes themselves
//      (exact; the per-position scale multiplies the logits in f32 afterwards), V as code x scale;
//   3. every warp computes S = Q K^T (16 x 64, mma.sync.m16n8k16, K fragments by ldmatrix), the
//      online softmax of its 16 rows in registers (the accumulator fragments of S are the A
//      fragments of P, no shuffle), and O += P V (V fragments by ldmatrix.trans).
// Compared with walking the prefix once per group of four rows on the decode kernel, the int8 ->
// fp16 conversion is shared by 64 query rows instead of 16, and K / V are fetched once per 16
// positions instead of once per 4.
//
// Arithmetic against the reference's golden pipeline (engine/src/kernel_math.h:265-331): logits in
// f32 from fp16 operands that hold q (bf16 -> fp16, exact in fp16's range) and the codes exactly, probabilities rounded
// to fp16 instead of bf16, V dequantised to fp16 instead of bf16: inside the 0.03 absolute bar the
// reference sets for its own kernels (engine/tests/test_kernels.cu:2055).
//
// The only waits are cp.async.wait_group (the thread's own copies) and __syncthreads.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <climits>
#include <cmath>
#include <cstdint>
#include <cstdlib>

#include "g4_host.h"
#include "g4_math.cuh"

namespace g4 {
namespace {

constexpr int kD = 128;        // head dim
constexpr int kQRows = 16;     // query positions per CTA
constexpr int kTileP = 64;     // cache positions per tile
constexpr int kPfWarps = 4;    // = query heads per kv head
constexpr int kHPitch = kD + 8;  // halves per converted row: 272 bytes, ldmatrix rows hit distinct banks

struct PrefillParams {
  const uint16_t* q;
  const int8_t* ck;
  const int8_t* cv;
  const float* ks;
  const float* vs;
  const int* pt;  // position -> pool row, or NULL (identity)
  uint16_t* out;
  int rows, base_pos, Hq, Hk;
  long long stride;
  float scale_log2;  // softmax scale x log2(e)
};

struct PrefillSmem {
  int8_t raw_k[2][kTileP][kD];
  int8_t raw_v[2][kTileP][kD];
  float ks[2][kTileP];
  float vs[2][kTileP];
  __half kh[kTileP][kHPitch];
  __half vh[kTileP][kHPitch];
};

__device__ __forceinline__ void pf_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void pf_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void pf_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void pf_cp16(void* dst, const void* src, bool real) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  const int n = real ? 16 : 0;  // 0: nothing is read, the bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void pf_cp4(void* dst, const void* src, bool real) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  const int n = real ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ float pf_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pf_pack(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// Four int8 codes -> two half2 holding the codes exactly: each byte, biased to unsigned, goes into
// the mantissa of 1024.0 (0x6400 + code + 128 = code + 1152), and 1152 is subtracted (exact).
__device__ __forceinline__ void pf_codes4(uint32_t w, __half2& lo, __half2& hi) {
  w ^= 0x80808080u;
  const uint32_t a = __byte_perm(w, 0x64646464u, 0x4140), b = __byte_perm(w, 0x64646464u, 0x4342);
  const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
  lo = __hsub2(*reinterpret_cast<const __half2*>(&a), bias);
  hi = __hsub2(*reinterpret_cast<const __half2*>(&b), bias);
}

__global__ void __launch_bounds__(kPfWarps * 32, 3) attn_prefill_kernel(const PrefillParams p) {
  extern __shared__ __align__(16) unsigned char pf_smem[];
  PrefillSmem& sm = *reinterpret_cast<PrefillSmem*>(pf_smem);
  pdl_begin();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int qb = static_cast<int>(gridDim.x - 1 - blockIdx.x);  // the longest prefixes start first
  const int hkv = blockIdx.y, head = hkv * kPfWarps + warp;
  const int r0 = qb * kQRows;
  const int nrows = min(kQRows, p.rows - r0);
  const int kv_len = p.base_pos + r0 + nrows;  // cache positions some row of this CTA sees
  const int ntiles = (kv_len + kTileP - 1) / kTileP;
  const size_t head_row0 = static_cast<size_t>(hkv) * p.stride;
  const int pos_a = p.base_pos + r0 + min(g, nrows - 1), pos_b = p.base_pos + r0 + min(g + 8, nrows - 1);

  // raw rows of one tile: thread -> (row, 64-byte half); zero-filled past kv_len
  const int crow = tid >> 1, chalf = tid & 1;
  auto gather = [&](int stage, int tile) {
    const int pos = tile * kTileP + crow;
    const bool have = pos < kv_len;
    int prow = have ? (p.pt != nullptr ? __ldg(p.pt + pos) : pos) : 0;
    prow = min(max(prow, 0), static_cast<int>(p.stride) - 1);
    const size_t off = (head_row0 + prow) * kD + chalf * 64;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      pf_cp16(&sm.raw_k[stage][crow][chalf * 64 + 16 * i], p.ck + off + 16 * i, have);
      pf_cp16(&sm.raw_v[stage][crow][chalf * 64 + 16 * i], p.cv + off + 16 * i, have);
    }
    if (chalf == 0) pf_cp4(&sm.ks[stage][crow], p.ks + head_row0 + prow, have);
    else pf_cp4(&sm.vs[stage][crow], p.vs + head_row0 + prow, have);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  gather(0, 0);

  // Q as the A operand: rows g and g + 8 of this warp's head; bf16 -> fp16 is exact
  uint32_t qa[8][4];
  {
    const uint16_t* qra = p.q + (static_cast<size_t>(r0 + min(g, nrows - 1)) * p.Hq + head) * kD;
    const uint16_t* qrb = p.q + (static_cast<size_t>(r0 + min(g + 8, nrows - 1)) * p.Hq + head) * kD;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t w0 = __ldg(reinterpret_cast<const uint32_t*>(qra + kk * 16 + 2 * t));
      const uint32_t w1 = __ldg(reinterpret_cast<const uint32_t*>(qrb + kk * 16 + 2 * t));
      const uint32_t w2 = __ldg(reinterpret_cast<const uint32_t*>(qra + kk * 16 + 8 + 2 * t));
      const uint32_t w3 = __ldg(reinterpret_cast<const uint32_t*>(qrb + kk * 16 + 8 + 2 * t));
      qa[kk][0] = pf_pack(bf16_lo(w0), bf16_hi(w0)), qa[kk][1] = pf_pack(bf16_lo(w1), bf16_hi(w1));
      qa[kk][2] = pf_pack(bf16_lo(w2), bf16_hi(w2)), qa[kk][3] = pf_pack(bf16_lo(w3), bf16_hi(w3));
    }
  }

  float o[16][4];
#pragma unroll
  for (int nb = 0; nb < 16; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

  for (int tile = 0; tile < ntiles; ++tile) {
    const int stage = tile & 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // the raw stage is complete; every warp is done with the previous fp16 tiles
    if (tile + 1 < ntiles) gather(stage ^ 1, tile + 1);

    // ---- int8 -> fp16, once for the four warps. Item = 8 codes of a row: 16 consecutive lanes read
    // one raw row (128 contiguous bytes) and write 256 contiguous bytes of the fp16 row: no bank
    // conflicts either way.
#pragma unroll
    for (int it = 0; it < kTileP * 16 / (kPfWarps * 32); ++it) {
      const int item = it * (kPfWarps * 32) + tid, row = item >> 4, piece = item & 15;
      const uint2 rk = *reinterpret_cast<const uint2*>(&sm.raw_k[stage][row][piece * 8]);
      const uint2 rv = *reinterpret_cast<const uint2*>(&sm.raw_v[stage][row][piece * 8]);
      const __half2 vs2 = __float2half2_rn(sm.vs[stage][row]);
      __half2 kh2[4], vh2[4];
      pf_codes4(rk.x, kh2[0], kh2[1]), pf_codes4(rk.y, kh2[2], kh2[3]);
      pf_codes4(rv.x, vh2[0], vh2[1]), pf_codes4(rv.y, vh2[2], vh2[3]);
#pragma unroll
      for (int j = 0; j < 4; ++j) vh2[j] = __hmul2(vh2[j], vs2);
      *reinterpret_cast<uint4*>(&sm.kh[row][piece * 8]) = *reinterpret_cast<const uint4*>(&kh2[0]);
      *reinterpret_cast<uint4*>(&sm.vh[row][piece * 8]) = *reinterpret_cast<const uint4*>(&vh2[0]);
    }
    if (tid < kTileP) sm.ks[stage][tid] *= p.scale_log2;  // logits come out in the base-2 domain
    __syncthreads();

    // ---- S = Q K^T (16 x 64 per warp)
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < 8; kk += 2) {
#pragma unroll
      for (int jj = 0; jj < 8; jj += 4) {  // four fragments in flight; no two consecutive MMAs share an accumulator
        uint32_t b[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) pf_ldmatrix_x4(b[j], &sm.kh[(jj + j) * 8 + (lane & 7)][kk * 16 + (lane >> 3) * 8]);
#pragma unroll
        for (int j = 0; j < 4; ++j) pf_mma(s[jj + j], qa[kk], b[j][0], b[j][1]);
#pragma unroll
        for (int j = 0; j < 4; ++j) pf_mma(s[jj + j], qa[kk + 1], b[j][2], b[j][3]);
      }
    }

    // ---- per-position scale, causal mask, online softmax of rows g and g + 8
    const int c0 = tile * kTileP;
    const bool diag = c0 + kTileP - 1 > p.base_pos + r0;  // some entry of the tile may be masked (uniform)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float2 f = *reinterpret_cast<const float2*>(&sm.ks[stage][j * 8 + 2 * t]);
      s[j][0] *= f.x, s[j][1] *= f.y, s[j][2] *= f.x, s[j][3] *= f.y;
      if (diag) {
        const int col = c0 + j * 8 + 2 * t;
        if (col > pos_a) s[j][0] = -INFINITY;
        if (col + 1 > pos_a) s[j][1] = -INFINITY;
        if (col > pos_b) s[j][2] = -INFINITY;
        if (col + 1 > pos_b) s[j][3] = -INFINITY;
      }
      mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
    }
    float corr[2], base[2], rsum[2] = {0.0f, 0.0f};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
      mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
      const float m_new = fmaxf(m_run[e], mx[e]);
      corr[e] = m_new == -INFINITY ? 1.0f : pf_ex2(m_run[e] - m_new);
      base[e] = m_new == -INFINITY ? 0.0f : m_new;
      m_run[e] = m_new;
    }
    uint32_t pa[4][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float p0 = pf_ex2(s[j][0] - base[0]), p1 = pf_ex2(s[j][1] - base[0]);
      const float p2 = pf_ex2(s[j][2] - base[1]), p3 = pf_ex2(s[j][3] - base[1]);
      rsum[0] += p0 + p1, rsum[1] += p2 + p3;
      pa[j >> 1][(j & 1) * 2] = pf_pack(p0, p1);      // row g
      pa[j >> 1][(j & 1) * 2 + 1] = pf_pack(p2, p3);  // row g + 8
    }
    l_run[0] = l_run[0] * corr[0] + rsum[0], l_run[1] = l_run[1] * corr[1] + rsum[1];
    if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
      for (int nb = 0; nb < 16; ++nb)
        o[nb][0] *= corr[0], o[nb][1] *= corr[0], o[nb][2] *= corr[1], o[nb][3] *= corr[1];
    }

    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int nb = 0; nb < 16; nb += 2) {
        uint32_t b[4];
        pf_ldmatrix_x4_trans(b, &sm.vh[kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][nb * 8 + (lane >> 4) * 8]);
        pf_mma(o[nb], pa[kk], b[0], b[1]);
        pf_mma(o[nb + 1], pa[kk], b[2], b[3]);
      }
    }
  }

  // ---- normalise and store rows g and g + 8
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 1);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 2);
  }
  const float inv_a = l_run[0] > 0.0f ? 1.0f / l_run[0] : 0.0f, inv_b = l_run[1] > 0.0f ? 1.0f / l_run[1] : 0.0f;
  uint16_t* out_a = p.out + (static_cast<size_t>(r0 + g) * p.Hq + head) * kD + 2 * t;
  uint16_t* out_b = p.out + (static_cast<size_t>(r0 + g + 8) * p.Hq + head) * kD + 2 * t;
#pragma unroll
  for (int nb = 0; nb < 16; ++nb) {
    if (g < nrows) *reinterpret_cast<uint32_t*>(out_a + nb * 8) = pack_bf16x2(o[nb][0] * inv_a, o[nb][1] * inv_a);
    if (g + 8 < nrows) *reinterpret_cast<uint32_t*>(out_b + nb * 8) = pack_bf16x2(o[nb][2] * inv_b, o[nb][3] * inv_b);
  }
}

// The same with 32 query positions per CTA: every warp owns two 16-row tiles of its head, so a K or V
// fragment fetched from shared memory feeds four MMAs instead of two and the conversion is shared by 128
// query rows. The accumulators of two tiles leave no registers for Q and a 64-column S, so Q (fp16) lives
// in shared memory and a tile of 64 positions is consumed as two halves of 32.
constexpr int kQRows2 = 32;
struct PrefillSmem2 {
  PrefillSmem t;
  __half qh[kPfWarps][kQRows2][kHPitch];
};

__global__ void __launch_bounds__(kPfWarps * 32, 2) attn_prefill2_kernel(const PrefillParams p) {
  extern __shared__ __align__(16) unsigned char pf_smem[];
  PrefillSmem2& sm2 = *reinterpret_cast<PrefillSmem2*>(pf_smem);
  PrefillSmem& sm = sm2.t;
  pdl_begin();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int qb = static_cast<int>(gridDim.x - 1 - blockIdx.x);
  const int hkv = blockIdx.y, head = hkv * kPfWarps + warp;
  const int r0 = qb * kQRows2;
  const int nrows = min(kQRows2, p.rows - r0);
  const int kv_len = p.base_pos + r0 + nrows;
  const int ntiles = (kv_len + kTileP - 1) / kTileP;
  const size_t head_row0 = static_cast<size_t>(hkv) * p.stride;
  int pos_row[2][2];  // [tile of 16 rows][row g / g + 8]
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int e = 0; e < 2; ++e) pos_row[mt][e] = p.base_pos + r0 + min(mt * 16 + g + 8 * e, nrows - 1);

  const int crow = tid >> 1, chalf = tid & 1;
  auto gather = [&](int stage, int tile) {
    const int pos = tile * kTileP + crow;
    const bool have = pos < kv_len;
    int prow = have ? (p.pt != nullptr ? __ldg(p.pt + pos) : pos) : 0;
    prow = min(max(prow, 0), static_cast<int>(p.stride) - 1);
    const size_t off = (head_row0 + prow) * kD + chalf * 64;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      pf_cp16(&sm.raw_k[stage][crow][chalf * 64 + 16 * i], p.ck + off + 16 * i, have);
      pf_cp16(&sm.raw_v[stage][crow][chalf * 64 + 16 * i], p.cv + off + 16 * i, have);
    }
    if (chalf == 0) pf_cp4(&sm.ks[stage][crow], p.ks + head_row0 + prow, have);
    else pf_cp4(&sm.vs[stage][crow], p.vs + head_row0 + prow, have);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  gather(0, 0);

  // this warp's 32 Q rows -> fp16 in shared memory (rows past the chunk repeat the last row)
  for (int i = lane; i < kQRows2 * (kD / 8); i += 32) {
    const int row = i >> 4, piece = i & 15;
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(r0 + min(row, nrows - 1)) * p.Hq + head) * kD) + piece);
    uint4 h;
    h.x = pf_pack(bf16_lo(w.x), bf16_hi(w.x)), h.y = pf_pack(bf16_lo(w.y), bf16_hi(w.y));
    h.z = pf_pack(bf16_lo(w.z), bf16_hi(w.z)), h.w = pf_pack(bf16_lo(w.w), bf16_hi(w.w));
    *reinterpret_cast<uint4*>(&sm2.qh[warp][row][piece * 8]) = h;
  }
  __syncwarp();

  float o[2][16][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nb = 0; nb < 16; ++nb) o[mt][nb][0] = o[mt][nb][1] = o[mt][nb][2] = o[mt][nb][3] = 0.0f;
  float m_run[2][2], l_run[2][2];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) m_run[mt][0] = m_run[mt][1] = -INFINITY, l_run[mt][0] = l_run[mt][1] = 0.0f;

  for (int tile = 0; tile < ntiles; ++tile) {
    const int stage = tile & 1;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    if (tile + 1 < ntiles) gather(stage ^ 1, tile + 1);
#pragma unroll
    for (int it = 0; it < kTileP * 16 / (kPfWarps * 32); ++it) {
      const int item = it * (kPfWarps * 32) + tid, row = item >> 4, piece = item & 15;
      const uint2 rk = *reinterpret_cast<const uint2*>(&sm.raw_k[stage][row][piece * 8]);
      const uint2 rv = *reinterpret_cast<const uint2*>(&sm.raw_v[stage][row][piece * 8]);
      const __half2 vs2 = __float2half2_rn(sm.vs[stage][row]);
      __half2 kh2[4], vh2[4];
      pf_codes4(rk.x, kh2[0], kh2[1]), pf_codes4(rk.y, kh2[2], kh2[3]);
      pf_codes4(rv.x, vh2[0], vh2[1]), pf_codes4(rv.y, vh2[2], vh2[3]);
#pragma unroll
      for (int j = 0; j < 4; ++j) vh2[j] = __hmul2(vh2[j], vs2);
      *reinterpret_cast<uint4*>(&sm.kh[row][piece * 8]) = *reinterpret_cast<const uint4*>(&kh2[0]);
      *reinterpret_cast<uint4*>(&sm.vh[row][piece * 8]) = *reinterpret_cast<const uint4*>(&vh2[0]);
    }
    if (tid < kTileP) sm.ks[stage][tid] *= p.scale_log2;
    __syncthreads();

#pragma unroll 1
    for (int half = 0; half < 2; ++half) {  // 32 positions at a time
      const int c0 = tile * kTileP + half * 32;
      if (c0 >= kv_len) break;  // uniform over the CTA
      // ---- S = Q K^T: two 16 x 32 tiles; a K fragment serves both
      float s[2][4][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[mt][j][0] = s[mt][j][1] = s[mt][j][2] = s[mt][j][3] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < 8; kk += 2) {
        uint32_t qa[2][2][4];  // [row tile][k-step kk, kk + 1]
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
          for (int u = 0; u < 2; ++u)
            pf_ldmatrix_x4(qa[mt][u], &sm2.qh[warp][mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][(kk + u) * 16 + (lane >> 4) * 8]);
#pragma unroll
        uint32_t b[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) pf_ldmatrix_x4(b[j], &sm.kh[half * 32 + j * 8 + (lane & 7)][kk * 16 + (lane >> 3) * 8]);
#pragma unroll
        for (int u = 0; u < 2; ++u)  // no two consecutive MMAs share an accumulator
#pragma unroll
          for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) pf_mma(s[mt][j], qa[mt][u], b[j][2 * u], b[j][2 * u + 1]);
      }
      // ---- scale, mask, online softmax; P fragments
      const bool diag = c0 + 31 > p.base_pos + r0;
      uint32_t pa[2][2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = *reinterpret_cast<const float2*>(&sm.ks[stage][half * 32 + j * 8 + 2 * t]);
          s[mt][j][0] *= f.x, s[mt][j][1] *= f.y, s[mt][j][2] *= f.x, s[mt][j][3] *= f.y;
          if (diag) {
            const int col = c0 + j * 8 + 2 * t;
            if (col > pos_row[mt][0]) s[mt][j][0] = -INFINITY;
            if (col + 1 > pos_row[mt][0]) s[mt][j][1] = -INFINITY;
            if (col > pos_row[mt][1]) s[mt][j][2] = -INFINITY;
            if (col + 1 > pos_row[mt][1]) s[mt][j][3] = -INFINITY;
          }
          mx[0] = fmaxf(mx[0], fmaxf(s[mt][j][0], s[mt][j][1]));
          mx[1] = fmaxf(mx[1], fmaxf(s[mt][j][2], s[mt][j][3]));
        }
        float corr[2], base[2], rsum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
          mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
          const float m_new = fmaxf(m_run[mt][e], mx[e]);
          corr[e] = m_new == -INFINITY ? 1.0f : pf_ex2(m_run[mt][e] - m_new);
          base[e] = m_new == -INFINITY ? 0.0f : m_new;
          m_run[mt][e] = m_new;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float p0 = pf_ex2(s[mt][j][0] - base[0]), p1 = pf_ex2(s[mt][j][1] - base[0]);
          const float p2 = pf_ex2(s[mt][j][2] - base[1]), p3 = pf_ex2(s[mt][j][3] - base[1]);
          rsum[0] += p0 + p1, rsum[1] += p2 + p3;
          pa[mt][j >> 1][(j & 1) * 2] = pf_pack(p0, p1);
          pa[mt][j >> 1][(j & 1) * 2 + 1] = pf_pack(p2, p3);
        }
        l_run[mt][0] = l_run[mt][0] * corr[0] + rsum[0], l_run[mt][1] = l_run[mt][1] * corr[1] + rsum[1];
        if (__any_sync(0xffffffffu, corr[0] != 1.0f || corr[1] != 1.0f)) {
#pragma unroll
          for (int nb = 0; nb < 16; ++nb)
            o[mt][nb][0] *= corr[0], o[mt][nb][1] *= corr[0], o[mt][nb][2] *= corr[1], o[mt][nb][3] *= corr[1];
        }
      }
      // ---- O += P V: a V fragment serves both row tiles
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
        for (int nb = 0; nb < 16; nb += 2) {
          uint32_t b[4];
          pf_ldmatrix_x4_trans(b, &sm.vh[half * 32 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][nb * 8 + (lane >> 4) * 8]);
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            pf_mma(o[mt][nb], pa[mt][kk], b[0], b[1]);
            pf_mma(o[mt][nb + 1], pa[mt][kk], b[2], b[3]);
          }
        }
      }
    }
  }

#pragma unroll
  for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      l_run[mt][e] += __shfl_xor_sync(0xffffffffu, l_run[mt][e], 1);
      l_run[mt][e] += __shfl_xor_sync(0xffffffffu, l_run[mt][e], 2);
    }
    const float inv_a = l_run[mt][0] > 0.0f ? 1.0f / l_run[mt][0] : 0.0f;
    const float inv_b = l_run[mt][1] > 0.0f ? 1.0f / l_run[mt][1] : 0.0f;
    const int ra = mt * 16 + g, rb = ra + 8;
    uint16_t* out_a = p.out + (static_cast<size_t>(r0 + ra) * p.Hq + head) * kD + 2 * t;
    uint16_t* out_b = p.out + (static_cast<size_t>(r0 + rb) * p.Hq + head) * kD + 2 * t;
#pragma unroll
    for (int nb = 0; nb < 16; ++nb) {
      if (ra < nrows) *reinterpret_cast<uint32_t*>(out_a + nb * 8) = pack_bf16x2(o[mt][nb][0] * inv_a, o[mt][nb][1] * inv_a);
      if (rb < nrows) *reinterpret_cast<uint32_t*>(out_b + nb * 8) = pack_bf16x2(o[mt][nb][2] * inv_b, o[mt][nb][3] * inv_b);
    }
  }
}

}  // namespace

// csrc/attn_prefill_tc.cu: the tcgen05 form (0 done, 1 not available here, -1 launch error)
int attn_prefill_tc(const char* fn, const uint16_t* d_q, float scale, int Hq, int Hk, int base_pos, int rows,
                    int stride, uint16_t* d_out, const int8_t* d_ck, const int8_t* d_cv, const float* d_ks,
                    const float* d_vs, const int* d_pt);

// Launch of the flash form for a whole chunk; arguments as granite4_prefill_attention_int8 (validated there).
// Chunks of 64 rows or more run on the tcgen05 kernel (G4_PREFILL_TC=0 keeps them on the mma.sync
// kernels below, for A/B runs and for tests that compare the two).
int attn_prefill_flash(const char* fn, const uint16_t* d_q, float scale, int Hq, int Hk, int base_pos, int rows,
                       int stride, uint16_t* d_out, const int8_t* d_ck, const int8_t* d_cv, const float* d_ks,
                       const float* d_vs, const int* d_pt) {
  const char* tc_env = std::getenv("G4_PREFILL_TC");
  if (rows >= 64 && !(tc_env != nullptr && tc_env[0] == '0')) {
    const int rc = attn_prefill_tc(fn, d_q, scale, Hq, Hk, base_pos, rows, stride, d_out, d_ck, d_cv, d_ks, d_vs, d_pt);
    if (rc <= 0) return rc;
  }
  static bool attr_set[64];
  int dev = 0;
  G4_CUDA_TRY(fn, cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    G4_CUDA_TRY(fn, cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(sizeof(PrefillSmem))));
    G4_CUDA_TRY(fn, cudaFuncSetAttribute(attn_prefill2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(sizeof(PrefillSmem2))));
    attr_set[dev] = true;
  }
  PrefillParams p{};
  p.q = d_q, p.ck = d_ck, p.cv = d_cv, p.ks = d_ks, p.vs = d_vs, p.pt = d_pt, p.out = d_out;
  p.rows = rows, p.base_pos = base_pos, p.Hq = Hq, p.Hk = Hk, p.stride = stride;
  p.scale_log2 = scale * 1.4426950408889634f;
  const char* v = std::getenv("G4_PREFILL_ROWS32");  // 0: 16 query positions per CTA
  if (!(v != nullptr && v[0] == '0')) {
    const dim3 grid(static_cast<unsigned>((rows + kQRows2 - 1) / kQRows2), static_cast<unsigned>(Hk));
    G4_LAUNCH_PDL(fn, attn_prefill2_kernel, grid, dim3(kPfWarps * 32), sizeof(PrefillSmem2), current_stream(), p);
    return 0;
  }
  const dim3 grid(static_cast<unsigned>((rows + kQRows - 1) / kQRows), static_cast<unsigned>(Hk));
  G4_LAUNCH_PDL(fn, attn_prefill_kernel, grid, dim3(kPfWarps * 32), sizeof(PrefillSmem), current_stream(), p);
  return 0;
}

}  // namespace g4
