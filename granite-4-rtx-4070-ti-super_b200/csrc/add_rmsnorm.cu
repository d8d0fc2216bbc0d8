// Residual add (x residual_multiplier) + RMSNorm with bf16 and per-tensor FP8
// e4m3 outputs, and the plain / final RMSNorm.
//
// Formulation (reference: residual epilogue engine/src/prefill_gemm.cu:81-88,
// norm engine/src/kernels_phase2.cu:51-132 and engine/src/kernel_math.h:178-184,
// per-tensor FP8 rule engine/src/checkpoint_main.cc:118-122, :702-723):
//   h  = bf16(res + rm * y)
//   ms = float(sum_double(h^2) / cols);  r = 1.0f / sqrtf(ms + eps)
//   n  = bf16((h * r) * w)
//   amax = max |n| over the whole tensor; scale = float(amax / 448)
//   code = e4m3_rne(n / scale)
//
// Data layout: rows are contiguous, cols % 8 == 0, every row 16-byte aligned.
//
// Stats sweep (add_rmsnorm_kernel): one CTA owns one row; a thread owns V chunks
// of 8 elements (one 128-bit load each for bf16, two for f32), strided by the
// CTA width so a warp reads 512 contiguous bytes per load. The row stays in
// registers between the reduction and the normalise step, so each input byte is
// read once. It writes h, optionally n as bf16 and the row's r, and folds
// max |n| into d_scale_amax[1] with an integer atomicMax.
//
// The FP8 scale depends on every row, so the codes come from a second sweep:
//   * with r saved per row (d_rstd given): norm_encode_kernel streams the bf16
//     hidden state once more (8 KB per row, not the 16 KB of y and res),
//     recomputes n = bf16(h r w) elementwise and writes the codes;
//   * without it, the row kernel runs again in encode mode and repeats the
//     reduction in the same order, so n is bit-identical either way.
// The second sweep walks the rows backwards: the rows the first sweep wrote
// last are the ones most likely still in L2.
//
// Algorithmic bytes per row at cols = 4096, bf16 y and res, h + FP8 out:
// 8192 + 8192 read, 8192 + 4096 written = 28 672; the second sweep adds another
// 8192-byte read of h.
#include "g4_cluster.cuh"
#include "g4_host.h"
#include "g4_math.cuh"

#include "../../include/granite4_b200.h"

#include <algorithm>
#include <atomic>
#include <cstdlib>

namespace g4 {
namespace {

struct NormParams {
  const void* y;
  const void* res;
  const uint16_t* w;
  uint16_t* h_out;
  uint16_t* n_bf16;
  uint8_t* n_fp8;
  float* scale_amax;  // [0] scale, [1] amax
  float* rstd;        // [rows] or NULL
  float eps;
  float rm;
  int rows;
  int cols8;  // cols / 8
  int cols;
  int reverse;  // walk rows from the last to the first
  float keep_h;  // > 0: a second sweep re-reads h; fraction of its lines to hold in L2 (evict_last)
  double inv_cols;  // 1 / cols when cols is a power of two (the scaling is then exact), else 0
};

// kCluster: the whole grid is one cluster of at most 16 CTAs with one row each; stats and encode in
// one launch (g4_cluster.cuh).
enum { kStats = 0, kEncode = 1, kCluster = 2 };

// Load one 8-element chunk as floats.
template <bool F32>
__device__ __forceinline__ void load_chunk(const void* base, size_t chunk, float (&v)[8]) {
  if (F32) {
    const float4* p = reinterpret_cast<const float4*>(base) + 2 * chunk;
    const float4 a = ld_stream(p), b = ld_stream(p + 1);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w;
    v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  } else {
    unpack8(ld_stream(reinterpret_cast<const uint4*>(base) + chunk), v);
  }
}

// Widest CTA each V is launched with (pick_v keeps to it).
constexpr int max_threads_for(int V) { return V == 1 ? 1024 : (V == 4 ? 256 : 512); }

template <bool Y_F32, bool RES_F32, int V, int PHASE>
__global__ void __launch_bounds__(max_threads_for(V))
    add_rmsnorm_kernel(const NormParams p) {
  pdl_begin();
  if (PHASE == kCluster) cluster_announce();
  const int T = blockDim.x;
  const int t = threadIdx.x;
  // A cluster is a power of two wide: its spare CTAs redo the last row without storing anything,
  // so that they reach the cluster barrier with a harmless contribution.
  const bool live = PHASE != kCluster || static_cast<int>(blockIdx.x) < p.rows;
  const int row = PHASE == kCluster ? (live ? static_cast<int>(blockIdx.x) : p.rows - 1)
                                    : (p.reverse ? p.rows - 1 - static_cast<int>(blockIdx.x) : blockIdx.x);
  const size_t row_chunk0 = static_cast<size_t>(row) * p.cols8;

  float h[V][8];
  const bool has_res = p.res != nullptr;

  // ---- load, add, round to the bf16 hidden state ---------------------------
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const int c = t + j * T;
    if (c < p.cols8) {
      load_chunk<Y_F32>(p.y, row_chunk0 + c, h[j]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) h[j][e] = 0.0f;
    }
  }
  if (has_res) {
    float rv[V][8];
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const int c = t + j * T;
      if (c < p.cols8) load_chunk<RES_F32>(p.res, row_chunk0 + c, rv[j]);
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const int c = t + j * T;
      if (c < p.cols8) {
#pragma unroll
        for (int e = 0; e < 8; ++e) h[j][e] = __fadd_rn(rv[j][e], __fmul_rn(p.rm, h[j][e]));
      }
    }
  }
  // the norm reads the bf16-rounded hidden state, as the reference's separate norm kernel does
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const uint4 hb = pack8(h[j]);
    unpack8(hb, h[j]);
    if (PHASE != kEncode && live && p.h_out != nullptr) {
      const int c = t + j * T;
      // default cache policy: the second sweep re-reads it
      if (c < p.cols8) reinterpret_cast<uint4*>(p.h_out)[row_chunk0 + c] = hb;
    }
  }

  // ---- sum of squares in double, fixed order ----------------------------------
  // A bf16 value converts to double exactly and its square is exact there; the
  // double sum then carries ~29 spare bits, so float(sum / cols) equals the
  // host's sequential double sum except when the quotient lies within ~1e-13
  // relative of a float rounding boundary.
  double acc = 0.0;
#pragma unroll
  for (int j = 0; j < V; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const double d = static_cast<double>(h[j][e]);
      acc = fma(d, d, acc);
    }
  acc = warp_sum(acc);
  __shared__ double s_part[32];
  __shared__ uint32_t s_amax[32];
  const int warp = t >> 5, lane = t & 31, nwarps = T >> 5;
  if (lane == 0) s_part[warp] = acc;
  __syncthreads();
  double total = 0.0;
  for (int i = 0; i < nwarps; ++i) total += s_part[i];
  const float ms = static_cast<float>(p.inv_cols != 0.0 ? total * p.inv_cols
                                                         : total / static_cast<double>(p.cols));
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, p.eps)));
  if (PHASE != kEncode && live && p.rstd != nullptr && t == 0) p.rstd[row] = r;

  // ---- normalise -----------------------------------------------------------------
  Fp8Scale fs{};
  if (PHASE == kEncode) fs = fp8_scale_from_amax(__ldcg(p.scale_amax + 1));
  uint32_t amax = 0u;
  uint4 kept[PHASE == kCluster ? V : 1];  // kCluster: n stays in registers across the barrier
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const int c = t + j * T;
    if (c < p.cols8) {
      float wv[8], n[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(p.w) + c), wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) n[e] = __fmul_rn(__fmul_rn(h[j][e], r), wv[e]);
      const uint4 nb = pack8(n);
      if (PHASE == kCluster) {
        if (live && p.n_bf16 != nullptr)
          st_stream(reinterpret_cast<uint4*>(p.n_bf16) + row_chunk0 + c, nb);
        kept[PHASE == kCluster ? j : 0] = nb;
        amax = amax_acc(amax, nb);
      } else if (PHASE == kStats) {
        if (p.n_bf16 != nullptr) {
          uint4* dst = reinterpret_cast<uint4*>(p.n_bf16) + row_chunk0 + c;
          if (p.n_fp8 != nullptr) *dst = nb; else st_stream(dst, nb);
        }
        amax = amax_acc(amax, nb);
      } else {
        st_stream(reinterpret_cast<uint2*>(p.n_fp8) + row_chunk0 + c, fp8x8_quant(nb, fs));
      }
    }
  }
  if (PHASE == kStats && p.scale_amax != nullptr) {
    amax = amax_warp(amax);
    if (lane == 0) s_amax[warp] = amax;
    __syncthreads();
    if (t == 0) {
      uint32_t m = 0u;
      for (int i = 0; i < nwarps; ++i) m = max_u16x2(m, s_amax[i]);
      atomic_amax(p.scale_amax + 1, amax_value(m));
    }
  }
  if (PHASE == kEncode && blockIdx.x == 0 && t == 0) p.scale_amax[0] = fs.scale;
  if (PHASE == kCluster) {
    __shared__ uint32_t s_slots[kMaxClusterCtas];
    const float tensor_amax = __uint_as_float(cluster_amax_bits(amax, s_amax, s_slots));
    fs = fp8_scale_from_amax(tensor_amax);
    if (live) {
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const int c = t + j * T;
        if (c < p.cols8)
          st_stream(reinterpret_cast<uint2*>(p.n_fp8) + row_chunk0 + c, fp8x8_quant(kept[PHASE == kCluster ? j : 0], fs));
      }
    }
    if (blockIdx.x == 0 && t == 0) p.scale_amax[0] = fs.scale, p.scale_amax[1] = tensor_amax;
  }
}

// The stats sweep for the shape every launch of the Granite sequence has: bf16 y (and res),
// cols8 == 4 * blockDim.x (a 4096-wide row on 128 threads). Same arithmetic in the same order as
// add_rmsnorm_kernel<false, false, 4, kStats> - the results are bit-identical - with the bounds
// tests, the input-type switches and the unused outputs compiled away.
template <bool HAS_RES, bool WANT_AMAX>
__global__ void __launch_bounds__(256) add_rmsnorm_fast_kernel(const NormParams p) {
  pdl_begin();
  constexpr int V = 4;
  const int T = blockDim.x;
  const int t = threadIdx.x;
  const int row = blockIdx.x;
  const size_t row_chunk0 = static_cast<size_t>(row) * p.cols8;
  const uint4* yp = reinterpret_cast<const uint4*>(p.y) + row_chunk0 + t;
  const uint4* rp = reinterpret_cast<const uint4*>(p.res) + row_chunk0 + t;
  uint4 yraw[V], rraw[V];
#pragma unroll
  for (int j = 0; j < V; ++j) yraw[j] = ld_stream(yp + j * T);
  if (HAS_RES) {
#pragma unroll
    for (int j = 0; j < V; ++j) rraw[j] = ld_stream(rp + j * T);
  }
  float h[V][8];
  double acc = 0.0;
  const bool keep = WANT_AMAX && p.keep_h > 0.0f;
  const uint64_t pol = keep ? l2_policy_evict_last(p.keep_h) : 0ull;
#pragma unroll
  for (int j = 0; j < V; ++j) {
    unpack8(yraw[j], h[j]);
    if (HAS_RES) {
      float rv[8];
      unpack8(rraw[j], rv);
#pragma unroll
      for (int e = 0; e < 8; ++e) h[j][e] = __fadd_rn(rv[e], __fmul_rn(p.rm, h[j][e]));
    }
    const uint4 hb = pack8(h[j]);
    unpack8(hb, h[j]);
    if (p.h_out != nullptr) {
      uint4* dst = reinterpret_cast<uint4*>(p.h_out) + row_chunk0 + t + j * T;
      if (keep) st_l2_hint(dst, hb, pol); else *dst = hb;
    }
  }
#pragma unroll
  for (int j = 0; j < V; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const double d = static_cast<double>(h[j][e]);
      acc = fma(d, d, acc);
    }
  acc = warp_sum(acc);
  __shared__ double s_part[8];
  __shared__ uint32_t s_amax[8];
  const int warp = t >> 5, lane = t & 31, nwarps = T >> 5;
  if (lane == 0) s_part[warp] = acc;
  __syncthreads();
  double total = 0.0;
  for (int i = 0; i < nwarps; ++i) total += s_part[i];
  const float ms = static_cast<float>(p.inv_cols != 0.0 ? total * p.inv_cols
                                                         : total / static_cast<double>(p.cols));
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, p.eps)));
  if (p.rstd != nullptr && t == 0) p.rstd[row] = r;
  if (p.n_bf16 == nullptr && !WANT_AMAX) return;  // h (and r) were all that was asked for
  uint32_t amax = 0u;
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const int c = t + j * T;
    float wv[8], n[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(p.w) + c), wv);
#pragma unroll
    for (int e = 0; e < 8; ++e) n[e] = __fmul_rn(__fmul_rn(h[j][e], r), wv[e]);
    const uint4 nb = pack8(n);
    if (p.n_bf16 != nullptr) {
      uint4* dst = reinterpret_cast<uint4*>(p.n_bf16) + row_chunk0 + c;
      if (WANT_AMAX) *dst = nb; else st_stream(dst, nb);
    }
    if (WANT_AMAX) amax = amax_acc(amax, nb);
  }
  if (WANT_AMAX) {
    amax = amax_warp(amax);
    if (lane == 0) s_amax[warp] = amax;
    __syncthreads();
    if (t == 0) {
      uint32_t m = 0u;
      for (int i = 0; i < nwarps; ++i) m = max_u16x2(m, s_amax[i]);
      atomic_amax(p.scale_amax + 1, amax_value(m));
    }
  }
}

// Second sweep with r known per row: a plain streaming pass. A CTA takes kRowsPerCta
// consecutive rows; a thread takes the chunks t, t + T, ... of each, so every
// thread has kRowsPerCta * ceil(cols8 / T) independent 128-bit loads to issue
// before it needs any of them.
constexpr int kRowsPerCta = 4;
constexpr int kEncodeThreads = 256;
constexpr int kEncodeMaxIter = 2;  // cols8 <= 512 per pass of the unrolled body

// FULL: cols8 == kEncodeThreads * kEncodeMaxIter (a 4096-wide row) and rows a multiple of
// kRowsPerCta - the shape of every launch of the Granite sequence - so that no bounds test is
// left in the loop bodies.
template <bool FULL>
__global__ void __launch_bounds__(kEncodeThreads) norm_encode_kernel(const NormParams p) {
  pdl_begin();
  const int t = threadIdx.x;
  const int tiles = (p.rows + kRowsPerCta - 1) / kRowsPerCta;
  const int tile = p.reverse ? tiles - 1 - static_cast<int>(blockIdx.x) : blockIdx.x;
  const int row0 = tile * kRowsPerCta;
  const Fp8Scale fs = fp8_scale_from_amax(__ldcg(p.scale_amax + 1));
  if (blockIdx.x == 0 && t == 0) p.scale_amax[0] = fs.scale;
  const uint4* h = reinterpret_cast<const uint4*>(p.h_out);
  uint2* out = reinterpret_cast<uint2*>(p.n_fp8);
  const bool kept = p.keep_h > 0.0f;
  const uint64_t pol = kept ? l2_policy_evict_first() : 0ull;  // h was held for this read: let go of it
  const int pass_cols = kEncodeThreads * kEncodeMaxIter;
  for (int c0 = 0; c0 < (FULL ? pass_cols : p.cols8); c0 += pass_cols) {
    uint4 hv[kRowsPerCta][kEncodeMaxIter];
    uint4 wv[kEncodeMaxIter];
    float rr[kRowsPerCta];
#pragma unroll
    for (int k = 0; k < kEncodeMaxIter; ++k) {
      const int c = c0 + k * kEncodeThreads + t;
      if (FULL || c < p.cols8) {
        wv[k] = __ldg(reinterpret_cast<const uint4*>(p.w) + c);
#pragma unroll
        for (int j = 0; j < kRowsPerCta; ++j)
          if (FULL || row0 + j < p.rows) {
            const uint4* src = h + static_cast<size_t>(row0 + j) * p.cols8 + c;
            hv[j][k] = kept ? ld_l2_hint(src, pol) : ld_stream(src);
          }
      }
    }
#pragma unroll
    for (int j = 0; j < kRowsPerCta; ++j) rr[j] = (FULL || row0 + j < p.rows) ? __ldg(p.rstd + row0 + j) : 0.0f;
#pragma unroll
    for (int k = 0; k < kEncodeMaxIter; ++k) {
      const int c = c0 + k * kEncodeThreads + t;
      if (!FULL && c >= p.cols8) continue;
      float wf[8];
      unpack8(wv[k], wf);  // once per column chunk, shared by the rows
#pragma unroll
      for (int j = 0; j < kRowsPerCta; ++j) {
        if (!FULL && row0 + j >= p.rows) continue;
        float hf[8], n[8];
        unpack8(hv[j][k], hf);
#pragma unroll
        for (int e = 0; e < 8; ++e) n[e] = __fmul_rn(__fmul_rn(hf[e], rr[j]), wf[e]);
        st_stream(out + static_cast<size_t>(row0 + j) * p.cols8 + c, fp8x8_quant(pack8(n), fs));
      }
    }
  }
}

// Any cols, any alignment: one CTA per row, scalar accesses, the row re-read
// for the normalise step. Only shapes the vector kernel cannot take land here
// (cols not a multiple of 8, misaligned rows, rows wider than 32 K elements).
__global__ void __launch_bounds__(256)
    rmsnorm_generic_kernel(const uint16_t* x, const uint16_t* w, float eps, int cols, uint16_t* out) {
  const size_t base = static_cast<size_t>(blockIdx.x) * cols;
  double acc = 0.0;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const double v = static_cast<double>(bf16_to_f32(x[base + c]));
    acc = fma(v, v, acc);
  }
  acc = warp_sum(acc);
  __shared__ double s_part[8];
  if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
  __syncthreads();
  double total = 0.0;
  for (int i = 0; i < 8; ++i) total += s_part[i];
  const float ms = static_cast<float>(total / static_cast<double>(cols));
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)));
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = bf16_to_f32(x[base + c]);
    out[base + c] = static_cast<uint16_t>(
        f32_to_bf16_bits(__fmul_rn(__fmul_rn(v, r), bf16_to_f32(w[c]))));
  }
}

// Elementwise per-tensor FP8 of a bf16 tensor: amax sweep, then encode sweep.
constexpr int kQuantUnroll = 4;
__global__ void __launch_bounds__(256) amax_bf16_kernel(const uint4* x, long long n8, float* scale_amax) {
  pdl_begin();
  uint32_t amax = 0u;
  const long long base = static_cast<long long>(blockIdx.x) * (256 * kQuantUnroll) + threadIdx.x;
  uint4 v[kQuantUnroll];
#pragma unroll
  for (int k = 0; k < kQuantUnroll; ++k) {
    const long long i = base + k * 256;
    v[k] = i < n8 ? __ldg(x + i) : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int k = 0; k < kQuantUnroll; ++k) amax = amax_acc(amax, v[k]);
  amax = amax_warp(amax);
  __shared__ uint32_t s[8];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t m = 0u;
    for (int i = 0; i < 8; ++i) m = max_u16x2(m, s[i]);
    atomic_amax(scale_amax + 1, amax_value(m));
  }
}

__global__ void __launch_bounds__(256)
    encode_bf16_kernel(const uint4* x, long long n8, uint2* codes, float* scale_amax) {
  pdl_begin();
  const Fp8Scale fs = fp8_scale_from_amax(__ldcg(scale_amax + 1));
  if (blockIdx.x == 0 && threadIdx.x == 0) scale_amax[0] = fs.scale;
  // last element first: the tail of the tensor is what the amax sweep left in L2
  const long long base = static_cast<long long>(blockIdx.x) * (256 * kQuantUnroll) + threadIdx.x;
  uint4 v[kQuantUnroll];
#pragma unroll
  for (int k = 0; k < kQuantUnroll; ++k) {
    const long long i = n8 - 1 - (base + k * 256);
    if (i >= 0) v[k] = ld_stream(x + i);
  }
#pragma unroll
  for (int k = 0; k < kQuantUnroll; ++k) {
    const long long i = n8 - 1 - (base + k * 256);
    if (i >= 0) st_stream(codes + i, fp8x8_quant(v[k], fs));
  }
}

// The same for a decode-size tensor (up to 16 rows of 4096): one CTA keeps the tensor in registers,
// finds max |x| through shared memory and encodes - one launch instead of a memset and two sweeps.
constexpr int kQuantSmallThreads = 1024, kQuantSmallItems = 8;
__global__ void __launch_bounds__(kQuantSmallThreads)
    quant_small_kernel(const uint4* x, int n8, uint2* codes, float* scale_amax) {
  pdl_begin();
  __shared__ uint32_t s[kQuantSmallThreads / 32];
  uint4 v[kQuantSmallItems];
  uint32_t amax = 0u;
#pragma unroll
  for (int k = 0; k < kQuantSmallItems; ++k) {
    const int i = k * kQuantSmallThreads + threadIdx.x;
    v[k] = i < n8 ? __ldg(x + i) : make_uint4(0, 0, 0, 0);
    amax = amax_acc(amax, v[k]);
  }
  amax = amax_warp(amax);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = amax;
  __syncthreads();
  uint32_t m = s[threadIdx.x & 31];
  m = amax_warp(m);
  const float a = amax_value(m);
  const Fp8Scale fs = fp8_scale_from_amax(a);
  if (threadIdx.x == 0) scale_amax[0] = fs.scale, scale_amax[1] = a;
#pragma unroll
  for (int k = 0; k < kQuantSmallItems; ++k) {
    const int i = k * kQuantSmallThreads + threadIdx.x;
    if (i < n8) codes[i] = fp8x8_quant(v[k], fs);
  }
}

int env_int(const char* name, int fallback) {
  const char* v = std::getenv(name);
  return (v != nullptr && *v != '\0') ? std::atoi(v) : fallback;
}

// Chunks per thread: 4 keeps a 4096-wide row in one 128-thread CTA with eight
// 128-bit loads in flight per thread. G4_NORM_V overrides it for A/B runs.
int pick_v(int cols8) {
  static const int forced = env_int("G4_NORM_V", 0);
  if (forced == 1 || forced == 2 || forced == 4 || forced == 8) {
    if ((cols8 + forced - 1) / forced <= max_threads_for(forced)) return forced;
  }
  if (cols8 <= 64) return 1;
  if (cols8 <= 256) return 2;
  if (cols8 <= 4 * max_threads_for(4)) return 4;
  return 8;
}
constexpr int kMaxVectorCols = 8 * 8 * max_threads_for(8);  // 32768

template <bool Y_F32, bool RES_F32, int PHASE>
cudaError_t launch_v(const NormParams& p, int V, int threads, cudaStream_t st) {
  const dim3 grid(static_cast<unsigned>(p.rows)), block(static_cast<unsigned>(threads));
  switch (V) {
    case 1: return launch_pdl(add_rmsnorm_kernel<Y_F32, RES_F32, 1, PHASE>, grid, block, 0, st, p);
    case 2: return launch_pdl(add_rmsnorm_kernel<Y_F32, RES_F32, 2, PHASE>, grid, block, 0, st, p);
    case 4: return launch_pdl(add_rmsnorm_kernel<Y_F32, RES_F32, 4, PHASE>, grid, block, 0, st, p);
    default: return launch_pdl(add_rmsnorm_kernel<Y_F32, RES_F32, 8, PHASE>, grid, block, 0, st, p);
  }
}

template <int PHASE>
cudaError_t launch_phase(const NormParams& p, bool y_f32, bool res_f32, cudaStream_t st) {
  const int V = pick_v(p.cols8);
  const int threads = ((p.cols8 + V - 1) / V + 31) / 32 * 32;
  if (y_f32) {
    if (res_f32) return launch_v<true, true, PHASE>(p, V, threads, st);
    return launch_v<true, false, PHASE>(p, V, threads, st);
  }
  if (res_f32) return launch_v<false, true, PHASE>(p, V, threads, st);
  return launch_v<false, false, PHASE>(p, V, threads, st);
}

long long quant_grid(long long n8) { return (n8 + 256 * kQuantUnroll - 1) / (256 * kQuantUnroll); }

}  // namespace

// Shared by the kept rmsnorm entry points and the fused one.
int add_rmsnorm_launch(const char* fn, const void* d_y, int y_is_f32, const void* d_res,
                       int res_is_f32, const uint16_t* d_w, float eps, float rm, int rows, int cols,
                       uint16_t* d_h_out, uint16_t* d_n_bf16, uint8_t* d_n_fp8,
                       float* d_scale_amax, float* d_rstd) {
  cudaStream_t st = current_stream();
  NormParams p{};
  p.y = d_y, p.res = d_res, p.w = d_w, p.h_out = d_h_out, p.n_bf16 = d_n_bf16, p.n_fp8 = d_n_fp8;
  p.scale_amax = d_n_fp8 != nullptr ? d_scale_amax : nullptr;
  p.rstd = d_rstd;
  p.eps = eps, p.rm = rm, p.rows = rows, p.cols = cols, p.cols8 = cols / 8, p.reverse = 0;
  p.inv_cols = (cols & (cols - 1)) == 0 ? 1.0 / static_cast<double>(cols) : 0.0;
  // the rstd form of the second sweep re-reads h: hold as much of it in L2 as is likely to fit
  p.keep_h = (d_n_fp8 != nullptr && d_n_bf16 == nullptr && d_h_out != nullptr && d_rstd != nullptr)
                 ? l2_keep_fraction(static_cast<double>(rows) * cols * 2.0) : 0.0f;
  if (d_n_fp8 != nullptr && rows <= kMaxClusterCtas && p.cols8 <= max_threads_for(1) && cluster_enabled()) {
    const int ctas = cluster_ctas_for(rows);
    const int threads = (p.cols8 + 31) / 32 * 32;
    cudaError_t e;
    if (y_is_f32) {
      e = res_is_f32 ? cluster_launch(add_rmsnorm_kernel<true, true, 1, kCluster>, ctas, threads, p, st)
                     : cluster_launch(add_rmsnorm_kernel<true, false, 1, kCluster>, ctas, threads, p, st);
    } else {
      e = res_is_f32 ? cluster_launch(add_rmsnorm_kernel<false, true, 1, kCluster>, ctas, threads, p, st)
                     : cluster_launch(add_rmsnorm_kernel<false, false, 1, kCluster>, ctas, threads, p, st);
    }
    if (e == cudaSuccess) return 0;
    if (e != cudaErrorInvalidConfiguration) {
      std::fprintf(stderr, "granite4: %s: cluster launch failed: %s\n", fn, cudaGetErrorString(e));
      return -1;
    }
    // the device cannot place such a cluster: the multi-launch form below takes over
  }
  if (d_n_fp8 != nullptr && !amax_prezeroed())
    G4_CUDA_TRY(fn, cudaMemsetAsync(d_scale_amax, 0, 2 * sizeof(float), st));
  const int fast_threads = p.cols8 / 4;
  const bool fast = !y_is_f32 && (d_res == nullptr || !res_is_f32) && p.cols8 % 4 == 0 &&
                    fast_threads % 32 == 0 && fast_threads <= 256 && pick_v(p.cols8) == 4;
  if (fast) {
    const bool amax = p.scale_amax != nullptr;
    const dim3 grid(static_cast<unsigned>(rows)), block(static_cast<unsigned>(fast_threads));
    if (d_res != nullptr) {
      if (amax) G4_LAUNCH_PDL(fn, add_rmsnorm_fast_kernel<true, true>, grid, block, 0, st, p);
      else G4_LAUNCH_PDL(fn, add_rmsnorm_fast_kernel<true, false>, grid, block, 0, st, p);
    } else {
      if (amax) G4_LAUNCH_PDL(fn, add_rmsnorm_fast_kernel<false, true>, grid, block, 0, st, p);
      else G4_LAUNCH_PDL(fn, add_rmsnorm_fast_kernel<false, false>, grid, block, 0, st, p);
    }
  } else {
    G4_CUDA_TRY(fn, launch_phase<kStats>(p, y_is_f32 != 0, res_is_f32 != 0, st));
  }
  if (d_n_fp8 != nullptr) {
    if (d_n_bf16 != nullptr) {
      // n already sits in memory as bf16: encode it elementwise.
      const long long n8 = static_cast<long long>(rows) * (cols / 8);
      G4_LAUNCH_PDL(fn, encode_bf16_kernel, dim3(static_cast<unsigned>(quant_grid(n8))), dim3(256), 0, st,
                    reinterpret_cast<const uint4*>(d_n_bf16), n8, reinterpret_cast<uint2*>(d_n_fp8),
                    d_scale_amax);
    } else if (d_h_out != nullptr && d_rstd != nullptr) {
      NormParams q = p;
      q.reverse = 1;
      const unsigned grid = static_cast<unsigned>((rows + kRowsPerCta - 1) / kRowsPerCta);
      if (q.cols8 == kEncodeThreads * kEncodeMaxIter && rows % kRowsPerCta == 0)
        G4_LAUNCH_PDL(fn, norm_encode_kernel<true>, dim3(grid), dim3(kEncodeThreads), 0, st, q);
      else
        G4_LAUNCH_PDL(fn, norm_encode_kernel<false>, dim3(grid), dim3(kEncodeThreads), 0, st, q);
    } else {
      NormParams q = p;
      q.reverse = 1;
      if (d_h_out != nullptr) {  // re-read the bf16 hidden state, not y and res
        q.y = d_h_out, q.res = nullptr;
        G4_CUDA_TRY(fn, launch_phase<kEncode>(q, false, false, st));
      } else {
        G4_CUDA_TRY(fn, launch_phase<kEncode>(q, y_is_f32 != 0, res_is_f32 != 0, st));
      }
    }
  }
  return 0;
}

int max_vector_cols() { return kMaxVectorCols; }

int rmsnorm_entry(const char* fn, const uint16_t* d_x, const uint16_t* d_w, float eps, int rows,
                  int cols, uint16_t* d_out, int max_rows) {
  if (d_x == nullptr || d_w == nullptr || d_out == nullptr || !std::isfinite(eps) || eps <= 0.0f ||
      rows <= 0 || rows > max_rows || cols <= 0 || static_cast<long long>(rows) * cols > INT_MAX)
    return fail(fn, "invalid arguments");
  const bool vec = (cols % 8 == 0) && cols <= kMaxVectorCols && aligned16(d_x) && aligned16(d_w) &&
                   aligned16(d_out);
  if (!vec) {
    rmsnorm_generic_kernel<<<rows, 256, 0, current_stream()>>>(d_x, d_w, eps, cols, d_out);
    G4_LAUNCH_CHECK(fn);
    return 0;
  }
  return add_rmsnorm_launch(fn, d_x, 0, nullptr, 0, d_w, eps, 1.0f, rows, cols, nullptr, d_out,
                            nullptr, nullptr, nullptr);
}

}  // namespace g4

extern "C" {

int granite4_kernel_rmsnorm(const uint16_t* d_x, const uint16_t* d_w, float eps, int rows, int cols,
                            uint16_t* d_out) {
  return g4::rmsnorm_entry("granite4_kernel_rmsnorm", d_x, d_w, eps, rows, cols, d_out, INT_MAX);
}

int granite4_kernel_rmsnorm_batched(const uint16_t* d_x, const uint16_t* d_w, float eps, int rows,
                                    int cols, uint16_t* d_out) {
  return g4::rmsnorm_entry("granite4_kernel_rmsnorm_batched", d_x, d_w, eps, rows, cols, d_out,
                           GRANITE4_MAX_VERIFY_ROWS);
}

int granite4_kernel_add_rmsnorm_fp8(const void* d_y, int y_is_f32, const void* d_res,
                                    int res_is_f32, const uint16_t* d_w, float eps,
                                    float resid_mult, int rows, int cols, uint16_t* d_h_out,
                                    uint16_t* d_n_bf16, uint8_t* d_n_fp8, float* d_scale_amax,
                                    float* d_rstd) {
  const char* fn = "granite4_kernel_add_rmsnorm_fp8";
  if (d_y == nullptr || d_w == nullptr || !std::isfinite(eps) || eps <= 0.0f ||
      !std::isfinite(resid_mult) || rows <= 0 || cols <= 0 ||
      static_cast<long long>(rows) * cols > INT_MAX)
    return g4::fail(fn, "invalid arguments");
  if (d_h_out == nullptr && d_n_bf16 == nullptr && d_n_fp8 == nullptr)
    return g4::fail(fn, "no output requested");
  if (d_n_fp8 != nullptr && d_scale_amax == nullptr)
    return g4::fail(fn, "FP8 output needs d_scale_amax");
  if (cols % 8 != 0 || cols > g4::max_vector_cols())
    return g4::fail(fn, "cols must be a multiple of 8 and at most 32768");
  if (!g4::aligned16(d_y) || !g4::aligned16(d_res) || !g4::aligned16(d_w) ||
      !g4::aligned16(d_h_out) || !g4::aligned16(d_n_bf16) || !g4::aligned16(d_n_fp8))
    return g4::fail(fn, "pointers must be 16-byte aligned");
  return g4::add_rmsnorm_launch(fn, d_y, y_is_f32, d_res, res_is_f32, d_w, eps, resid_mult, rows,
                                cols, d_h_out, d_n_bf16, d_n_fp8, d_scale_amax, d_rstd);
}

int granite4_kernel_fp8_quant(const uint16_t* d_x, long long n, uint8_t* d_codes,
                              float* d_scale_amax) {
  const char* fn = "granite4_kernel_fp8_quant";
  if (d_x == nullptr || d_codes == nullptr || d_scale_amax == nullptr || n <= 0 || n % 8 != 0 ||
      !g4::aligned16(d_x) || !g4::aligned16(d_codes))
    return g4::fail(fn, "invalid arguments");
  cudaStream_t st = g4::current_stream();
  const long long n8 = n / 8;
  const long long grid = g4::quant_grid(n8);
  if (grid > INT_MAX) return g4::fail(fn, "tensor too large");
  if (n8 <= g4::kQuantSmallThreads * g4::kQuantSmallItems && g4::cluster_enabled()) {  // G4_CLUSTER=0: the two-sweep form
    G4_LAUNCH_PDL(fn, g4::quant_small_kernel, dim3(1), dim3(g4::kQuantSmallThreads), 0, st,
                  reinterpret_cast<const uint4*>(d_x), static_cast<int>(n8), reinterpret_cast<uint2*>(d_codes),
                  d_scale_amax);
    return 0;
  }
  G4_CUDA_TRY(fn, cudaMemsetAsync(d_scale_amax, 0, 2 * sizeof(float), st));
  G4_LAUNCH_PDL(fn, g4::amax_bf16_kernel, dim3(static_cast<unsigned>(grid)), dim3(256), 0, st,
                reinterpret_cast<const uint4*>(d_x), n8, d_scale_amax);
  G4_LAUNCH_PDL(fn, g4::encode_bf16_kernel, dim3(static_cast<unsigned>(grid)), dim3(256), 0, st,
                reinterpret_cast<const uint4*>(d_x), n8, reinterpret_cast<uint2*>(d_codes), d_scale_amax);
  return 0;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// The fused add + norm + FP8 op for callers that cannot hand over scratch memory.
//
// Some hosts of this library have no way to allocate device memory when the call is made: a
// serving engine that carved up the whole card at start-up (the reference engine sizes its KV
// arena to what is left of the 16 GB and its launchers allocate nothing by convention), or a
// thin binding from another language (ctypes, cgo) that loads this library but not the CUDA
// runtime, so it has no cudaMalloc of its own to call. granite4_kernel_add_rmsnorm_fp8 asks such
// a caller for the per-row 1/rms buffer if it wants the cheap second sweep; this variant keeps
// that buffer inside the library instead, in a fixed array that every GPU loading the library
// holds until the process exits.
constexpr int kNoAllocMaxRows = 65536;  // 256 KB of scratch per device
static __device__ __align__(256) float g_noalloc_rstd[kNoAllocMaxRows];

namespace g4 {
namespace {
// Device address of g_noalloc_rstd on each device. In host code the array's name is only a
// handle for the runtime, not an address a kernel can use; the address is looked up once per
// device, with that device current, and cached.
std::atomic<float*> g_noalloc_rstd_ptr[64];  // relaxed: any thread may fill it, all with the same value

float* noalloc_rstd_ptr(const char* fn) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    fail(fn, "cannot identify the current device");
    return nullptr;
  }
  float* known = g_noalloc_rstd_ptr[dev].load(std::memory_order_relaxed);
  if (known == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_rstd);
    if (e != cudaSuccess || p == nullptr) {
      std::fprintf(stderr, "granite4: %s: cudaGetSymbolAddress failed: %s\n", fn,
                   cudaGetErrorString(e));
      return nullptr;
    }
    known = static_cast<float*>(p);
    g_noalloc_rstd_ptr[dev].store(known, std::memory_order_relaxed);
  }
  return known;
}
}  // namespace
}  // namespace g4

extern "C" {

// The first call on a device looks up the scratch array's device address (one
// cudaGetSymbolAddress); make that first call before starting any stream capture. Calls share
// the one array per device: two calls whose kernels can overlap on the GPU (different streams,
// no dependency between them) race on it. Nothing is allocated or freed, here or by anything
// this calls.
int granite4_kernel_add_rmsnorm_fp8_noalloc(const void* d_y, int y_is_f32, const void* d_res,
                                            int res_is_f32, const uint16_t* d_w, float eps,
                                            float resid_mult, int rows, int cols,
                                            uint16_t* d_h_out, uint8_t* d_n_fp8,
                                            float* d_scale_amax) {
  const char* fn = "granite4_kernel_add_rmsnorm_fp8_noalloc";
  if (d_y == nullptr || d_w == nullptr || d_h_out == nullptr || d_n_fp8 == nullptr ||
      d_scale_amax == nullptr || !std::isfinite(eps) || eps <= 0.0f || !std::isfinite(resid_mult) ||
      rows <= 0 || cols <= 0 || static_cast<long long>(rows) * cols > INT_MAX)
    return g4::fail(fn, "invalid arguments");
  if (rows > kNoAllocMaxRows)
    return g4::fail(fn, "more than 65536 rows: the built-in scratch holds one float per row for at "
                        "most 65536 rows; split the batch or use granite4_kernel_add_rmsnorm_fp8 with "
                        "your own d_rstd");
  if (cols % 8 != 0 || cols > g4::max_vector_cols())
    return g4::fail(fn, "cols must be a multiple of 8 and at most 32768");
  if (!g4::aligned16(d_y) || !g4::aligned16(d_res) || !g4::aligned16(d_w) ||
      !g4::aligned16(d_h_out) || !g4::aligned16(d_n_fp8))
    return g4::fail(fn, "pointers must be 16-byte aligned");
  float* rstd = g4::noalloc_rstd_ptr(fn);
  if (rstd == nullptr) return -1;
  // The first sweep writes rstd[0 .. rows) in full before the second sweep reads it, so nothing
  // in the shared array has to be cleared between calls.
  return g4::add_rmsnorm_launch(fn, d_y, y_is_f32, d_res, res_is_f32, d_w, eps, resid_mult, rows,
                                cols, d_h_out, nullptr, d_n_fp8, d_scale_amax, rstd);
}

}  // extern "C"
