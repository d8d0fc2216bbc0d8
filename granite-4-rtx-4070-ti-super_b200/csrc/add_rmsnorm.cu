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
// One CTA owns one row; a thread owns V chunks of 8 elements (one 128-bit load
// each for bf16, two for f32), strided by the CTA width so a warp reads 512
// contiguous bytes per load. The row stays in registers between the reduction
// and the normalise step, so each input byte is read once per sweep.
//
// The FP8 scale depends on every row, so FP8 output takes two sweeps: the
// stats sweep writes h (and n as bf16 if asked) and folds max |n| into
// d_scale_amax[1] with an integer atomicMax; the encode sweep re-reads the
// bf16 hidden state (8 KB per row instead of the 16 KB of y and res), repeats
// the same reduction in the same order (so n is bit-identical) and writes the
// codes. The encode sweep walks the rows backwards: the rows the stats sweep
// wrote last are the ones most likely still in L2.
//
// Algorithmic bytes per row at cols = 4096, bf16 y and res, h + FP8 out:
// 8192 + 8192 read, 8192 + 4096 written = 28 672; the encode sweep adds a
// second 8192-byte read of h.
#include "g4_host.h"
#include "g4_math.cuh"

#include "../../include/granite4_b200.h"

#include <algorithm>
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
  float eps;
  float rm;
  int rows;
  int cols8;  // cols / 8
  int cols;
  int reverse;  // walk rows from the last to the first
};

enum { kStats = 0, kEncode = 1 };

// Load one 8-element chunk as floats.
template <bool F32>
__device__ __forceinline__ void load_chunk(const void* base, size_t chunk, float (&v)[8]) {
  if (F32) {
    const float4* p = reinterpret_cast<const float4*>(base) + 2 * chunk;
    const float4 a = ld_stream(p), b = ld_stream(p + 1);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w;
    v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  } else {
    const uint4 u = ld_stream(reinterpret_cast<const uint4*>(base) + chunk);
    v[0] = bf16_lo(u.x), v[1] = bf16_hi(u.x), v[2] = bf16_lo(u.y), v[3] = bf16_hi(u.y);
    v[4] = bf16_lo(u.z), v[5] = bf16_hi(u.z), v[6] = bf16_lo(u.w), v[7] = bf16_hi(u.w);
  }
}

// Widest CTA each V is launched with (pick_v keeps to it).
constexpr int max_threads_for(int V) { return V == 1 ? 1024 : (V == 4 ? 256 : 512); }

template <bool Y_F32, bool RES_F32, int V, int PHASE>
__global__ void __launch_bounds__(max_threads_for(V))
    add_rmsnorm_kernel(const NormParams p) {
  const int T = blockDim.x;
  const int t = threadIdx.x;
  const int row = p.reverse ? p.rows - 1 - static_cast<int>(blockIdx.x) : blockIdx.x;
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
  uint4 hb[V];
#pragma unroll
  for (int j = 0; j < V; ++j) {
    hb[j].x = pack_bf16x2(h[j][0], h[j][1]);
    hb[j].y = pack_bf16x2(h[j][2], h[j][3]);
    hb[j].z = pack_bf16x2(h[j][4], h[j][5]);
    hb[j].w = pack_bf16x2(h[j][6], h[j][7]);
    h[j][0] = bf16_lo(hb[j].x), h[j][1] = bf16_hi(hb[j].x);
    h[j][2] = bf16_lo(hb[j].y), h[j][3] = bf16_hi(hb[j].y);
    h[j][4] = bf16_lo(hb[j].z), h[j][5] = bf16_hi(hb[j].z);
    h[j][6] = bf16_lo(hb[j].w), h[j][7] = bf16_hi(hb[j].w);
  }
  if (PHASE == kStats && p.h_out != nullptr) {
    uint4* dst = reinterpret_cast<uint4*>(p.h_out) + row_chunk0;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const int c = t + j * T;
      if (c < p.cols8) dst[c] = hb[j];  // default policy: the encode sweep re-reads it
    }
  }

  // ---- sum of squares in double, fixed order ----------------------------------
  // Each square of a bf16 value is exact in f32; the double sum then carries
  // ~29 spare bits, so float(sum / cols) equals the host's sequential double
  // sum except when the quotient lies within ~1e-13 relative of a float
  // rounding boundary.
  double acc = 0.0;
#pragma unroll
  for (int j = 0; j < V; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += static_cast<double>(__fmul_rn(h[j][e], h[j][e]));
  acc = warp_sum(acc);
  __shared__ double s_part[32];
  __shared__ float s_amax[32];
  const int warp = t >> 5, lane = t & 31, nwarps = T >> 5;
  if (lane == 0) s_part[warp] = acc;
  __syncthreads();
  double total = 0.0;
  for (int i = 0; i < nwarps; ++i) total += s_part[i];
  const float ms = static_cast<float>(total / static_cast<double>(p.cols));
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, p.eps)));

  // ---- normalise -----------------------------------------------------------------
  float scale = 0.0f;
  if (PHASE == kEncode) scale = fp8_scale_from_amax(__ldcg(p.scale_amax + 1));
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < V; ++j) {
    const int c = t + j * T;
    if (c < p.cols8) {
      const uint4 wu = __ldg(reinterpret_cast<const uint4*>(p.w) + c);
      float wv[8] = {bf16_lo(wu.x), bf16_hi(wu.x), bf16_lo(wu.y), bf16_hi(wu.y),
                     bf16_lo(wu.z), bf16_hi(wu.z), bf16_lo(wu.w), bf16_hi(wu.w)};
      float n[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) n[e] = __fmul_rn(__fmul_rn(h[j][e], r), wv[e]);
      uint4 nb;
      nb.x = pack_bf16x2(n[0], n[1]);
      nb.y = pack_bf16x2(n[2], n[3]);
      nb.z = pack_bf16x2(n[4], n[5]);
      nb.w = pack_bf16x2(n[6], n[7]);
      if (PHASE == kStats) {
        if (p.n_bf16 != nullptr) {
          uint4* dst = reinterpret_cast<uint4*>(p.n_bf16) + row_chunk0 + c;
          if (p.n_fp8 != nullptr) *dst = nb; else st_stream(dst, nb);
        }
        // |bf16| as bits: clear the two sign bits and take the integer max.
        const uint32_t m0 = nb.x & 0x7fff7fffu, m1 = nb.y & 0x7fff7fffu;
        const uint32_t m2 = nb.z & 0x7fff7fffu, m3 = nb.w & 0x7fff7fffu;
        amax = fmaxf(amax, fmaxf(fmaxf(bf16_lo(m0), bf16_hi(m0)), fmaxf(bf16_lo(m1), bf16_hi(m1))));
        amax = fmaxf(amax, fmaxf(fmaxf(bf16_lo(m2), bf16_hi(m2)), fmaxf(bf16_lo(m3), bf16_hi(m3))));
      } else {
        uint2 codes;
        codes.x = fp8x4_quant(bf16_lo(nb.x), bf16_hi(nb.x), bf16_lo(nb.y), bf16_hi(nb.y), scale);
        codes.y = fp8x4_quant(bf16_lo(nb.z), bf16_hi(nb.z), bf16_lo(nb.w), bf16_hi(nb.w), scale);
        st_stream(reinterpret_cast<uint2*>(p.n_fp8) + row_chunk0 + c, codes);
      }
    }
  }
  if (PHASE == kStats && p.scale_amax != nullptr) {
    amax = warp_max(amax);
    if (lane == 0) s_amax[warp] = amax;
    __syncthreads();
    if (t == 0) {
      float m = 0.0f;
      for (int i = 0; i < nwarps; ++i) m = fmaxf(m, s_amax[i]);
      atomic_amax(p.scale_amax + 1, m);
    }
  }
  if (PHASE == kEncode && blockIdx.x == 0 && t == 0) p.scale_amax[0] = scale;
}

// Any cols, any alignment: one CTA per row, scalar accesses, the row re-read
// for the normalise step. Only shapes the vector kernel cannot take land here
// (cols not a multiple of 8, misaligned rows, rows wider than 32 K elements).
__global__ void __launch_bounds__(256)
    rmsnorm_generic_kernel(const uint16_t* x, const uint16_t* w, float eps, int cols, uint16_t* out) {
  const size_t base = static_cast<size_t>(blockIdx.x) * cols;
  double acc = 0.0;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = bf16_to_f32(x[base + c]);
    acc += static_cast<double>(__fmul_rn(v, v));
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
__global__ void __launch_bounds__(256) amax_bf16_kernel(const uint4* x, long long n8, float* scale_amax) {
  float amax = 0.0f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 u = __ldg(x + i);
    const uint32_t m0 = u.x & 0x7fff7fffu, m1 = u.y & 0x7fff7fffu, m2 = u.z & 0x7fff7fffu,
                   m3 = u.w & 0x7fff7fffu;
    amax = fmaxf(amax, fmaxf(fmaxf(bf16_lo(m0), bf16_hi(m0)), fmaxf(bf16_lo(m1), bf16_hi(m1))));
    amax = fmaxf(amax, fmaxf(fmaxf(bf16_lo(m2), bf16_hi(m2)), fmaxf(bf16_lo(m3), bf16_hi(m3))));
  }
  amax = warp_max(amax);
  __shared__ float s[8];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.0f;
    for (int i = 0; i < 8; ++i) m = fmaxf(m, s[i]);
    atomic_amax(scale_amax + 1, m);
  }
}

__global__ void __launch_bounds__(256)
    encode_bf16_kernel(const uint4* x, long long n8, uint2* codes, float* scale_amax) {
  const float scale = fp8_scale_from_amax(__ldcg(scale_amax + 1));
  if (blockIdx.x == 0 && threadIdx.x == 0) scale_amax[0] = scale;
  // last element first: the tail of the tensor is what the amax sweep left in L2
  for (long long k = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; k < n8;
       k += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long i = n8 - 1 - k;
    const uint4 u = ld_stream(x + i);
    uint2 c;
    c.x = fp8x4_quant(bf16_lo(u.x), bf16_hi(u.x), bf16_lo(u.y), bf16_hi(u.y), scale);
    c.y = fp8x4_quant(bf16_lo(u.z), bf16_hi(u.z), bf16_lo(u.w), bf16_hi(u.w), scale);
    st_stream(codes + i, c);
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
void launch_v(const NormParams& p, int V, int threads, cudaStream_t st) {
  switch (V) {
    case 1: add_rmsnorm_kernel<Y_F32, RES_F32, 1, PHASE><<<p.rows, threads, 0, st>>>(p); break;
    case 2: add_rmsnorm_kernel<Y_F32, RES_F32, 2, PHASE><<<p.rows, threads, 0, st>>>(p); break;
    case 4: add_rmsnorm_kernel<Y_F32, RES_F32, 4, PHASE><<<p.rows, threads, 0, st>>>(p); break;
    default: add_rmsnorm_kernel<Y_F32, RES_F32, 8, PHASE><<<p.rows, threads, 0, st>>>(p); break;
  }
}

template <int PHASE>
void launch_phase(const NormParams& p, bool y_f32, bool res_f32, cudaStream_t st) {
  const int V = pick_v(p.cols8);
  const int threads = ((p.cols8 + V - 1) / V + 31) / 32 * 32;
  if (y_f32) {
    if (res_f32) launch_v<true, true, PHASE>(p, V, threads, st);
    else launch_v<true, false, PHASE>(p, V, threads, st);
  } else {
    if (res_f32) launch_v<false, true, PHASE>(p, V, threads, st);
    else launch_v<false, false, PHASE>(p, V, threads, st);
  }
}

}  // namespace

// Shared by the kept rmsnorm entry points and the fused one.
int add_rmsnorm_launch(const char* fn, const void* d_y, int y_is_f32, const void* d_res,
                       int res_is_f32, const uint16_t* d_w, float eps, float rm, int rows, int cols,
                       uint16_t* d_h_out, uint16_t* d_n_bf16, uint8_t* d_n_fp8,
                       float* d_scale_amax) {
  cudaStream_t st = current_stream();
  NormParams p{};
  p.y = d_y, p.res = d_res, p.w = d_w, p.h_out = d_h_out, p.n_bf16 = d_n_bf16, p.n_fp8 = d_n_fp8;
  p.scale_amax = d_n_fp8 != nullptr ? d_scale_amax : nullptr;
  p.eps = eps, p.rm = rm, p.rows = rows, p.cols = cols, p.cols8 = cols / 8, p.reverse = 0;
  if (d_n_fp8 != nullptr)
    G4_CUDA_TRY(fn, cudaMemsetAsync(d_scale_amax, 0, 2 * sizeof(float), st));
  launch_phase<kStats>(p, y_is_f32 != 0, res_is_f32 != 0, st);
  G4_LAUNCH_CHECK(fn);
  if (d_n_fp8 != nullptr) {
    if (d_n_bf16 != nullptr) {
      // n already sits in memory as bf16: encode it elementwise.
      const long long n8 = static_cast<long long>(rows) * (cols / 8);
      const int grid = static_cast<int>(std::min<long long>((n8 + 255) / 256, sm_count() * 16LL));
      encode_bf16_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint4*>(d_n_bf16), n8,
                                               reinterpret_cast<uint2*>(d_n_fp8), d_scale_amax);
    } else {
      NormParams q = p;
      q.reverse = 1;
      if (d_h_out != nullptr) {  // re-read the bf16 hidden state, not y and res
        q.y = d_h_out, q.res = nullptr;
        launch_phase<kEncode>(q, false, false, st);
      } else {
        launch_phase<kEncode>(q, y_is_f32 != 0, res_is_f32 != 0, st);
      }
    }
    G4_LAUNCH_CHECK(fn);
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
                            nullptr, nullptr);
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
                                    uint16_t* d_n_bf16, uint8_t* d_n_fp8, float* d_scale_amax) {
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
                                cols, d_h_out, d_n_bf16, d_n_fp8, d_scale_amax);
}

int granite4_kernel_fp8_quant(const uint16_t* d_x, long long n, uint8_t* d_codes,
                              float* d_scale_amax) {
  const char* fn = "granite4_kernel_fp8_quant";
  if (d_x == nullptr || d_codes == nullptr || d_scale_amax == nullptr || n <= 0 || n % 8 != 0 ||
      !g4::aligned16(d_x) || !g4::aligned16(d_codes))
    return g4::fail(fn, "invalid arguments");
  cudaStream_t st = g4::current_stream();
  const long long n8 = n / 8;
  const int grid = static_cast<int>(std::min<long long>((n8 + 255) / 256, g4::sm_count() * 16LL));
  G4_CUDA_TRY(fn, cudaMemsetAsync(d_scale_amax, 0, 2 * sizeof(float), st));
  g4::amax_bf16_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint4*>(d_x), n8, d_scale_amax);
  G4_LAUNCH_CHECK(fn);
  g4::encode_bf16_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint4*>(d_x), n8,
                                               reinterpret_cast<uint2*>(d_codes), d_scale_amax);
  G4_LAUNCH_CHECK(fn);
  return 0;
}

}  // extern "C"
