// SwiGLU on the gate/up GEMM output with bf16 and per-tensor FP8 e4m3 outputs.
//
// Formulation (reference: engine/src/kernel_math.h:239, :571-584 for the fp32
// golden form; engine/src/prefill_gemm.cu:1194-1203 for the prefill kernel's
// f32 [rows][2 I] input; per-tensor FP8 rule engine/src/checkpoint_main.cc:
// 118-122, :702-723):
//   a = bf16(silu(g) * u),  silu(g) = g / (1 + expf(-g))
//   amax = max |a| over the tensor, scale = float(amax / 448), code = e4m3(a / scale)
//
// Data layout: gate and up are [rows][I] views with a common row pitch ld
// (ld = I for separate tensors, 2 I for one fused [gate | up] GEMM output);
// I % 8 == 0 and 16-byte aligned rows. The work is cut into items of 8
// elements; a thread takes kUnroll items strided by the CTA width, so a warp
// reads 512 contiguous bytes per load instruction and has 2 * kUnroll 128-bit
// loads in flight per thread.
//
// FP8 needs two sweeps because the scale depends on every element: the amax
// sweep computes a and max |a| (and writes a as bf16 when asked); the encode
// sweep recomputes a from gate/up (or reads the bf16 copy when one was written)
// and writes the codes, walking the items backwards so that it starts on the
// part of the input the first sweep left in L2.
//
// Algorithmic bytes per row at I = 12800, bf16 in, FP8 out: 2 * 25 600 read +
// 12 800 written = 64 000; the encode sweep adds a second 51 200-byte read.
#include "g4_host.h"
#include "g4_math.cuh"

#include "../../include/granite4_b200.h"
#include "../../include/granite4_b200.hpp"

#include <algorithm>

namespace g4 {
namespace {

struct SwigluParams {
  const void* gate;
  const void* up;
  uint16_t* act_bf16;  // [rows][I] or NULL
  uint8_t* act_fp8;    // [rows][I] or NULL
  float* scale_amax;   // [0] scale, [1] amax
  long long ld;        // input row pitch, elements
  long long items;     // rows * I / 8
  int ipr;             // items per row = I / 8
  int contiguous;      // ld == I: item index is the element offset / 8
};

enum { kAmax = 0, kEncode = 1, kPlain = 2 };
constexpr int kThreads = 256;
constexpr int kUnroll = 4;

template <bool F32>
__device__ __forceinline__ void load8(const void* base, long long elem_off, float (&v)[8]) {
  if (F32) {
    const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + elem_off);
    const float4 a = ld_stream(p), b = ld_stream(p + 1);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  } else {
    const uint4 u =
        ld_stream(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + elem_off));
    v[0] = bf16_lo(u.x), v[1] = bf16_hi(u.x), v[2] = bf16_lo(u.y), v[3] = bf16_hi(u.y);
    v[4] = bf16_lo(u.z), v[5] = bf16_hi(u.z), v[6] = bf16_lo(u.w), v[7] = bf16_hi(u.w);
  }
}

// MODE kPlain: bf16 out only. kAmax: amax (+ optional bf16 out). kEncode: codes.
template <bool F32, int MODE, bool FROM_BF16>
__global__ void __launch_bounds__(kThreads) swiglu_kernel(const SwigluParams p) {
  const long long tile0 = static_cast<long long>(blockIdx.x) * (kThreads * kUnroll);
  float scale = 0.0f;
  if (MODE == kEncode) {
    scale = fp8_scale_from_amax(__ldcg(p.scale_amax + 1));
    if (blockIdx.x == 0 && threadIdx.x == 0) p.scale_amax[0] = scale;
  }
  long long item[kUnroll];
  bool ok[kUnroll];
  uint4 a_bits[kUnroll];
  float g[kUnroll][8], u[kUnroll][8];
#pragma unroll
  for (int k = 0; k < kUnroll; ++k) {
    long long it = tile0 + k * kThreads + threadIdx.x;
    ok[k] = it < p.items;
    if (MODE == kEncode) it = p.items - 1 - it;  // backwards
    item[k] = it;
    if (ok[k]) {
      if (FROM_BF16) {
        a_bits[k] = ld_stream(reinterpret_cast<const uint4*>(p.act_bf16) + it);
      } else {
        long long off;
        if (p.contiguous) {
          off = it * 8;
        } else {
          const long long row = it / p.ipr;
          off = row * p.ld + (it - row * p.ipr) * 8;
        }
        load8<F32>(p.gate, off, g[k]);
        load8<F32>(p.up, off, u[k]);
      }
    }
  }
  float amax = 0.0f;
#pragma unroll
  for (int k = 0; k < kUnroll; ++k) {
    if (!ok[k]) continue;
    if (!FROM_BF16) {
      float a[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] = swiglu(g[k][e], u[k][e]);
      a_bits[k].x = pack_bf16x2(a[0], a[1]);
      a_bits[k].y = pack_bf16x2(a[2], a[3]);
      a_bits[k].z = pack_bf16x2(a[4], a[5]);
      a_bits[k].w = pack_bf16x2(a[6], a[7]);
    }
    const uint4 ab = a_bits[k];
    if (MODE != kEncode) {
      if (p.act_bf16 != nullptr) {
        uint4* dst = reinterpret_cast<uint4*>(p.act_bf16) + item[k];
        if (MODE == kAmax) *dst = ab; else st_stream(dst, ab);
      }
      if (MODE == kAmax) {
        const uint32_t m0 = ab.x & 0x7fff7fffu, m1 = ab.y & 0x7fff7fffu, m2 = ab.z & 0x7fff7fffu,
                       m3 = ab.w & 0x7fff7fffu;
        amax = fmaxf(amax, fmaxf(fmaxf(bf16_lo(m0), bf16_hi(m0)), fmaxf(bf16_lo(m1), bf16_hi(m1))));
        amax = fmaxf(amax, fmaxf(fmaxf(bf16_lo(m2), bf16_hi(m2)), fmaxf(bf16_lo(m3), bf16_hi(m3))));
      }
    } else {
      uint2 c;
      c.x = fp8x4_quant(bf16_lo(ab.x), bf16_hi(ab.x), bf16_lo(ab.y), bf16_hi(ab.y), scale);
      c.y = fp8x4_quant(bf16_lo(ab.z), bf16_hi(ab.z), bf16_lo(ab.w), bf16_hi(ab.w), scale);
      st_stream(reinterpret_cast<uint2*>(p.act_fp8) + item[k], c);
    }
  }
  if (MODE == kAmax) {
    amax = warp_max(amax);
    __shared__ float s[kThreads / 32];
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = 0.0f;
#pragma unroll
      for (int i = 0; i < kThreads / 32; ++i) m = fmaxf(m, s[i]);
      atomic_amax(p.scale_amax + 1, m);
    }
  }
}

template <bool F32>
int launch_swiglu(const char* fn, const SwigluParams& p) {
  cudaStream_t st = current_stream();
  const long long tiles = (p.items + kThreads * kUnroll - 1) / (kThreads * kUnroll);
  if (tiles > INT_MAX) return fail(fn, "tensor too large");
  const unsigned grid = static_cast<unsigned>(tiles);
  if (p.act_fp8 == nullptr) {
    swiglu_kernel<F32, kPlain, false><<<grid, kThreads, 0, st>>>(p);
    G4_LAUNCH_CHECK(fn);
    return 0;
  }
  G4_CUDA_TRY(fn, cudaMemsetAsync(p.scale_amax, 0, 2 * sizeof(float), st));
  swiglu_kernel<F32, kAmax, false><<<grid, kThreads, 0, st>>>(p);
  G4_LAUNCH_CHECK(fn);
  if (p.act_bf16 != nullptr)
    swiglu_kernel<F32, kEncode, true><<<grid, kThreads, 0, st>>>(p);
  else
    swiglu_kernel<F32, kEncode, false><<<grid, kThreads, 0, st>>>(p);
  G4_LAUNCH_CHECK(fn);
  return 0;
}

}  // namespace
}  // namespace g4

extern "C" {

int granite4_kernel_swiglu_fp8(const void* d_gate, const void* d_up, int in_is_f32, long long ld,
                               int rows, int I, uint16_t* d_act_bf16, uint8_t* d_act_fp8,
                               float* d_scale_amax) {
  const char* fn = "granite4_kernel_swiglu_fp8";
  if (d_gate == nullptr || d_up == nullptr || rows <= 0 || I <= 0 || ld < I ||
      (d_act_bf16 == nullptr && d_act_fp8 == nullptr))
    return g4::fail(fn, "invalid arguments");
  if (d_act_fp8 != nullptr && d_scale_amax == nullptr)
    return g4::fail(fn, "FP8 output needs d_scale_amax");
  const int esz = in_is_f32 ? 4 : 2;
  if (I % 8 != 0 || (ld * esz) % 16 != 0 || !g4::aligned16(d_gate) || !g4::aligned16(d_up) ||
      !g4::aligned16(d_act_bf16) || !g4::aligned16(d_act_fp8))
    return g4::fail(fn, "I must be a multiple of 8 and rows 16-byte aligned");
  g4::SwigluParams p{};
  p.gate = d_gate, p.up = d_up, p.act_bf16 = d_act_bf16, p.act_fp8 = d_act_fp8;
  p.scale_amax = d_scale_amax, p.ld = ld, p.ipr = I / 8;
  p.items = static_cast<long long>(rows) * p.ipr, p.contiguous = (ld == I);
  return in_is_f32 ? g4::launch_swiglu<true>(fn, p) : g4::launch_swiglu<false>(fn, p);
}

int granite4_prefill_silu_mul(const float* gu, int I, int rows, uint16_t* act) {
  const char* fn = "prefill_silu_mul";
  if (rows <= 0 || I <= 0) return -1;  // engine/src/prefill_gemm.cu:1469
  if (gu == nullptr || act == nullptr) return g4::fail(fn, "invalid arguments");
  return granite4_kernel_swiglu_fp8(gu, gu + I, 1, 2LL * I, rows, I, act, nullptr, nullptr);
}

}  // extern "C"

namespace granite4 {
int prefill_silu_mul(const float* gu, int I, int rows, std::uint16_t* act) {
  return granite4_prefill_silu_mul(gu, I, rows, act);
}
}  // namespace granite4
