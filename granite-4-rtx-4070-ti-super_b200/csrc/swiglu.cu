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
// FP8 needs two sweeps because the scale depends on every element. The first
// computes a and max |a|. If the caller passes a bf16 buffer for a (as an
// output it wants, or purely as workspace) the first sweep stores a there and
// the second sweep is a light bf16 -> e4m3 pass over it; without one the second
// sweep recomputes a from gate and up. Both move the same number of bytes
// (115 200 per row at I = 12800), but the first evaluates the exponential once,
// and at HBM speed an SM has only ~15 issue slots per element, which the
// exponential, the reciprocal and the quantiser together overrun. The second
// sweep walks the items backwards so that it starts on what the first left in L2.
//
// Algorithmic bytes per row at I = 12800, bf16 in, FP8 out: 2 * 25 600 read +
// 12 800 written = 64 000.
#include "g4_cluster.cuh"
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
  unsigned ipr;        // items per row = I / 8
  int contiguous;      // ld == I: item index is the element offset / 8
};

enum { kAmax = 0, kEncode = 1, kPlain = 2 };
constexpr int kThreads = 256;
constexpr int kUnroll = 4;

__device__ __forceinline__ long long item_offset(const SwigluParams& p, long long it) {
  if (p.contiguous) return it * 8;
  // items < 2^32 is checked by the launcher, so a 32-bit division does
  const unsigned row = static_cast<unsigned>(it) / p.ipr;
  return static_cast<long long>(row) * p.ld + static_cast<long long>(static_cast<unsigned>(it) - row * p.ipr) * 8;
}

// gate / up item -> 8 activations, packed bf16
template <bool F32>
__device__ __forceinline__ uint4 swiglu8(const void* gate, const void* up, long long off) {
  float g[8], u[8], a[8];
  if (F32) {
    const float4* gp = reinterpret_cast<const float4*>(static_cast<const float*>(gate) + off);
    const float4* up4 = reinterpret_cast<const float4*>(static_cast<const float*>(up) + off);
    const float4 g0 = ld_stream(gp), g1 = ld_stream(gp + 1), u0 = ld_stream(up4), u1 = ld_stream(up4 + 1);
    g[0] = g0.x, g[1] = g0.y, g[2] = g0.z, g[3] = g0.w, g[4] = g1.x, g[5] = g1.y, g[6] = g1.z, g[7] = g1.w;
    u[0] = u0.x, u[1] = u0.y, u[2] = u0.z, u[3] = u0.w, u[4] = u1.x, u[5] = u1.y, u[6] = u1.z, u[7] = u1.w;
  } else {
    unpack8(ld_stream(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(gate) + off)), g);
    unpack8(ld_stream(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(up) + off)), u);
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) a[e] = swiglu(g[e], u[e]);
  return pack8(a);
}

// MODE kPlain: bf16 out only. kAmax: amax (+ bf16 out when a buffer is given).
// kEncode: codes, from the bf16 buffer (FROM_BF16) or recomputed.
template <bool F32, int MODE, bool FROM_BF16>
__global__ void __launch_bounds__(kThreads) swiglu_kernel(const SwigluParams p) {
  pdl_begin();
  const long long tile0 = static_cast<long long>(blockIdx.x) * (kThreads * kUnroll) + threadIdx.x;
  Fp8Scale fs{};
  if (MODE == kEncode) {
    fs = fp8_scale_from_amax(__ldcg(p.scale_amax + 1));
    if (blockIdx.x == 0 && threadIdx.x == 0) p.scale_amax[0] = fs.scale;
  }
  long long item[kUnroll];
  uint4 a[kUnroll];
  uint4 graw[kUnroll], uraw[kUnroll];  // bf16 inputs: every load is issued before any math
#pragma unroll
  for (int k = 0; k < kUnroll; ++k) {
    long long it = tile0 + k * kThreads;
    if (it >= p.items) {
      item[k] = -1;
      a[k] = graw[k] = uraw[k] = make_uint4(0, 0, 0, 0);
      continue;
    }
    if (MODE == kEncode) it = p.items - 1 - it;  // backwards
    item[k] = it;
    if (FROM_BF16) {
      a[k] = ld_stream(reinterpret_cast<const uint4*>(p.act_bf16) + it);
    } else if (F32) {
      a[k] = swiglu8<true>(p.gate, p.up, item_offset(p, it));
    } else {
      const long long off = item_offset(p, it);
      graw[k] = ld_stream(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.gate) + off));
      uraw[k] = ld_stream(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.up) + off));
    }
  }
  if (!FROM_BF16 && !F32) {
#pragma unroll
    for (int k = 0; k < kUnroll; ++k) {
      float g[8], u[8], v[8];
      unpack8(graw[k], g);
      unpack8(uraw[k], u);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = swiglu(g[e], u[e]);
      a[k] = pack8(v);
    }
  }
  uint32_t amax = 0u;
#pragma unroll
  for (int k = 0; k < kUnroll; ++k) {
    if (item[k] < 0) continue;
    if (MODE == kEncode) {
      st_stream(reinterpret_cast<uint2*>(p.act_fp8) + item[k], fp8x8_quant(a[k], fs));
    } else {
      if (p.act_bf16 != nullptr) {
        uint4* dst = reinterpret_cast<uint4*>(p.act_bf16) + item[k];
        if (MODE == kAmax) *dst = a[k]; else st_stream(dst, a[k]);  // kAmax: re-read by the encode sweep
      }
      if (MODE == kAmax) amax = amax_acc(amax, a[k]);
    }
  }
  if (MODE == kAmax) {
    amax = amax_warp(amax);
    __shared__ uint32_t s[kThreads / 32];
    if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t m = 0u;
#pragma unroll
      for (int i = 0; i < kThreads / 32; ++i) m = max_u16x2(m, s[i]);
      atomic_amax(p.scale_amax + 1, amax_value(m));
    }
  }
}

// Small tensors (a decode or verify step: up to 16 rows of 12800): the whole grid is one cluster,
// the activations stay in registers between the amax exchange and the encode step, so one launch
// replaces the memset and the two sweeps (g4_cluster.cuh). A CTA owns kClusterThreads * kUnroll
// consecutive items.
constexpr int kClusterThreads = 512;
constexpr long long kClusterItemsPerCta = static_cast<long long>(kClusterThreads) * kUnroll;

template <bool F32>
__global__ void __launch_bounds__(kClusterThreads) swiglu_cluster_kernel(const SwigluParams p) {
  pdl_begin();
  cluster_announce();
  const long long tile0 = static_cast<long long>(blockIdx.x) * kClusterItemsPerCta + threadIdx.x;
  uint4 a[kUnroll];
  uint32_t amax = 0u;
#pragma unroll
  for (int k = 0; k < kUnroll; ++k) {
    const long long it = tile0 + k * kClusterThreads;
    a[k] = make_uint4(0, 0, 0, 0);
    if (it < p.items) {
      a[k] = swiglu8<F32>(p.gate, p.up, item_offset(p, it));
      if (p.act_bf16 != nullptr) st_stream(reinterpret_cast<uint4*>(p.act_bf16) + it, a[k]);
    }
    amax = amax_acc(amax, a[k]);
  }
  __shared__ uint32_t s_warp[kClusterThreads / 32];
  __shared__ uint32_t s_slots[kMaxClusterCtas];
  const float tensor_amax = __uint_as_float(cluster_amax_bits(amax, s_warp, s_slots));
  const Fp8Scale fs = fp8_scale_from_amax(tensor_amax);
#pragma unroll
  for (int k = 0; k < kUnroll; ++k) {
    const long long it = tile0 + k * kClusterThreads;
    if (it < p.items) st_stream(reinterpret_cast<uint2*>(p.act_fp8) + it, fp8x8_quant(a[k], fs));
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) p.scale_amax[0] = fs.scale, p.scale_amax[1] = tensor_amax;
}

// The reference's prefill entry point takes any I: scalar form for I % 8 != 0.
__global__ void __launch_bounds__(256)
    silu_mul_scalar_kernel(const float* gu, int I, long long n, uint16_t* act) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const long long r = idx / I, i = idx % I;
  act[idx] = static_cast<uint16_t>(f32_to_bf16_bits(swiglu(gu[r * 2 * I + i], gu[r * 2 * I + I + i])));
}

template <bool F32>
int launch_swiglu(const char* fn, const SwigluParams& p) {
  cudaStream_t st = current_stream();
  const long long tiles = (p.items + kThreads * kUnroll - 1) / (kThreads * kUnroll);
  if (tiles > INT_MAX || p.items > 0xffffffffLL) return fail(fn, "tensor too large");
  const unsigned grid = static_cast<unsigned>(tiles);
  if (p.act_fp8 == nullptr) {
    G4_LAUNCH_PDL(fn, swiglu_kernel<F32, kPlain, false>, dim3(grid), dim3(kThreads), 0, st, p);
    return 0;
  }
  if (p.items <= kMaxClusterCtas * kClusterItemsPerCta && cluster_enabled()) {
    const int ctas = cluster_ctas_for((p.items + kClusterItemsPerCta - 1) / kClusterItemsPerCta);
    const cudaError_t e = cluster_launch(swiglu_cluster_kernel<F32>, ctas, kClusterThreads, p, st);
    if (e == cudaSuccess) return 0;
    if (e != cudaErrorInvalidConfiguration) {
      std::fprintf(stderr, "granite4: %s: cluster launch failed: %s\n", fn, cudaGetErrorString(e));
      return -1;
    }
    // the device cannot place such a cluster: the multi-launch form below takes over
  }
  if (!amax_prezeroed()) G4_CUDA_TRY(fn, cudaMemsetAsync(p.scale_amax, 0, 2 * sizeof(float), st));
  G4_LAUNCH_PDL(fn, swiglu_kernel<F32, kAmax, false>, dim3(grid), dim3(kThreads), 0, st, p);
  if (p.act_bf16 != nullptr)
    G4_LAUNCH_PDL(fn, swiglu_kernel<F32, kEncode, true>, dim3(grid), dim3(kThreads), 0, st, p);
  else
    G4_LAUNCH_PDL(fn, swiglu_kernel<F32, kEncode, false>, dim3(grid), dim3(kThreads), 0, st, p);
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
  p.scale_amax = d_scale_amax, p.ld = ld, p.ipr = static_cast<unsigned>(I / 8);
  p.items = static_cast<long long>(rows) * p.ipr, p.contiguous = (ld == I);
  return in_is_f32 ? g4::launch_swiglu<true>(fn, p) : g4::launch_swiglu<false>(fn, p);
}

int granite4_kernel_fp8_encode_with_amax(const uint16_t* d_x, long long n, uint8_t* d_codes,
                                         float* d_scale_amax) {
  const char* fn = "granite4_kernel_fp8_encode_with_amax";
  if (d_x == nullptr || d_codes == nullptr || d_scale_amax == nullptr || n <= 0 || n % 8 != 0 ||
      n / 8 >= (1ll << 32) || !g4::aligned16(d_x) || !g4::aligned16(d_codes))
    return g4::fail(fn, "needs n % 8 == 0 and 16-byte aligned buffers");
  g4::SwigluParams p{};
  p.act_bf16 = const_cast<uint16_t*>(d_x), p.act_fp8 = d_codes, p.scale_amax = d_scale_amax;
  p.items = n / 8, p.ipr = 1, p.contiguous = 1, p.ld = 8;
  const long long tiles = (p.items + g4::kThreads * g4::kUnroll - 1) / (g4::kThreads * g4::kUnroll);
  G4_LAUNCH_PDL(fn, (g4::swiglu_kernel<false, g4::kEncode, true>), dim3(static_cast<unsigned>(tiles)),
                dim3(g4::kThreads), 0, g4::current_stream(), p);
  return 0;
}

int granite4_prefill_silu_mul(const float* gu, int I, int rows, uint16_t* act) {
  const char* fn = "prefill_silu_mul";
  if (rows <= 0 || I <= 0) return -1;  // engine/src/prefill_gemm.cu:1469
  if (gu == nullptr || act == nullptr) return g4::fail(fn, "invalid arguments");
  if (I % 8 != 0 || !g4::aligned16(gu) || !g4::aligned16(act)) {
    const long long n = static_cast<long long>(rows) * I;
    g4::silu_mul_scalar_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0,
                                 g4::current_stream()>>>(gu, I, n, act);
    G4_LAUNCH_CHECK(fn);
    return 0;
  }
  return granite4_kernel_swiglu_fp8(gu, gu + I, 1, 2LL * I, rows, I, act, nullptr, nullptr);
}

}  // extern "C"

namespace granite4 {
int prefill_silu_mul(const float* gu, int I, int rows, std::uint16_t* act) {
  return granite4_prefill_silu_mul(gu, I, rows, act);
}
}  // namespace granite4
