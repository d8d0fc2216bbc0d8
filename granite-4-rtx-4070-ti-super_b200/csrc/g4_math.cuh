// Device scalar math of the Granite glue kernels (sm_100a).
//
// Every rounding point is spelled with an explicit round-to-nearest intrinsic
// (__fmul_rn / __fadd_rn / __fdiv_rn / __fsqrt_rn): the compiler may not fuse
// a multiply into a following add, so results equal the reference's host fp32
// formulation (engine/src/kernel_math.h, compiled without FMA) bit for bit
// wherever that formulation has no transcendental. All kernels here are
// HBM-bound, so the extra instructions are free.
#pragma once

#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace g4 {

// ---- bf16 <-> f32 (round to nearest even) ---------------------------------
// Reference: engine/src/device_math.cuh:31-39, engine/src/kernel_math.h:39-55.
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ float bf16_to_f32(uint16_t b) {
  return __uint_as_float(static_cast<uint32_t>(b) << 16);
}
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  uint32_t u = __float_as_uint(f);
  u += 0x7fffu + ((u >> 16) & 1u);
  return u >> 16;
}
// (lo, hi) -> packed pair, lo in the low half.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  return f32_to_bf16_bits(lo) | (f32_to_bf16_bits(hi) << 16);
}
// Round a float to the nearest bf16 and return it as a float.
__device__ __forceinline__ float round_bf16(float f) {
  return __uint_as_float(f32_to_bf16_bits(f) << 16);
}

// ---- FP8 e4m3, per-tensor scale --------------------------------------------
// Reference rule (engine/src/checkpoint_main.cc:118-122, :702-723 over
// engine/src/fp8_convert.cc:47-122): scale = float(amax / 448) with the
// division in double; code = RNE_e4m3(double(v) / double(scale)) in exact
// arithmetic, |q| >= 464 clipping to +-448; scale == 0 -> encode v itself.
__device__ __forceinline__ float fp8_scale_from_amax(float amax) {
  return static_cast<float>(static_cast<double>(amax) / 448.0);
}

// The quotient handed to the hardware e4m3 conversion. The f32 quotient of two
// floats is the correctly rounded true quotient; rounding it a second time to
// e4m3 differs from rounding the true quotient only when the f32 quotient sits
// exactly on an e4m3 midpoint that the true quotient is not on. The exact
// remainder sign (one FMA) says which side the true quotient is on, and the
// quotient is moved one f32 ulp that way, off the midpoint. True ties (zero
// remainder) are left for the conversion's round-half-even, as the reference
// does. v is a bf16 value, so the double quotient the reference forms rounds to
// e4m3 exactly as the true quotient does.
__device__ __forceinline__ float fp8_scaled(float v, float scale) {
  float q = __fdiv_rn(v, scale);
  const uint32_t qb = __float_as_uint(q);
  const uint32_t mag = qb & 0x7fffffffu;
  bool tie;
  if (mag >= 0x3c800000u) {  // |q| >= 2^-6: 3 mantissa bits survive
    tie = (mag & 0x000fffffu) == 0x00080000u;
  } else {  // fixed step 2^-9
    const float y = __uint_as_float(mag) * 512.0f;
    tie = (y - floorf(y)) == 0.5f;
  }
  if (tie) {
    const float rem = __fmaf_rn(-q, scale, v);  // sign of (true quotient - q), scale > 0
    if (rem != 0.0f) {
      const bool up = rem > 0.0f;
      const bool neg = (qb >> 31) != 0u;
      q = __uint_as_float(up != neg ? qb + 1u : qb - 1u);
    }
  }
  return q;
}

// Two scaled values -> two e4m3 codes (lo in the low byte). cvt.rn.satfinite:
// round to nearest even, everything above 448 (incl. inf) saturates to 448,
// NaN -> 0x7F, the sign of zero is kept.
__device__ __forceinline__ uint32_t fp8x2_encode(float lo, float hi) {
  return static_cast<uint32_t>(
      __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ uint32_t fp8x2_quant(float lo, float hi, float scale) {
  if (scale > 0.0f) {
    lo = fp8_scaled(lo, scale);
    hi = fp8_scaled(hi, scale);
  }
  return fp8x2_encode(lo, hi);
}
// Four values -> four codes in one 32-bit word (element 0 in the low byte).
__device__ __forceinline__ uint32_t fp8x4_quant(float a, float b, float c, float d, float scale) {
  return fp8x2_quant(a, b, scale) | (fp8x2_quant(c, d, scale) << 16);
}

// ---- int8 KV rows (Q8_0) ----------------------------------------------------
// Reference: engine/src/device_math.cuh:105-134, engine/src/kernel_math.h:71-86.
// s = amax / 127 (IEEE division), code = clamp(round_half_away(x / s), +-127),
// s == 0 -> 0.
__device__ __forceinline__ float kv8_scale(float amax) { return __fdiv_rn(amax, 127.0f); }
__device__ __forceinline__ int kv8_quant(float x, float s) {
  if (s == 0.0f) return 0;
  const float q = __fdiv_rn(x, s);
  float t = truncf(q);
  const float fr = q - t;  // exact
  if (fabsf(fr) >= 0.5f) t += copysignf(1.0f, q);
  t = fminf(fmaxf(t, -127.0f), 127.0f);
  return static_cast<int>(t);
}
__device__ __forceinline__ uint32_t pack_i8x4(int a, int b, int c, int d) {
  return (static_cast<uint32_t>(a) & 0xffu) | ((static_cast<uint32_t>(b) & 0xffu) << 8) |
         ((static_cast<uint32_t>(c) & 0xffu) << 16) | ((static_cast<uint32_t>(d) & 0xffu) << 24);
}

// ---- RoPE, Llama half split -------------------------------------------------
// Reference: engine/src/kernel_math.h:208-219. (a, b) = (x[i], x[i + d/2]):
// lo = a c - b s, hi = b c + a s, products rounded before the add.
__device__ __forceinline__ void rope_pair(float a, float b, float c, float s, float& lo, float& hi) {
  lo = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
  hi = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, s));
}

// ---- SwiGLU -----------------------------------------------------------------
// Reference: engine/src/kernel_math.h:239, :571-584: silu(g) * u with
// silu(g) = g / (1 + expf(-g)); expf is the accurate library routine.
__device__ __forceinline__ float swiglu(float g, float u) {
  const float sg = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
  return __fmul_rn(sg, u);
}

// ---- memory helpers -----------------------------------------------------------
// Read-once / write-once data goes through the streaming cache policy so it
// does not push reusable lines (norm weights, RoPE tables, the hidden state a
// second phase re-reads) out of L2.
__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) { __stcs(p, v); }
__device__ __forceinline__ void st_stream(uint2* p, uint2 v) { __stcs(p, v); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// amax is >= 0 (or NaN): its bit pattern orders like an unsigned integer, so an
// integer max is exact and independent of arrival order.
__device__ __forceinline__ void atomic_amax(float* slot, float v) {
  atomicMax(reinterpret_cast<unsigned int*>(slot), __float_as_uint(v));
}

}  // namespace g4
