// Device scalar math of the Granite glue kernels (sm_100a).
//
// Every rounding point is spelled with an explicit round-to-nearest intrinsic
// (__fmul_rn / __fadd_rn / ...): the compiler may not fuse a multiply into a
// following add, so results equal the reference's host fp32 formulation
// (engine/src/kernel_math.h, compiled without FMA) bit for bit wherever that
// formulation has no transcendental.
//
// These kernels move 3-6 bytes per element, which at HBM speed leaves an SM
// only 10-20 issue slots per element. The quantisers therefore have a short
// common path (a multiply by the reciprocal of the scale and a hardware
// conversion) and an exact path (IEEE division and the rounding rule spelled
// out) that is taken only by the few elements whose quotient lies so close to a
// rounding boundary that the short path could pick the other side. The results
// are those of the exact path everywhere.
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
// The reference's integer form (add 0x7fff + lsb, shift). Kept for scalar
// fallback kernels.
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float f) {
  uint32_t u = __float_as_uint(f);
  u += 0x7fffu + ((u >> 16) & 1u);
  return u >> 16;
}
// (lo, hi) -> packed pair, lo in the low half: one conversion instruction for
// two elements. It rounds to nearest even exactly as the integer form does for
// every finite input and for infinities (NaN payloads may differ).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
// Round a float to the nearest bf16 and return it as a float.
__device__ __forceinline__ float round_bf16(float f) {
  return __uint_as_float(pack_bf16x2(0.0f, f) & 0xffff0000u);
}

__device__ __forceinline__ void unpack8(uint4 u, float (&v)[8]) {
  v[0] = bf16_lo(u.x), v[1] = bf16_hi(u.x), v[2] = bf16_lo(u.y), v[3] = bf16_hi(u.y);
  v[4] = bf16_lo(u.z), v[5] = bf16_hi(u.z), v[6] = bf16_lo(u.w), v[7] = bf16_hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]);
  u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]);
  u.w = pack_bf16x2(v[6], v[7]);
  return u;
}

// ---- running max |x| over packed bf16 pairs -----------------------------------
// Clearing the two sign bits leaves magnitudes whose bit patterns order like
// unsigned 16-bit integers, so the running maximum is one AND and one packed
// integer max per two elements.
__device__ __forceinline__ uint32_t max_u16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t amax_acc(uint32_t acc, uint32_t bf16_pair) {
  return max_u16x2(acc, bf16_pair & 0x7fff7fffu);
}
__device__ __forceinline__ uint32_t amax_acc(uint32_t acc, uint4 v) {
  return amax_acc(amax_acc(amax_acc(amax_acc(acc, v.x), v.y), v.z), v.w);
}
__device__ __forceinline__ uint32_t amax_warp(uint32_t acc) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc = max_u16x2(acc, __shfl_xor_sync(0xffffffffu, acc, o));
  return acc;
}
// Larger half of the packed accumulator, as a float.
__device__ __forceinline__ float amax_value(uint32_t acc) {
  const uint32_t lo = acc & 0xffffu, hi = acc >> 16;
  return __uint_as_float((lo > hi ? lo : hi) << 16);
}

// ---- FP8 e4m3, per-tensor scale --------------------------------------------
// Reference rule (engine/src/checkpoint_main.cc:118-122, :702-723 over
// engine/src/fp8_convert.cc:47-122): scale = float(amax / 448) with the
// division in double; code = RNE_e4m3(double(v) / double(scale)) in exact
// arithmetic, |q| >= 464 clipping to +-448; scale == 0 -> encode v itself.
// v is always a bf16 value here, so the double quotient the reference forms
// rounds to e4m3 exactly as the true quotient v / scale does.
//
// The quantiser is exact and branch-free, five instructions per element plus
// half a conversion:
//  1. 1 / scale, nudged up by less than 2^-38 relative, is split into a 16-bit
//     head and a 24-bit tail. A bf16 value has 8 significant bits, so v * head is
//     exact in f32, and one FMA rounding TOWARD ZERO adds v * tail: q is the
//     true quotient v / scale truncated to 24 bits. (The nudge keeps the product
//     from falling a hair below an exactly representable quotient. It cannot
//     carry the product past an e4m3 midpoint: v has 8 significant bits and
//     scale 24, so a quotient that is not exactly a midpoint is at least 2^-29
//     relative away from it.)
//  2. rem = fma(-q, scale, v) is the exact remainder, zero iff q is the true
//     quotient.
//  3. If it is not, the last mantissa bit of q is set: q is now the true quotient
//     rounded TO ODD. A value rounded to odd at 24 bits rounds to nearest even at
//     any precision two or more bits shorter exactly as the unrounded value does,
//     so the hardware e4m3 conversion that follows returns the reference's code
//     for every input: true ties go to even, near-ties (about one bf16 mantissa
//     pattern in 128 is a would-be tie that the rounding of the scale itself
//     moved off the midpoint) go to the side the double quotient is on, and the
//     e4m3 subnormal range and the saturation need no special case.
struct Fp8Scale {
  float scale;   // 0 when the tensor is all zeros
  float div;     // divisor used for the remainder: scale, or 1 when scale == 0
  float inv_hi;  // head of 1 / div: low 8 mantissa bits clear
  float inv_lo;  // tail, rounded up
};
__device__ __forceinline__ Fp8Scale fp8_scale_from_amax(float amax) {
  Fp8Scale s;
  s.scale = static_cast<float>(static_cast<double>(amax) / 448.0);
  s.div = s.scale > 0.0f ? s.scale : 1.0f;
  const double inv = (1.0 / static_cast<double>(s.div)) * (1.0 + 0x1p-45);
  s.inv_hi = __uint_as_float(__float_as_uint(__double2float_rz(inv)) & 0xffffff00u);
  s.inv_lo = __double2float_ru(inv - static_cast<double>(s.inv_hi));
  return s;
}

// Two floats -> two e4m3 codes (lo in the low byte). cvt.rn.satfinite: round to
// nearest even, everything above 448 (incl. inf) saturates to 448, NaN -> 0x7F,
// the sign of zero is kept.
__device__ __forceinline__ uint32_t fp8x2_encode(float lo, float hi) {
  return static_cast<uint32_t>(
      __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}

// v / scale rounded to odd (see above); v is a bf16-valued float.
__device__ __forceinline__ float fp8_quotient_odd(float v, const Fp8Scale s) {
  const float q = __fmaf_rz(v, s.inv_lo, __fmul_rn(v, s.inv_hi));
  const float rem = __fmaf_rn(-q, s.div, v);
  uint32_t qb = __float_as_uint(q);
  if (rem != 0.0f) qb |= 1u;
  return __uint_as_float(qb);
}

// Eight packed bf16 values -> eight codes (element 0 in the low byte of .x).
__device__ __forceinline__ uint2 fp8x8_quant(uint4 p, const Fp8Scale s) {
  float v[8];
  unpack8(p, v);
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = fp8_quotient_odd(v[e], s);
  uint2 c;
  c.x = fp8x2_encode(v[0], v[1]) | (fp8x2_encode(v[2], v[3]) << 16);
  c.y = fp8x2_encode(v[4], v[5]) | (fp8x2_encode(v[6], v[7]) << 16);
  return c;
}

// ---- int8 KV rows (Q8_0) ----------------------------------------------------
// Reference: engine/src/device_math.cuh:105-134, engine/src/kernel_math.h:71-86.
// s = amax / 127 (IEEE division), code = clamp(round_half_away(x / s), +-127),
// s == 0 -> 0.
struct Kv8Scale {
  float s;
  float inv;  // ~1 / s (SFU reciprocal; only the short path uses it), or 0 when s == 0
};
__device__ __forceinline__ Kv8Scale kv8_scale(float amax) {
  Kv8Scale k;
  k.s = __fdiv_rn(amax, 127.0f);
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(k.s));
  k.inv = k.s != 0.0f ? r : 0.0f;
  return k;
}
static __device__ __noinline__ int kv8_quant_exact(float x, float s) {
  if (s == 0.0f) return 0;
  const float q = __fdiv_rn(x, s);
  float t = truncf(q);
  const float fr = q - t;  // exact
  if (fabsf(fr) >= 0.5f) t += copysignf(1.0f, q);
  t = fminf(fmaxf(t, -127.0f), 127.0f);
  return static_cast<int>(t);
}
// Short path: x * inv is within 4e-5 of the true quotient (|q| <= 127), so its
// nearest integer is the right code unless the fraction is that close to one
// half; such a group of eight takes the exact path. |x| <= amax keeps
// |q| <= 127 + 1e-4, which rounds into range without a clamp. Adding the magic
// constant 1.5 * 2^23 makes the f32 add itself round to the nearest integer and
// leaves it, as a two's complement byte, in the low 8 bits of the sum.
// Eight values -> eight codes in two words; one branch for the whole group.
__device__ __forceinline__ uint2 kv8_quant8(const float (&x)[8], const Kv8Scale k) {
  float t[8];
  bool doubt = false;
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float q = __fmul_rn(x[e], k.inv);
    t[e] = __fadd_rn(q, 12582912.0f);
    const float d = __fsub_rn(q, __fsub_rn(t[e], 12582912.0f));
    // written so that a NaN (an overflowed reciprocal of a subnormal s) also raises the doubt
    doubt = doubt || !(fabsf(d) <= 0.4999f);
  }
  uint2 out;
  if (!doubt) {
    const uint32_t b0 = __float_as_uint(t[0]), b1 = __float_as_uint(t[1]), b2 = __float_as_uint(t[2]),
                   b3 = __float_as_uint(t[3]), b4 = __float_as_uint(t[4]), b5 = __float_as_uint(t[5]),
                   b6 = __float_as_uint(t[6]), b7 = __float_as_uint(t[7]);
    out.x = __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
    out.y = __byte_perm(__byte_perm(b4, b5, 0x0040), __byte_perm(b6, b7, 0x0040), 0x5410);
  } else {
    // rare (one group in several hundred): redo the test per element, exact path where it fails
    uint32_t c[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float q = __fmul_rn(x[e], k.inv);
      const float d = __fsub_rn(q, __fsub_rn(t[e], 12582912.0f));
      c[e] = __float_as_uint(t[e]) & 0xffu;
      if (!(fabsf(d) <= 0.4999f)) c[e] = static_cast<uint32_t>(kv8_quant_exact(x[e], k.s)) & 0xffu;
    }
    out.x = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
    out.y = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
  }
  return out;
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
// silu(g) = g / (1 + expf(-g)), rounded to bf16 by the caller.
// exp and the reciprocal use the SFU approximations (ex2.approx, rcp.approx):
// the f32 result is within a few f32 ulp of the host's, which the bf16 rounding
// that follows hides except for roughly one element in several thousand, where
// the bf16 result is the neighbouring value (the stated tolerance is 1 bf16
// ulp; the reference's own device kernels are tested to the same bound against
// this host formula).
// For g below about -87.3 the sum d = 1 + e^-g passes 2^126, where the flushed
// reciprocal would be zero, while the host still divides by a finite number until
// expf(-g) overflows at -g = 88.7228... (there its quotient is a normal float of
// magnitude ~1e-36; three bf16 gates fall in that window: -87.5, -88, -88.5).
// The reciprocal is therefore taken of d / 4 - exact scaling, and d / 4 <= 2^126 for
// every finite d - and the factor 1/4 applied to the product afterwards: the same
// mantissas as g * rcp(d) * u wherever that is in range (the unit's result depends
// on the exponent only through its sign flip), the host's quotient in the window,
// and g * 0 = -0 once e^-g overflows to infinity, as on the host. No test, no branch:
// two multiplications by a power of two per element. (g * r is four times the
// result and overflows for |g| above 8.5e37, which no gate of a network reaches.)
__device__ __forceinline__ float swiglu(float g, float u) {
  float e, r;
  const float t = __fmul_rn(g, -1.4426950408889634f);
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t));
  const float d = __fmul_rn(__fadd_rn(1.0f, e), 0.25f);
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
  return __fmul_rn(__fmul_rn(__fmul_rn(g, r), 0.25f), u);
}

// ---- memory helpers -----------------------------------------------------------
// Read-once / write-once data goes through the streaming cache policy so it
// does not push reusable lines (norm weights, RoPE tables, data a second sweep
// re-reads) out of L2.
__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) { __stcs(p, v); }
__device__ __forceinline__ void st_stream(uint2* p, uint2 v) { __stcs(p, v); }

// L2 eviction-priority hints on single loads and stores (an instruction-level policy operand;
// nothing about the device or the context is configured). A tensor that one sweep writes and the
// next sweep re-reads is stored with evict_last so that the read-once inputs streaming past it do
// not push it out, and re-read with evict_first so that its lines are the first to go afterwards.
// `fraction` of the lines touched get the priority, the rest the default (evict_first for the
// store-side policy of a tensor larger than L2: see the callers).
__device__ __forceinline__ uint64_t l2_policy_evict_last(float fraction) {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.L2::evict_first.b64 %0, %1;" : "=l"(pol) : "f"(fraction));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void st_l2_hint(uint4* p, uint4 v, uint64_t pol) {
  asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;"
               :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(pol) : "memory");
}
__device__ __forceinline__ uint4 ld_l2_hint(const uint4* p, uint64_t pol) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.b32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(pol));
  return v;
}

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

// First statements of every kernel that is launched with programmatic stream serialisation
// (g4_host.h launch_pdl), executed by every thread of every CTA before anything else - above all
// before any early return, or a CTA that left without waiting would let the grid count as
// complete, and its successor start, while the predecessor still runs.
// griddepcontrol.wait blocks until the previous kernel has completed and its writes are visible;
// it is a no-op in a kernel launched without the attribute. Only a decode-size grid (a few CTAs)
// also signals launch_dependents early, so that the next small kernel is already resident when
// this one ends; a large grid leaves the signal to its CTAs' exits. Measured on B200: with an
// early signal in every kernel, the staged CTAs of the next kernel (thousands of them behind a
// persistent kernel, which has all its CTAs resident from the start) sat on the SMs waiting and
// cost the running kernel 12 % of the whole step.
__device__ __forceinline__ void pdl_begin() {
  if (gridDim.x * gridDim.y <= 64u) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace g4
