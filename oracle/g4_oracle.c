/* CPU oracle for the Granite 4.2 8B per-layer glue kernels: implementation.
 *
 * TEST INFRASTRUCTURE ONLY (see g4_oracle.h). Plain C, scalar, one thread;
 * callers that want several cores split the rows and call concurrently (every
 * function here is re-entrant and rows are independent).
 *
 * Build with -ffp-contract=off: the reference's host code is compiled for
 * baseline x86-64 (no FMA), so "a * c - b * s" is two roundings there, and it
 * must be two roundings here.
 */
#include "g4_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------ */
/* scalar codecs                                                            */
/* ------------------------------------------------------------------------ */

float g4o_bf16_to_f32(uint16_t bits) {
  uint32_t u = (uint32_t)bits << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

uint16_t g4o_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  /* the reference adds the rounding bias to the raw bits (NaN / overflow are
   * not special-cased there either) */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

uint8_t g4o_fp8_e4m3_encode(double v) {
  if (v != v) return 0x7F;
  const uint8_t sign = signbit(v) ? 0x80u : 0x00u;
  const double a = fabs(v);
  if (a >= 464.0) return (uint8_t)(sign | 0x7Eu); /* also +-inf */
  if (a == 0.0) return sign;
  /* The grid step is 2^-9 below 2^-6 (subnormals and the first binade share
   * it) and 2^(floor(log2 a) - 3) above. a / step is an exact scaling, rint
   * is round-half-even in the default rounding mode. */
  int e;
  (void)frexp(a, &e); /* a = m * 2^e, m in [0.5, 1) */
  int fl = e - 1;
  if (fl < -6) fl = -6;
  const double k = rint(ldexp(a, 3 - fl)); /* 0..16 */
  int ki = (int)k;
  if (ki == 0) return sign;
  if (fl == -6 && ki < 8) return (uint8_t)(sign | (uint8_t)ki); /* subnormal m * 2^-9 */
  if (ki == 16) {
    ki = 8;
    fl += 1;
  }
  int code = ((fl + 7) << 3) | (ki - 8);
  if (code > 0x7E) code = 0x7E; /* never emit the NaN slot */
  return (uint8_t)(sign | (uint8_t)code);
}

float g4o_fp8_e4m3_decode(uint8_t code) {
  const int e = (code >> 3) & 0xF, m = code & 7;
  float mag;
  if (e == 0xF && m == 7) {
    /* the reference maps the NaN slot to bf16 bits 0x7F80 / 0xFF80, which read
     * back as +-infinity */
    mag = INFINITY;
  } else if (e == 0) {
    mag = ldexpf((float)m, -9);
  } else {
    mag = ldexpf(1.0f + (float)m / 8.0f, e - 7);
  }
  return (code & 0x80) ? -mag : mag;
}

float g4o_kv8_scale(float amax) { return amax / 127.0f; }

int8_t g4o_kv8_quant(float x, float scale) {
  if (scale == 0.0f) return 0;
  const float r = roundf(x / scale); /* half away from zero */
  if (r > 127.0f) return 127;
  if (r < -127.0f) return -127;
  return (int8_t)(long long)r;
}

float g4o_kv8_dequant(int8_t q, float scale) { return scale * (float)q; }

float g4o_silu(float x) { return x / (1.0f + expf(-x)); }

/* ------------------------------------------------------------------------ */
/* xorshift64* input stream                                                  */
/* ------------------------------------------------------------------------ */

void g4o_rng_seed(g4o_rng* r, uint64_t seed) { r->s = seed ? seed : 0x9e3779b97f4a7c15ull; }

uint64_t g4o_rng_next(g4o_rng* r) {
  uint64_t s = r->s;
  s ^= s << 13;
  s ^= s >> 7;
  s ^= s << 17;
  r->s = s;
  return s * 0x2545F4914F6CDD1Dull;
}

float g4o_rng_float(g4o_rng* r) {
  const uint32_t u = (uint32_t)(g4o_rng_next(r) >> 41);
  return (float)u * 0x1p-23f;
}

float g4o_rng_range(g4o_rng* r, double a) {
  const float u = g4o_rng_float(r);
  return (u * 2.0f - 1.0f) * (float)a;
}

void g4o_fill_bf16(uint64_t seed, double a, long n, uint16_t* out) {
  g4o_rng r;
  g4o_rng_seed(&r, seed);
  for (long i = 0; i < n; ++i) out[i] = g4o_f32_to_bf16(g4o_rng_range(&r, a));
}

/* ------------------------------------------------------------------------ */
/* a1: embedding gather                                                      */
/* ------------------------------------------------------------------------ */

void g4o_embed_rows(const int32_t* tokens, long start, long rows, const uint16_t* emb,
                    float mult, uint16_t* out, int H) {
  for (long r = 0; r < rows; ++r) {
    const uint16_t* src = emb + (size_t)tokens[start + r] * (size_t)H;
    uint16_t* dst = out + (size_t)r * (size_t)H;
    for (int j = 0; j < H; ++j) dst[j] = g4o_f32_to_bf16(mult * g4o_bf16_to_f32(src[j]));
  }
}

/* ------------------------------------------------------------------------ */
/* a2 / a5: residual add + RMSNorm                                           */
/* ------------------------------------------------------------------------ */

void g4o_add_rmsnorm(const void* y, int y_is_f32, const void* res, int res_is_f32,
                     const uint16_t* w, float eps, float rm, long rows, int cols,
                     uint16_t* h_out, uint16_t* n_out) {
  float* h = (float*)malloc(sizeof(float) * (size_t)cols);
  for (long r = 0; r < rows; ++r) {
    const size_t base = (size_t)r * (size_t)cols;
    for (int i = 0; i < cols; ++i) {
      const float yv = y_is_f32 ? ((const float*)y)[base + i]
                                : g4o_bf16_to_f32(((const uint16_t*)y)[base + i]);
      float hv;
      if (res != NULL) {
        const float rv = res_is_f32 ? ((const float*)res)[base + i]
                                    : g4o_bf16_to_f32(((const uint16_t*)res)[base + i]);
        const float scaled = rm * yv; /* product rounded, then the add */
        hv = rv + scaled;
      } else {
        hv = yv;
      }
      const uint16_t hb = g4o_f32_to_bf16(hv);
      if (h_out) h_out[base + i] = hb;
      h[i] = g4o_bf16_to_f32(hb); /* the norm reads the bf16 hidden */
    }
    if (n_out) {
      double s = 0.0;
      for (int i = 0; i < cols; ++i) s += (double)h[i] * h[i];
      const float rr = 1.0f / sqrtf((float)(s / cols) + eps);
      for (int i = 0; i < cols; ++i) {
        const float hr = h[i] * rr;
        n_out[base + i] = g4o_f32_to_bf16(hr * g4o_bf16_to_f32(w[i]));
      }
    }
  }
  free(h);
}

void g4o_amax_bf16(const uint16_t* v, long n, float* amax_out) {
  float mx = 0.0f;
  for (long i = 0; i < n; ++i) {
    const float a = fabsf(g4o_bf16_to_f32(v[i]));
    if (a > mx) mx = a;
  }
  *amax_out = mx;
}

float g4o_fp8_scale_from_amax(float amax) { return (float)((double)amax / 448.0f); }

void g4o_quant_fp8_with_scale(const uint16_t* v, long n, float scale, uint8_t* codes) {
  for (long i = 0; i < n; ++i) {
    const double f = (double)g4o_bf16_to_f32(v[i]);
    codes[i] = g4o_fp8_e4m3_encode(scale > 0.0f ? f / (double)scale : f);
  }
}

/* ------------------------------------------------------------------------ */
/* a3: RoPE + int8 paged KV                                                  */
/* ------------------------------------------------------------------------ */

void g4o_rope_tables(double theta, int d, long max_pos, float* cos_tbl, float* sin_tbl) {
  const int half = d / 2;
  for (int i = 0; i < half; ++i) {
    const double inv_freq = 1.0 / pow(theta, 2.0 * (double)i / d);
    for (long p = 0; p < max_pos; ++p) {
      const double ang = (double)p * inv_freq;
      cos_tbl[(size_t)p * half + i] = (float)cos(ang);
      sin_tbl[(size_t)p * half + i] = (float)sin(ang);
    }
  }
}

/* one head: out[i] = a c - b s, out[i + d/2] = b c + a s, each product rounded */
static void rope_head_f32(const uint16_t* x, const float* c, const float* s, int d, float* out) {
  const int half = d / 2;
  for (int i = 0; i < half; ++i) {
    const float a = g4o_bf16_to_f32(x[i]);
    const float b = g4o_bf16_to_f32(x[i + half]);
    const float ac = a * c[i], bs = b * s[i], bc = b * c[i], as = a * s[i];
    out[i] = ac - bs;
    out[i + half] = bc + as;
  }
}

void g4o_rope_rows(const uint16_t* x, const float* cos_tbl, const float* sin_tbl, long rows,
                   int d, uint16_t* out) {
  float tmp[1024];
  const int half = d / 2;
  for (long r = 0; r < rows; ++r) {
    rope_head_f32(x + (size_t)r * d, cos_tbl + (size_t)r * half, sin_tbl + (size_t)r * half, d,
                  tmp);
    for (int i = 0; i < d; ++i) out[(size_t)r * d + i] = g4o_f32_to_bf16(tmp[i]);
  }
}

static void kv8_store_row(const float* v, int d, int8_t* codes, float* scale_out) {
  float amax = 0.0f;
  for (int i = 0; i < d; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float s = g4o_kv8_scale(amax);
  *scale_out = s;
  for (int i = 0; i < d; ++i) codes[i] = g4o_kv8_quant(v[i], s);
}

void g4o_rope_kv_int8(const uint16_t* qkv, const float* cos_tbl, const float* sin_tbl,
                      const int32_t* pos_rows, const int32_t* kv_rows, long rows, int Hq,
                      int Hk, int d, long stride, int k_from_bf16, uint16_t* q_rot,
                      int8_t* cache_k, int8_t* cache_v, float* k_scale, float* v_scale) {
  float tmp[1024];
  const int half = d / 2;
  const size_t nq = (size_t)Hq * d, nk = (size_t)Hk * d, pitch = nq + 2 * nk;
  for (long r = 0; r < rows; ++r) {
    const uint16_t* row = qkv + (size_t)r * pitch;
    const float* c = cos_tbl + (size_t)pos_rows[r] * half;
    const float* s = sin_tbl + (size_t)pos_rows[r] * half;
    for (int h = 0; h < Hq; ++h) {
      rope_head_f32(row + (size_t)h * d, c, s, d, tmp);
      for (int i = 0; i < d; ++i) q_rot[(size_t)r * nq + (size_t)h * d + i] = g4o_f32_to_bf16(tmp[i]);
    }
    for (int h = 0; h < Hk; ++h) {
      const size_t sc = (size_t)h * (size_t)stride + (size_t)kv_rows[r];
      rope_head_f32(row + nq + (size_t)h * d, c, s, d, tmp);
      if (k_from_bf16)
        for (int i = 0; i < d; ++i) tmp[i] = g4o_bf16_to_f32(g4o_f32_to_bf16(tmp[i]));
      kv8_store_row(tmp, d, cache_k + sc * d, k_scale + sc);
      for (int i = 0; i < d; ++i) tmp[i] = g4o_bf16_to_f32(row[nq + nk + (size_t)h * d + i]);
      kv8_store_row(tmp, d, cache_v + sc * d, v_scale + sc);
    }
  }
}

void g4o_kv_append_int8(const uint16_t* src_k, const uint16_t* src_v, const int32_t* kv_rows,
                        long rows, int Hk, int d, long stride, int8_t* cache_k,
                        int8_t* cache_v, float* k_scale, float* v_scale) {
  float tmp[1024];
  for (long r = 0; r < rows; ++r)
    for (int h = 0; h < Hk; ++h) {
      const size_t src = ((size_t)r * Hk + h) * d;
      const size_t sc = (size_t)h * (size_t)stride + (size_t)kv_rows[r];
      for (int i = 0; i < d; ++i) tmp[i] = g4o_bf16_to_f32(src_k[src + i]);
      kv8_store_row(tmp, d, cache_k + sc * d, k_scale + sc);
      for (int i = 0; i < d; ++i) tmp[i] = g4o_bf16_to_f32(src_v[src + i]);
      kv8_store_row(tmp, d, cache_v + sc * d, v_scale + sc);
    }
}

/* ------------------------------------------------------------------------ */
/* a4: SwiGLU                                                                */
/* ------------------------------------------------------------------------ */

void g4o_swiglu(const void* gate, const void* up, int in_is_f32, long ld, long rows, int I,
                uint16_t* act) {
  for (long r = 0; r < rows; ++r)
    for (int i = 0; i < I; ++i) {
      const size_t o = (size_t)r * (size_t)ld + i;
      const float g = in_is_f32 ? ((const float*)gate)[o] : g4o_bf16_to_f32(((const uint16_t*)gate)[o]);
      const float u = in_is_f32 ? ((const float*)up)[o] : g4o_bf16_to_f32(((const uint16_t*)up)[o]);
      const float sg = g4o_silu(g);
      act[(size_t)r * I + i] = g4o_f32_to_bf16(sg * u);
    }
}

void g4o_argmax_rows(const uint16_t* logits, long rows, int V, int32_t* out) {
  for (long r = 0; r < rows; ++r) {
    const uint16_t* p = logits + (size_t)r * V;
    int best = 0;
    float bv = g4o_bf16_to_f32(p[0]);
    for (int i = 1; i < V; ++i) {
      const float v = g4o_bf16_to_f32(p[i]);
      if (v > bv) {
        bv = v;
        best = i;
      }
    }
    out[r] = best;
  }
}

/* ------------------------------------------------------------------------ */
/* Decode attention over the int8 pool                                        */
/* ------------------------------------------------------------------------ */
/* The reference's golden pipeline, engine/src/kernel_math.h:265-331, on cache rows
 * dequantised the way its kernels do (engine/src/attention_split.cu:229-234:
 * bf16(code * scale)): logits rounded to bf16, softmax with the maximum
 * subtracted and the sum in double (:226-233), probabilities rounded to bf16,
 * value accumulation in float, output rounded to bf16. */
void g4o_attn_decode_int8(const uint16_t* q, const int8_t* ck, const int8_t* cv, const float* ks,
                          const float* vs, const int32_t* row_pos, const int32_t* const* row_pt,
                          long rows, int Hq, int Hk, int d, long stride, float scale,
                          uint16_t* out) {
  const int gh = Hq / Hk;
  for (long r = 0; r < rows; ++r) {
    const int len = row_pos[r] + 1;
    const int32_t* pt = row_pt != NULL ? row_pt[r] : NULL;
    for (int hq = 0; hq < Hq; ++hq) {
      uint16_t* o = out + ((size_t)r * Hq + hq) * d;
      if (len <= 0) {
        memset(o, 0, (size_t)d * sizeof(uint16_t));
        continue;
      }
      const int hkv = hq / gh;
      const uint16_t* qh = q + ((size_t)r * Hq + hq) * d;
      float* logit = (float*)malloc((size_t)len * sizeof(float));
      float* prob = (float*)malloc((size_t)len * sizeof(float));
      float m = -INFINITY;
      for (int t = 0; t < len; ++t) {
        const size_t row = (size_t)hkv * stride + (pt != NULL ? pt[t] : t);
        float acc = 0.0f;
        for (int i = 0; i < d; ++i) {
          const float k = g4o_bf16_to_f32(g4o_f32_to_bf16(g4o_kv8_dequant(ck[row * d + i], ks[row])));
          acc += k * g4o_bf16_to_f32(qh[i]);
        }
        logit[t] = g4o_bf16_to_f32(g4o_f32_to_bf16(scale * acc));
        if (logit[t] > m) m = logit[t];
      }
      double sum = 0.0;
      for (int t = 0; t < len; ++t) sum += exp((double)(logit[t] - m));
      for (int t = 0; t < len; ++t)
        prob[t] = g4o_bf16_to_f32(g4o_f32_to_bf16((float)(exp((double)(logit[t] - m)) / sum)));
      for (int i = 0; i < d; ++i) {
        float acc = 0.0f;
        for (int t = 0; t < len; ++t) {
          const size_t row = (size_t)hkv * stride + (pt != NULL ? pt[t] : t);
          const float v = g4o_bf16_to_f32(g4o_f32_to_bf16(g4o_kv8_dequant(cv[row * d + i], vs[row])));
          acc += prob[t] * v;
        }
        o[i] = g4o_f32_to_bf16(acc);
      }
      free(logit);
      free(prob);
    }
  }
}

/* ------------------------------------------------------------------------ */
/* FP8 x FP8 GEMM                                                            */
/* ------------------------------------------------------------------------ */
void g4o_gemm_fp8(const uint8_t* a, long lda, const uint8_t* w, long M, long N, long K,
                  float a_scale, float s0, float s1, float s2, long seg1, long seg2, int out_kind,
                  const uint16_t* residual, float resid_scale, long ldc, uint16_t* out_bf16,
                  float* out_f32) {
  float lut[256];
  for (int c = 0; c < 256; ++c) lut[c] = g4o_fp8_e4m3_decode((uint8_t)c);
  for (long m = 0; m < M; ++m)
    for (long n = 0; n < N; ++n) {
      const uint8_t* ar = a + (size_t)m * lda;
      const uint8_t* wr = w + (size_t)n * K;
      float acc = 0.0f;
      for (long k = 0; k < K; ++k) acc += lut[wr[k]] * lut[ar[k]];
      const float ws = n < seg1 ? s0 : (n < seg2 ? s1 : s2);
      const float y = (a_scale * ws) * acc;
      const size_t off = (size_t)m * ldc + n;
      if (out_kind == 1) {
        out_f32[off] = y;
      } else if (out_kind == 0) {
        out_bf16[off] = g4o_f32_to_bf16(y);
      } else {
        out_bf16[off] = g4o_f32_to_bf16(g4o_bf16_to_f32(residual[off]) + resid_scale * y);
      }
    }
}
