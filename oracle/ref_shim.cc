// C-ABI shim over the reference engine's OWN host code, compiled from where it
// lies (see oracle/Makefile, target _ref). TEST INFRASTRUCTURE ONLY.
//
// The reference's fp32 golden math is header-only inline C++
// (engine/src/kernel_math.h) plus one translation unit
// (engine/src/fp8_convert.cc). This file adds no arithmetic of its own: each
// export either forwards to a reference function or loops it over rows with
// the rounding points the reference's kernels use. The one rule that cannot be
// linked (a static function in engine/src/checkpoint_main.cc:118-122,
// :702-723) is the per-tensor FP8 scale: scale = float(max_abs / 448.0f),
// code = fp8_e4m3_encode(double(v) / double(scale)), scale == 0 -> encode(v).
//
// Used to (1) validate the plain-C restatement in g4_oracle.c bit for bit and
// (2) serve as the "reference" CPU baseline the benchmark times.
#include "kernel_math.h"  // from the reference tree, via -I

#include <cstdint>
#include <cstring>
#include <vector>

using namespace granite4;

extern "C" {

float g4ref_bf16_to_f32(std::uint16_t b) { return bf16_to_f32_host(b); }
std::uint16_t g4ref_f32_to_bf16(float f) { return f32_to_bf16_host(f); }
std::uint8_t g4ref_fp8_e4m3_encode(double v) { return fp8_e4m3_encode(v, nullptr); }
float g4ref_fp8_e4m3_decode(std::uint8_t c) { return fp8_to_f32_host(c); }
float g4ref_kv8_scale(float amax) { return kv8_scale_host(amax); }
std::int8_t g4ref_kv8_quant(float x, float s) { return kv8_quant_host(x, s); }
float g4ref_kv8_dequant(std::int8_t q, float s) { return kv8_dequant_host(q, s); }
float g4ref_silu(float x) { return silu_f32(x); }

void g4ref_fill_bf16(std::uint64_t seed, double a, long n, std::uint16_t* out) {
  Xorshift64 rng(seed);
  for (long i = 0; i < n; ++i) out[i] = f32_to_bf16_host(rng.next_float_range(a));
}
void g4ref_rng_u64(std::uint64_t seed, long n, std::uint64_t* out) {
  Xorshift64 rng(seed);
  for (long i = 0; i < n; ++i) out[i] = rng.next();
}

void g4ref_embed_rows(const std::int32_t* tokens, long start, long rows, const std::uint16_t* emb,
                      float mult, std::uint16_t* out, int H) {
  for (long r = 0; r < rows; ++r) {
    const std::uint16_t* src = emb + static_cast<std::size_t>(tokens[start + r]) * H;
    for (int j = 0; j < H; ++j)
      out[static_cast<std::size_t>(r) * H + j] = f32_to_bf16_host(mult * bf16_to_f32_host(src[j]));
  }
}

void g4ref_add_rmsnorm(const void* y, int y_is_f32, const void* res, int res_is_f32,
                       const std::uint16_t* w, float eps, float rm, long rows, int cols,
                       std::uint16_t* h_out, std::uint16_t* n_out) {
  std::vector<float> h(cols), wf(cols), out(cols);
  for (int i = 0; i < cols; ++i) wf[i] = bf16_to_f32_host(w[i]);
  for (long r = 0; r < rows; ++r) {
    const std::size_t base = static_cast<std::size_t>(r) * cols;
    for (int i = 0; i < cols; ++i) {
      const float yv = y_is_f32 ? static_cast<const float*>(y)[base + i]
                                : bf16_to_f32_host(static_cast<const std::uint16_t*>(y)[base + i]);
      float hv = yv;
      if (res != nullptr) {
        float acc = res_is_f32 ? static_cast<const float*>(res)[base + i]
                               : bf16_to_f32_host(static_cast<const std::uint16_t*>(res)[base + i]);
        acc += rm * yv;  // the reference's "residual[r] += residual_multiplier * out[r]"
        hv = acc;
      }
      const std::uint16_t hb = f32_to_bf16_host(hv);
      if (h_out) h_out[base + i] = hb;
      h[i] = bf16_to_f32_host(hb);
    }
    if (n_out) {
      rmsnorm_f32(h.data(), wf.data(), eps, cols, out.data());
      for (int i = 0; i < cols; ++i) n_out[base + i] = f32_to_bf16_host(out[i]);
    }
  }
}

void g4ref_amax_bf16(const std::uint16_t* v, long n, float* amax_out) {
  double mx = 0.0;
  for (long i = 0; i < n; ++i) {
    const float f = bf16_to_f32_host(v[i]);
    const double a = f < 0.0 ? -static_cast<double>(f) : static_cast<double>(f);
    if (a > mx) mx = a;
  }
  *amax_out = static_cast<float>(mx);
}
float g4ref_fp8_scale_from_amax(float amax) {
  return static_cast<float>(static_cast<double>(amax) / kFp8E4M3MaxF);
}
void g4ref_quant_fp8_with_scale(const std::uint16_t* v, long n, float scale, std::uint8_t* codes) {
  for (long i = 0; i < n; ++i) {
    const float f = bf16_to_f32_host(v[i]);
    codes[i] = scale > 0.0f
                   ? fp8_e4m3_encode(static_cast<double>(f) / static_cast<double>(scale), nullptr)
                   : bf16_to_fp8_e4m3(v[i], nullptr);
  }
}

void g4ref_rope_tables(double theta, int d, long max_pos, float* cos_tbl, float* sin_tbl) {
  std::vector<float> c, s;
  rope_freqs_f32(theta, d, static_cast<int>(max_pos), &c, &s);
  std::memcpy(cos_tbl, c.data(), c.size() * sizeof(float));
  std::memcpy(sin_tbl, s.data(), s.size() * sizeof(float));
}

void g4ref_rope_rows(const std::uint16_t* x, const float* cos_tbl, const float* sin_tbl, long rows,
                     int d, std::uint16_t* out) {
  std::vector<float> xr(d), yr(d);
  const int half = d / 2;
  for (long r = 0; r < rows; ++r) {
    for (int i = 0; i < d; ++i) xr[i] = bf16_to_f32_host(x[static_cast<std::size_t>(r) * d + i]);
    rope_half_f32(xr.data(), cos_tbl + static_cast<std::size_t>(r) * half,
                  sin_tbl + static_cast<std::size_t>(r) * half, d, yr.data());
    for (int i = 0; i < d; ++i) out[static_cast<std::size_t>(r) * d + i] = f32_to_bf16_host(yr[i]);
  }
}

static void ref_kv8_row(const float* v, int d, std::int8_t* codes, float* scale_out) {
  float amax = 0.0f;
  for (int i = 0; i < d; ++i) amax = std::max(amax, std::fabs(v[i]));
  const float s = kv8_scale_host(amax);
  *scale_out = s;
  for (int i = 0; i < d; ++i) codes[i] = kv8_quant_host(v[i], s);
}

void g4ref_rope_kv_int8(const std::uint16_t* qkv, const float* cos_tbl, const float* sin_tbl,
                        const std::int32_t* pos_rows, const std::int32_t* kv_rows, long rows, int Hq,
                        int Hk, int d, long stride, int k_from_bf16, std::uint16_t* q_rot,
                        std::int8_t* cache_k, std::int8_t* cache_v, float* k_scale,
                        float* v_scale) {
  std::vector<float> xr(d), yr(d);
  const int half = d / 2;
  const std::size_t nq = static_cast<std::size_t>(Hq) * d, nk = static_cast<std::size_t>(Hk) * d;
  for (long r = 0; r < rows; ++r) {
    const std::uint16_t* row = qkv + static_cast<std::size_t>(r) * (nq + 2 * nk);
    const float* c = cos_tbl + static_cast<std::size_t>(pos_rows[r]) * half;
    const float* s = sin_tbl + static_cast<std::size_t>(pos_rows[r]) * half;
    for (int h = 0; h < Hq; ++h) {
      for (int i = 0; i < d; ++i) xr[i] = bf16_to_f32_host(row[static_cast<std::size_t>(h) * d + i]);
      rope_half_f32(xr.data(), c, s, d, yr.data());
      for (int i = 0; i < d; ++i)
        q_rot[static_cast<std::size_t>(r) * nq + static_cast<std::size_t>(h) * d + i] =
            f32_to_bf16_host(yr[i]);
    }
    for (int h = 0; h < Hk; ++h) {
      const std::size_t sc =
          static_cast<std::size_t>(h) * static_cast<std::size_t>(stride) + kv_rows[r];
      for (int i = 0; i < d; ++i)
        xr[i] = bf16_to_f32_host(row[nq + static_cast<std::size_t>(h) * d + i]);
      rope_half_f32(xr.data(), c, s, d, yr.data());
      if (k_from_bf16)
        for (int i = 0; i < d; ++i) yr[i] = bf16_to_f32_host(f32_to_bf16_host(yr[i]));
      ref_kv8_row(yr.data(), d, cache_k + sc * d, k_scale + sc);
      for (int i = 0; i < d; ++i)
        xr[i] = bf16_to_f32_host(row[nq + nk + static_cast<std::size_t>(h) * d + i]);
      ref_kv8_row(xr.data(), d, cache_v + sc * d, v_scale + sc);
    }
  }
}

void g4ref_kv_append_int8(const std::uint16_t* src_k, const std::uint16_t* src_v,
                          const std::int32_t* kv_rows, long rows, int Hk, int d, long stride,
                          std::int8_t* cache_k, std::int8_t* cache_v, float* k_scale,
                          float* v_scale) {
  std::vector<float> xr(d);
  for (long r = 0; r < rows; ++r)
    for (int h = 0; h < Hk; ++h) {
      const std::size_t src = (static_cast<std::size_t>(r) * Hk + h) * d;
      const std::size_t sc =
          static_cast<std::size_t>(h) * static_cast<std::size_t>(stride) + kv_rows[r];
      for (int i = 0; i < d; ++i) xr[i] = bf16_to_f32_host(src_k[src + i]);
      ref_kv8_row(xr.data(), d, cache_k + sc * d, k_scale + sc);
      for (int i = 0; i < d; ++i) xr[i] = bf16_to_f32_host(src_v[src + i]);
      ref_kv8_row(xr.data(), d, cache_v + sc * d, v_scale + sc);
    }
}

void g4ref_swiglu(const void* gate, const void* up, int in_is_f32, long ld, long rows, int I,
                  std::uint16_t* act) {
  for (long r = 0; r < rows; ++r)
    for (int i = 0; i < I; ++i) {
      const std::size_t o = static_cast<std::size_t>(r) * ld + i;
      const float g = in_is_f32 ? static_cast<const float*>(gate)[o]
                                : bf16_to_f32_host(static_cast<const std::uint16_t*>(gate)[o]);
      const float u = in_is_f32 ? static_cast<const float*>(up)[o]
                                : bf16_to_f32_host(static_cast<const std::uint16_t*>(up)[o]);
      act[static_cast<std::size_t>(r) * I + i] = f32_to_bf16_host(silu_f32(g) * u);
    }
}

// The reference's golden attention (gqa_attention_bf16, kernel_math.h:312-331) on the cache rows
// of each query row's sequence, gathered through its table and dequantised to bf16 as the
// reference's attention kernels do (attention_split.cu:229-234).
void g4ref_attn_decode_int8(const std::uint16_t* q, const std::int8_t* ck, const std::int8_t* cv,
                            const float* ks, const float* vs, const std::int32_t* row_pos,
                            const std::int32_t* const* row_pt, long rows, int Hq, int Hk, int d,
                            long stride, float scale, std::uint16_t* out) {
  for (long r = 0; r < rows; ++r) {
    const int len = row_pos[r] + 1;
    std::uint16_t* o = out + static_cast<std::size_t>(r) * Hq * d;
    if (len <= 0) {
      std::memset(o, 0, static_cast<std::size_t>(Hq) * d * sizeof(std::uint16_t));
      continue;
    }
    std::vector<std::uint16_t> k(static_cast<std::size_t>(Hk) * len * d), v(k.size());
    for (int h = 0; h < Hk; ++h)
      for (int t = 0; t < len; ++t) {
        const std::size_t row = static_cast<std::size_t>(h) * stride + (row_pt != nullptr ? row_pt[r][t] : t);
        for (int i = 0; i < d; ++i) {
          k[(static_cast<std::size_t>(h) * len + t) * d + i] =
              f32_to_bf16_host(kv8_dequant_host(ck[row * d + i], ks[row]));
          v[(static_cast<std::size_t>(h) * len + t) * d + i] =
              f32_to_bf16_host(kv8_dequant_host(cv[row * d + i], vs[row]));
        }
      }
    std::vector<std::uint16_t> res;
    gqa_attention_bf16(q + static_cast<std::size_t>(r) * Hq * d, k.data(), v.data(), scale, Hq, Hk, d, len,
                       &res);
    std::memcpy(o, res.data(), res.size() * sizeof(std::uint16_t));
  }
}

void g4ref_argmax_rows(const std::uint16_t* logits, long rows, int V, std::int32_t* out) {
  std::vector<float> f(V);
  for (long r = 0; r < rows; ++r) {
    for (int i = 0; i < V; ++i) f[i] = bf16_to_f32_host(logits[static_cast<std::size_t>(r) * V + i]);
    out[r] = sample_greedy_f32(f.data(), V);
  }
}

// The reference's golden GEMM (gemm_dequant_f32, kernel_math.h:250-262) on activations given as
// e4m3 codes: their decoded values are exact in bf16, the type the golden takes. scale 1 leaves
// the float accumulator as it is; the epilogue is prefill_gemm.cu:65-88 restated.
void g4ref_gemm_fp8(const std::uint8_t* a, long lda, const std::uint8_t* w, long M, long N, long K,
                    float a_scale, float s0, float s1, float s2, long seg1, long seg2, int out_kind,
                    const std::uint16_t* residual, float resid_scale, long ldc,
                    std::uint16_t* out_bf16, float* out_f32) {
  std::vector<std::uint16_t> A(static_cast<std::size_t>(M) * K);
  for (long m = 0; m < M; ++m)
    for (long k = 0; k < K; ++k)
      A[static_cast<std::size_t>(m) * K + k] = f32_to_bf16_host(fp8_to_f32_host(a[static_cast<std::size_t>(m) * lda + k]));
  std::vector<float> acc;
  gemm_dequant_f32(A.data(), w, 1.0f, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), &acc);
  for (long m = 0; m < M; ++m)
    for (long n = 0; n < N; ++n) {
      const float ws = n < seg1 ? s0 : (n < seg2 ? s1 : s2);
      const float y = (a_scale * ws) * acc[static_cast<std::size_t>(m) * N + n];
      const std::size_t off = static_cast<std::size_t>(m) * ldc + n;
      if (out_kind == 1)
        out_f32[off] = y;
      else if (out_kind == 0)
        out_bf16[off] = f32_to_bf16_host(y);
      else
        out_bf16[off] = f32_to_bf16_host(bf16_to_f32_host(residual[off]) + resid_scale * y);
    }
}

}  // extern "C"
