/* CPU oracle for the Granite 4.2 8B per-layer glue kernels.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the reference
 * engine's fp32 "golden" formulation of the five glue ops. Nothing that ships
 * calls it: it is the checker the CUDA path is compared with, and the code
 * the CPU-baseline leg of the benchmark times. It is pinned against the
 * reference's own known-answer tests and against the reference's host code
 * compiled as-is (see oracle/Makefile, target _ref).
 *
 * Every function cites the reference file:line it follows (paths are relative
 * to the reference project root).
 */
#ifndef G4_ORACLE_H
#define G4_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalar codecs ------------------------------------------------------ */

/* engine/src/kernel_math.h:39-44 */
float g4o_bf16_to_f32(uint16_t bits);
/* engine/src/kernel_math.h:49-55 (round to nearest, ties to even) */
uint16_t g4o_f32_to_bf16(float f);
/* engine/src/fp8_convert.cc:47-122: RNE to e4m3, |v| >= 464 clips to +-448,
 * NaN -> 0x7F, -0 keeps its sign. */
uint8_t g4o_fp8_e4m3_encode(double v);
/* engine/src/fp8_convert.cc:128-157 followed by kernel_math.h:59-61 */
float g4o_fp8_e4m3_decode(uint8_t code);
/* engine/src/kernel_math.h:71-86 */
float g4o_kv8_scale(float amax);
int8_t g4o_kv8_quant(float x, float scale);
float g4o_kv8_dequant(int8_t q, float scale);
/* engine/src/kernel_math.h:239 */
float g4o_silu(float x);

/* ---- deterministic input stream (engine/src/kernel_math.h:637-658) ------- */
typedef struct { uint64_t s; } g4o_rng;
void g4o_rng_seed(g4o_rng* r, uint64_t seed);
uint64_t g4o_rng_next(g4o_rng* r);
float g4o_rng_float(g4o_rng* r);               /* [0,1) */
float g4o_rng_range(g4o_rng* r, double a);     /* [-a,a) */
/* fills n bf16 values = bf16(range(a)), the generator the reference's device
 * tests use (engine/tests/test_kernels.cu:238-240 with a = 4.0) */
void g4o_fill_bf16(uint64_t seed, double a, long n, uint16_t* out);

/* ---- op a1: embedding gather x multiplier -------------------------------
 * out[r][j] = bf16(mult * f32(emb[tokens[start + r]][j]))
 * engine/src/prefill_gemm.cu:281-301, engine/src/device_math.cuh:258-265 */
void g4o_embed_rows(const int32_t* tokens, long start, long rows, const uint16_t* emb,
                    float mult, uint16_t* out, int H);

/* ---- op a2 / a5: residual add + RMSNorm ---------------------------------
 * h = bf16(f32(res) + rm * y)   (engine/src/kernel_math.h:528-529,
 *                                engine/src/prefill_gemm.cu:81-88)
 * n = bf16(h * r * w), r = 1.0f / sqrtf(float(sum_double(h^2) / cols) + eps)
 *                               (engine/src/kernel_math.h:178-184)
 * y: bf16 (y_is_f32 == 0) or f32; res: bf16 (res_is_f32 == 0) or f32, or NULL
 * (then h = bf16(y), and with y already bf16 the op is the plain / final norm).
 * h_out and n_out may each be NULL. */
void g4o_add_rmsnorm(const void* y, int y_is_f32, const void* res, int res_is_f32,
                     const uint16_t* w, float eps, float rm, long rows, int cols,
                     uint16_t* h_out, uint16_t* n_out);

/* Per-tensor FP8 quantisation of a bf16 tensor, the reference's weight
 * quantiser applied to activations: scale = float(amax / 448), code =
 * encode(double(v) / double(scale)), scale == 0 -> encode(v).
 * engine/src/checkpoint_main.cc:118-122, :702-723. Returns amax via *amax_out
 * (may be NULL). */
void g4o_amax_bf16(const uint16_t* v, long n, float* amax_out);
float g4o_fp8_scale_from_amax(float amax);
void g4o_quant_fp8_with_scale(const uint16_t* v, long n, float scale, uint8_t* codes);

/* ---- op a3: RoPE tables, RoPE(q,k) + int8 paged KV write ------------------
 * tables: engine/src/kernel_math.h:191-206 (double math, f32 storage,
 * [max_pos][d/2]). */
void g4o_rope_tables(double theta, int d, long max_pos, float* cos_tbl, float* sin_tbl);
/* plain RoPE of rows of one head each, table row = row index
 * (engine/src/kernel_math.h:208-219, engine/src/kernels_phase2.cu:138-162) */
void g4o_rope_rows(const uint16_t* x, const float* cos_tbl, const float* sin_tbl, long rows,
                   int d, uint16_t* out);
/* Token-major qkv [rows][(Hq + 2 Hk) d]; row r has RoPE position pos_rows[r]
 * and is written to pool row kv_rows[r].
 *   q_rot[r][h][:] = bf16(rope(q))
 *   K: k' = rope(k) kept in f32 (k_from_bf16 == 0, the prefill kernel,
 *      engine/src/prefill_gemm.cu:356-428) or rounded to bf16 first
 *      (k_from_bf16 == 1, the decode / verify kernel,
 *      engine/src/forward_gpu.cu:598-665); per (row, kv head): amax, s = amax /
 *      127, codes = clamp(round_half_away(k' / s)); V the same on the raw v.
 *   code offset (hkv * stride + kv_row) * d, scale offset hkv * stride + kv_row
 */
void g4o_rope_kv_int8(const uint16_t* qkv, const float* cos_tbl, const float* sin_tbl,
                      const int32_t* pos_rows, const int32_t* kv_rows, long rows, int Hq,
                      int Hk, int d, long stride, int k_from_bf16, uint16_t* q_rot,
                      int8_t* cache_k, int8_t* cache_v, float* k_scale, float* v_scale);
/* bf16 K/V rows quantised and appended (engine/src/kernels_phase2.cu:405-450) */
void g4o_kv_append_int8(const uint16_t* src_k, const uint16_t* src_v, const int32_t* kv_rows,
                        long rows, int Hk, int d, long stride, int8_t* cache_k,
                        int8_t* cache_v, float* k_scale, float* v_scale);

/* ---- op a4: SwiGLU --------------------------------------------------------
 * act = bf16(silu(g) * u), silu(g) = g / (1 + expf(-g))
 * (engine/src/kernel_math.h:239, :571-584). gate/up rows have pitch ld
 * elements; in_is_f32 selects f32 inputs (the reference prefill form,
 * engine/src/prefill_gemm.cu:1194-1203, takes f32 [rows][2 I]). */
void g4o_swiglu(const void* gate, const void* up, int in_is_f32, long ld, long rows, int I,
                uint16_t* act);

/* Greedy pick: out[r] = first index of the maximum of bf16 logits row r
 * (engine/src/kernel_math.h:592-601 sample_greedy_f32: strict > keeps the first
 * maximum). Rows without NaN only: the host rule starts from element 0 whatever
 * it is, the device kernel (engine/src/forward_gpu.cu:284-333) skips NaN. */
void g4o_argmax_rows(const uint16_t* logits, long rows, int V, int32_t* out);

/* Decode attention over the int8 pool, one independent sequence per query row:
 * row r attends to cache positions 0..row_pos[r], position t in pool row
 * row_pt[r][t] (row_pt == NULL: t). The reference's golden pipeline
 * (engine/src/kernel_math.h:265-331) over rows dequantised to bf16. */
void g4o_attn_decode_int8(const uint16_t* q, const int8_t* ck, const int8_t* cv, const float* ks,
                          const float* vs, const int32_t* row_pos, const int32_t* const* row_pt,
                          long rows, int Hq, int Hk, int d, long stride, float scale,
                          uint16_t* out);

/* FP8 x FP8 GEMM with the reference's epilogue. The contraction is the reference's
 * golden GEMM (engine/src/kernel_math.h:250-262: every element decoded exactly,
 * products accumulated in float in k order) applied to A given as e4m3 codes
 * (their decoded values are exact in bf16, the type that golden takes);
 * y = (a_scale * w_scale(n)) * acc with w_scale(n) = s0 for n < seg1, s1 for
 * n < seg2, else s2, and the three output kinds of
 * engine/src/prefill_gemm.cu:65-88: 0 bf16(y), 1 f32 y, 2 bf16(residual +
 * resid_scale * y). out / residual rows have pitch ldc elements. */
void g4o_gemm_fp8(const uint8_t* a, long lda, const uint8_t* w, long M, long N, long K,
                  float a_scale, float s0, float s1, float s2, long seg1, long seg2, int out_kind,
                  const uint16_t* residual, float resid_scale, long ldc, uint16_t* out_bf16,
                  float* out_f32);

#ifdef __cplusplus
}
#endif
#endif
