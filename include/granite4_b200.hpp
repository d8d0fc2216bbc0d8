// C++ launch entry points of libgranite4_b200.so, under the names and
// signatures the reference engine's forward pass calls (namespace granite4), so
// engine/src/forward_gpu.cu and engine/tests/test_kernels.cu resolve them
// against this library without source changes. Each forwards to the C entry
// point of the same meaning in granite4_b200.h; conventions are described there.
#ifndef GRANITE4_B200_HPP
#define GRANITE4_B200_HPP

#include <cstdint>

#include "granite4_b200.h"

namespace granite4 {

// engine/src/model_config.h:56, engine/src/forward_gpu_api.h:161
constexpr int kMaxVerifyRows = GRANITE4_MAX_VERIFY_ROWS;
constexpr int kMaxTreeDepth = GRANITE4_MAX_TREE_DEPTH;

// engine/src/forward_gpu_api.h:162-182 (same member order and types; the C
// struct granite4_multi_rows is its layout twin).
struct GpuMultiRows {
  int n;
  int pos[kMaxVerifyRows];
  const int* pt[kMaxVerifyRows];
  std::int32_t* tok[kMaxVerifyRows];
  int grp[kMaxVerifyRows];
  int tree;
  int slot[kMaxVerifyRows];
  int tbase[kMaxVerifyRows];
  int tail[kMaxVerifyRows][kMaxTreeDepth];
};
static_assert(sizeof(GpuMultiRows) == sizeof(granite4_multi_rows), "descriptor layout");

// engine/src/prefill_gemm.h:42-43
int prefill_embed_rows(const std::int32_t* d_tokens, int start, int rows, const std::uint16_t* emb,
                       float mult, std::uint16_t* out, int H);
// engine/src/prefill_gemm.h:58-64
int prefill_rope_split_append_int8(const std::uint16_t* qkv, const float* cos_tbl,
                                   const float* sin_tbl, int base_pos, int rows, int Hq, int Hk,
                                   int d, int stride, std::uint16_t* q_rot, std::int8_t* cache_k,
                                   std::int8_t* cache_v, float* cache_k_scale,
                                   float* cache_v_scale, const int* d_pt = nullptr);
// engine/src/prefill_gemm.h:86-101. Only int8 == true (and no int4 / k5 / window) is built; anything
// else returns -1, the reference's "take the other attention path".
int prefill_attention(const std::uint16_t* q_rot, const std::uint16_t* cache_k, const std::uint16_t* cache_v,
                      float scale, int Hq, int Hk, int d, int base_pos, int rows, int stride,
                      std::uint16_t* out, const std::int8_t* cache_k8, const std::int8_t* cache_v8,
                      const float* k_scale, const float* v_scale, bool int8, const std::uint8_t* cache_k4,
                      const std::uint8_t* cache_v4, bool int4, const int* d_pt = nullptr, bool k5 = false,
                      int window = 0);
// engine/src/prefill_gemm.h:105
int prefill_silu_mul(const float* gu, int I, int rows, std::uint16_t* act);
// engine/src/forward_gpu_api.h:224-227
int gpu_multi_rope_append(const std::uint16_t* q, const std::uint16_t* k, const std::uint16_t* v,
                          const float* cos_tbl, const float* sin_tbl, const GpuMultiRows* d_rows,
                          int rows, int Hq, int Hk, int d, int bits, void* cache_k, void* cache_v,
                          float* k_scale, float* v_scale, int stride, std::uint16_t* q_rot);
// engine/src/forward_gpu_api.h:219-220
int gpu_multi_rope(const std::uint16_t* x, const float* cos_tbl, const float* sin_tbl,
                   const GpuMultiRows* d_rows, int rows, int heads, int d, std::uint16_t* out);
// engine/src/forward_gpu_api.h:227-229
int gpu_multi_kv_append(const std::uint16_t* k, const std::uint16_t* v, int bits, void* cache_k,
                        void* cache_v, float* k_scale, float* v_scale, const GpuMultiRows* d_rows,
                        int rows, int stride, int Hk, int d);
// engine/src/prefill_gemm.h:48-52
int prefill_rope_split_append(const std::uint16_t* qkv, const float* cos_tbl, const float* sin_tbl,
                              int base_pos, int rows, int Hq, int Hk, int d, int stride,
                              std::uint16_t* q_rot, std::uint16_t* cache_k, std::uint16_t* cache_v,
                              const int* d_pt = nullptr);

}  // namespace granite4

#endif  // GRANITE4_B200_HPP
