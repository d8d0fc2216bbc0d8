// RoPE and KV append for a bf16 KV cache, and the RoPE-only primitives: the
// entry points of the reference that sit beside the int8 path (its bf16 cache
// format, its verify staging step and its multi-row helpers).
//
// Formulation (reference: engine/src/forward_gpu.cu:380-425 rope_multi_kernel /
// kv_append_multi_kernel, :796-854 rope_at_pos(_batched)_kernel, :3847-3874
// granite4_kernel_verify_qkv_stage; engine/src/prefill_gemm.cu:306-347
// rope_split_append_kernel; engine/src/kernels_phase2.cu:381-400
// kv_append_batched_kernel):
//   rotate  (a, b) = (x[i], x[i + d/2]): out[i] = bf16(a c - b s),
//           out[i + d/2] = bf16(b c + a s), c / s from table row `pos`
//   append  cache[(hkv * stride + kv_row) * d + i] = value (rotated K, raw V)
//
// One kernel serves all of them. A CTA owns one token row; its work is cut into
// items (head, j): item j of a head is the chunk [j C, j C + C) of the low half
// and the same chunk of the high half, i.e. both sides of C rotation pairs, so a
// rotation needs no exchange. C = 8 (128-bit accesses) when d is a multiple of
// 16 and everything is 16-byte aligned, else C = 1. Q heads rotate into q_rot;
// K heads rotate (or not) into k_rot and / or the cache; V heads are copied.
#include "g4_host.h"
#include "g4_math.cuh"

#include "../../include/granite4_b200.h"
#include "../../include/granite4_b200.hpp"

namespace g4 {
namespace {

enum TableMode { kTableRowIsRow = 0, kTableRowIsPos = 1, kTableDescriptor = 2 };
enum SlotMode { kSlotRun = 0, kSlotDescriptor = 1 };

struct RopeBf16Params {
  const uint16_t* q;  // NULL: no q
  const uint16_t* k;  // NULL: no k
  const uint16_t* v;  // NULL: no v
  long long pitch_q, pitch_k, pitch_v;  // row pitches, elements
  const float* cos_tbl;
  const float* sin_tbl;
  uint16_t* q_rot;    // [rows][Hq * d]
  uint16_t* k_rot;    // [rows][Hk * d] or NULL
  uint16_t* cache_k;  // [Hk][stride][d] or NULL
  uint16_t* cache_v;
  int table_mode, slot_mode;
  int base_pos;
  const int* d_pt;
  const granite4_multi_rows* mr;
  int rows, Hq, Hk, d;
  long long stride;
  int rotate_k;
};

template <int C>
struct Chunk;
template <>
struct Chunk<8> {
  uint4 raw;
  __device__ void load(const uint16_t* p) { raw = ld_stream(reinterpret_cast<const uint4*>(p)); }
  __device__ void store(uint16_t* p) const { *reinterpret_cast<uint4*>(p) = raw; }
  __device__ void to_f32(float (&f)[8]) const { unpack8(raw, f); }
  __device__ void from_f32(const float (&f)[8]) { raw = pack8(f); }
};
template <>
struct Chunk<1> {
  uint16_t raw;
  __device__ void load(const uint16_t* p) { raw = *p; }
  __device__ void store(uint16_t* p) const { *p = raw; }
  __device__ void to_f32(float (&f)[1]) const { f[0] = bf16_to_f32(raw); }
  __device__ void from_f32(const float (&f)[1]) { raw = static_cast<uint16_t>(f32_to_bf16_bits(f[0])); }
};

template <int C>
__global__ void __launch_bounds__(256) rope_bf16_kernel(const RopeBf16Params p) {
  const int r = blockIdx.x;
  const int half = p.d / 2;
  const int per_head = half / C;  // items per head
  const int Hq = p.q != nullptr ? p.Hq : 0;
  const int Hk = p.k != nullptr ? p.Hk : 0;
  const int Hv = p.v != nullptr ? p.Hk : 0;
  const int items = (Hq + Hk + Hv) * per_head;

  int pos = 0, kv_row = 0;
  if (p.table_mode == kTableRowIsRow) pos = r;
  else if (p.table_mode == kTableRowIsPos) pos = p.base_pos + r;
  else pos = p.mr->pos[r];
  if (p.cache_k == nullptr && p.cache_v == nullptr) {
    // RoPE only: the page tables are not looked at (a descriptor may carry none)
  } else if (p.slot_mode == kSlotRun) {
    const int at = p.base_pos + r;
    kv_row = p.d_pt != nullptr ? __ldg(p.d_pt + at) : at;
  } else {
    const int slot = p.mr->tree ? p.mr->slot[r] : p.mr->pos[r];
    kv_row = p.mr->pt[r][slot];
  }
  const float* cos_row = p.cos_tbl != nullptr ? p.cos_tbl + static_cast<size_t>(pos) * half : nullptr;
  const float* sin_row = p.sin_tbl != nullptr ? p.sin_tbl + static_cast<size_t>(pos) * half : nullptr;

  for (int it = threadIdx.x; it < items; it += blockDim.x) {
    const int head = it / per_head;
    const int i0 = (it - head * per_head) * C;  // first column of the low-half chunk
    const bool is_q = head < Hq;
    const bool is_k = !is_q && head < Hq + Hk;
    const uint16_t* src;
    int hh;  // head index within its own tensor
    if (is_q) hh = head, src = p.q + static_cast<size_t>(r) * p.pitch_q;
    else if (is_k) hh = head - Hq, src = p.k + static_cast<size_t>(r) * p.pitch_k;
    else hh = head - Hq - Hk, src = p.v + static_cast<size_t>(r) * p.pitch_v;
    src += static_cast<size_t>(hh) * p.d + i0;
    Chunk<C> lo, hi;
    lo.load(src);
    hi.load(src + half);
    if (is_q || (is_k && p.rotate_k)) {
      float a[C], b[C], ya[C], yb[C];
      lo.to_f32(a);
      hi.to_f32(b);
#pragma unroll
      for (int e = 0; e < C; ++e) rope_pair(a[e], b[e], __ldg(cos_row + i0 + e), __ldg(sin_row + i0 + e), ya[e], yb[e]);
      lo.from_f32(ya);
      hi.from_f32(yb);
    }
    if (is_q) {
      uint16_t* dst = p.q_rot + (static_cast<size_t>(r) * p.Hq + hh) * p.d + i0;
      lo.store(dst);
      hi.store(dst + half);
      continue;
    }
    if (is_k && p.k_rot != nullptr) {
      uint16_t* dst = p.k_rot + (static_cast<size_t>(r) * p.Hk + hh) * p.d + i0;
      lo.store(dst);
      hi.store(dst + half);
    }
    uint16_t* cache = is_k ? p.cache_k : p.cache_v;
    if (cache != nullptr) {
      uint16_t* dst = cache + (static_cast<size_t>(hh) * p.stride + kv_row) * p.d + i0;
      lo.store(dst);
      hi.store(dst + half);
    }
  }
}

int launch(const char* fn, const RopeBf16Params& p) {
  const bool vec = p.d % 16 == 0 && aligned16(p.q) && aligned16(p.k) && aligned16(p.v) &&
                   aligned16(p.q_rot) && aligned16(p.k_rot) && aligned16(p.cache_k) &&
                   aligned16(p.cache_v) && p.pitch_q % 8 == 0 && p.pitch_k % 8 == 0 &&
                   p.pitch_v % 8 == 0;
  cudaStream_t st = current_stream();
  if (vec) rope_bf16_kernel<8><<<static_cast<unsigned>(p.rows), 256, 0, st>>>(p);
  else rope_bf16_kernel<1><<<static_cast<unsigned>(p.rows), 256, 0, st>>>(p);
  G4_LAUNCH_CHECK(fn);
  return 0;
}

bool head_dim_ok(int d) { return d > 0 && (d & 1) == 0 && d <= GRANITE4_MAX_HEAD_DIM; }

}  // namespace

// bf16-cache form of gpu_multi_rope_append (rope_kv.cu forwards bits == 16 here).
int multi_rope_append_bf16(const char* fn, const uint16_t* q, const uint16_t* k, const uint16_t* v,
                           const float* cos_tbl, const float* sin_tbl,
                           const granite4_multi_rows* d_rows, int rows, int Hq, int Hk, int d,
                           uint16_t* cache_k, uint16_t* cache_v, int stride, uint16_t* q_rot) {
  if (q == nullptr || k == nullptr || v == nullptr || cos_tbl == nullptr || sin_tbl == nullptr ||
      cache_k == nullptr || cache_v == nullptr || q_rot == nullptr || Hq <= 0 || Hk <= 0 ||
      stride <= 0 || !head_dim_ok(d))
    return fail(fn, "invalid arguments");
  RopeBf16Params p{};
  p.q = q, p.k = k, p.v = v;
  p.pitch_q = static_cast<long long>(Hq) * d, p.pitch_k = p.pitch_v = static_cast<long long>(Hk) * d;
  p.cos_tbl = cos_tbl, p.sin_tbl = sin_tbl, p.q_rot = q_rot, p.cache_k = cache_k, p.cache_v = cache_v;
  p.table_mode = kTableDescriptor, p.slot_mode = kSlotDescriptor, p.mr = d_rows;
  p.rows = rows, p.Hq = Hq, p.Hk = Hk, p.d = d, p.stride = stride, p.rotate_k = 1;
  return launch(fn, p);
}

// int8 append over a row descriptor (rope_kv.cu).
int multi_kv_append_int8(const char* fn, const uint16_t* k, const uint16_t* v, int8_t* cache_k,
                         int8_t* cache_v, float* k_scale, float* v_scale,
                         const granite4_multi_rows* d_rows, int rows, int stride, int Hk, int d);

}  // namespace g4

extern "C" {

int granite4_kernel_rope_at_pos(const uint16_t* d_x, const float* d_cos, const float* d_sin,
                                int heads, int d, uint16_t* d_out) {
  const char* fn = "granite4_kernel_rope_at_pos";
  if (d_x == nullptr || d_cos == nullptr || d_sin == nullptr || d_out == nullptr || heads <= 0 ||
      !g4::head_dim_ok(d) || static_cast<long long>(heads) * d > INT_MAX)
    return g4::fail(fn, "invalid arguments");
  g4::RopeBf16Params p{};
  p.q = d_x, p.pitch_q = static_cast<long long>(heads) * d, p.q_rot = d_out;
  p.cos_tbl = d_cos, p.sin_tbl = d_sin;  // the caller passes the position's own table row
  p.table_mode = g4::kTableRowIsRow, p.slot_mode = g4::kSlotRun;
  p.rows = 1, p.Hq = heads, p.Hk = 0, p.d = d, p.stride = 1;
  return g4::launch(fn, p);
}

int granite4_kernel_rope_at_pos_batched(const uint16_t* d_x, const float* d_cos,
                                        const float* d_sin, int rows, int heads, int d,
                                        uint16_t* d_out) {
  const char* fn = "granite4_kernel_rope_at_pos_batched";
  if (d_x == nullptr || d_cos == nullptr || d_sin == nullptr || d_out == nullptr || rows <= 0 ||
      rows > GRANITE4_MAX_VERIFY_ROWS || heads <= 0 || !g4::head_dim_ok(d) ||
      static_cast<long long>(rows) * heads * d > INT_MAX)
    return g4::fail(fn, "invalid arguments");
  g4::RopeBf16Params p{};
  p.q = d_x, p.pitch_q = static_cast<long long>(heads) * d, p.q_rot = d_out;
  p.cos_tbl = d_cos, p.sin_tbl = d_sin;  // row r of the tables belongs to row r of x
  p.table_mode = g4::kTableRowIsRow, p.slot_mode = g4::kSlotRun;
  p.rows = rows, p.Hq = heads, p.Hk = 0, p.d = d, p.stride = 1;
  return g4::launch(fn, p);
}

int granite4_kernel_kv_append_batched(const uint16_t* d_src_k, const uint16_t* d_src_v,
                                      uint16_t* d_cache_k, uint16_t* d_cache_v, int base_pos,
                                      int rows, int stride, int Hk, int d, const int* d_pt) {
  const char* fn = "granite4_kernel_kv_append_batched";
  if (d_src_k == nullptr || d_src_v == nullptr || d_cache_k == nullptr || d_cache_v == nullptr ||
      base_pos < 0 || rows <= 0 || rows > GRANITE4_MAX_VERIFY_ROWS || Hk <= 0 || d <= 0 ||
      (d & 1) != 0 || base_pos > INT_MAX - rows || stride < base_pos + rows ||
      static_cast<long long>(Hk) * d > INT_MAX || stride > INT_MAX / (Hk > 1 ? Hk : 1))
    return g4::fail(fn, "invalid arguments");
  g4::RopeBf16Params p{};
  p.k = d_src_k, p.v = d_src_v, p.pitch_k = p.pitch_v = static_cast<long long>(Hk) * d;
  p.cache_k = d_cache_k, p.cache_v = d_cache_v;
  p.table_mode = g4::kTableRowIsRow, p.slot_mode = g4::kSlotRun, p.base_pos = base_pos, p.d_pt = d_pt;
  p.rows = rows, p.Hq = 0, p.Hk = Hk, p.d = d, p.stride = stride, p.rotate_k = 0;
  return g4::launch(fn, p);
}

int granite4_kernel_verify_qkv_stage(const uint16_t* d_q, const uint16_t* d_k, const uint16_t* d_v,
                                     const float* d_cos, const float* d_sin, int base_pos, int rows,
                                     int Hq, int Hk, int d, int cache_stride, uint16_t* d_q_rot,
                                     uint16_t* d_k_rot, uint16_t* d_cache_k, uint16_t* d_cache_v,
                                     const int* d_pt) {
  const char* fn = "granite4_kernel_verify_qkv_stage";
  if (d_q == nullptr || d_k == nullptr || d_v == nullptr || d_cos == nullptr || d_sin == nullptr ||
      d_q_rot == nullptr || d_k_rot == nullptr || d_cache_k == nullptr || d_cache_v == nullptr ||
      base_pos < 0 || rows <= 0 || rows > GRANITE4_MAX_VERIFY_ROWS || Hq <= 0 || Hk <= 0 ||
      Hq < Hk || Hq % Hk != 0 || !g4::head_dim_ok(d) ||
      static_cast<long long>(rows) * Hq * d > INT_MAX || base_pos > INT_MAX - rows + 1 ||
      cache_stride <= base_pos + rows - 1)
    return g4::fail(fn, "invalid arguments");
  g4::RopeBf16Params p{};
  p.q = d_q, p.k = d_k, p.v = d_v;
  p.pitch_q = static_cast<long long>(Hq) * d, p.pitch_k = p.pitch_v = static_cast<long long>(Hk) * d;
  p.cos_tbl = d_cos, p.sin_tbl = d_sin;  // position-specific rows: row r of the tables is row r's
  p.q_rot = d_q_rot, p.k_rot = d_k_rot, p.cache_k = d_cache_k, p.cache_v = d_cache_v;
  p.table_mode = g4::kTableRowIsRow, p.slot_mode = g4::kSlotRun, p.base_pos = base_pos, p.d_pt = d_pt;
  p.rows = rows, p.Hq = Hq, p.Hk = Hk, p.d = d, p.stride = cache_stride, p.rotate_k = 1;
  return g4::launch(fn, p);
}

int granite4_prefill_rope_split_append(const uint16_t* qkv, const float* cos_tbl,
                                       const float* sin_tbl, int base_pos, int rows, int Hq, int Hk,
                                       int d, int stride, uint16_t* q_rot, uint16_t* cache_k,
                                       uint16_t* cache_v, const int* d_pt) {
  const char* fn = "prefill_rope_split_append";
  // engine/src/prefill_gemm.cu:1314-1317 (pointers and head counts are checked too here)
  if (rows <= 0 || rows > 65535 || (d & 1) != 0 || d <= 0 || base_pos < 0 || stride < base_pos + rows)
    return -1;
  if (qkv == nullptr || cos_tbl == nullptr || sin_tbl == nullptr || q_rot == nullptr ||
      cache_k == nullptr || cache_v == nullptr || Hq <= 0 || Hk <= 0)
    return g4::fail(fn, "invalid arguments");
  g4::RopeBf16Params p{};
  const long long pitch = static_cast<long long>(Hq + 2 * Hk) * d;
  p.q = qkv, p.k = qkv + static_cast<size_t>(Hq) * d, p.v = qkv + static_cast<size_t>(Hq + Hk) * d;
  p.pitch_q = p.pitch_k = p.pitch_v = pitch;
  p.cos_tbl = cos_tbl, p.sin_tbl = sin_tbl, p.q_rot = q_rot, p.cache_k = cache_k, p.cache_v = cache_v;
  p.table_mode = g4::kTableRowIsPos, p.slot_mode = g4::kSlotRun, p.base_pos = base_pos, p.d_pt = d_pt;
  p.rows = rows, p.Hq = Hq, p.Hk = Hk, p.d = d, p.stride = stride, p.rotate_k = 1;
  return g4::launch(fn, p);
}

int granite4_gpu_multi_rope(const uint16_t* x, const float* cos_tbl, const float* sin_tbl,
                            const granite4_multi_rows* d_rows, int rows, int heads, int d,
                            uint16_t* out) {
  const char* fn = "gpu_multi_rope";
  // engine/src/forward_gpu.cu:3900-3901
  if (x == nullptr || d_rows == nullptr || rows < 1 || rows > GRANITE4_MAX_VERIFY_ROWS || (d & 1) != 0)
    return -1;
  if (cos_tbl == nullptr || sin_tbl == nullptr || out == nullptr || heads <= 0 || d <= 0)
    return g4::fail(fn, "invalid arguments");
  g4::RopeBf16Params p{};
  p.q = x, p.pitch_q = static_cast<long long>(heads) * d, p.q_rot = out;
  p.cos_tbl = cos_tbl, p.sin_tbl = sin_tbl;
  p.table_mode = g4::kTableDescriptor, p.slot_mode = g4::kSlotDescriptor, p.mr = d_rows;
  p.rows = rows, p.Hq = heads, p.Hk = 0, p.d = d, p.stride = 1;
  return g4::launch(fn, p);
}

int granite4_gpu_multi_kv_append(const uint16_t* k, const uint16_t* v, int bits, void* cache_k,
                                 void* cache_v, float* k_scale, float* v_scale,
                                 const granite4_multi_rows* d_rows, int rows, int stride, int Hk,
                                 int d) {
  const char* fn = "gpu_multi_kv_append";
  if (d_rows == nullptr || rows < 1 || rows > GRANITE4_MAX_VERIFY_ROWS) return -1;  // forward_gpu.cu:3918
  if (k == nullptr || v == nullptr || cache_k == nullptr || cache_v == nullptr || Hk <= 0 || d <= 0 ||
      (d & 1) != 0 || stride <= 0)
    return g4::fail(fn, "invalid arguments");
  if (bits == 8)
    return g4::multi_kv_append_int8(fn, k, v, static_cast<int8_t*>(cache_k),
                                    static_cast<int8_t*>(cache_v), k_scale, v_scale, d_rows, rows,
                                    stride, Hk, d);
  if (bits != 16) return g4::fail(fn, "only the int8 and bf16 cache formats are built (bits 8 or 16)");
  g4::RopeBf16Params p{};
  p.k = k, p.v = v, p.pitch_k = p.pitch_v = static_cast<long long>(Hk) * d;
  p.cache_k = static_cast<uint16_t*>(cache_k), p.cache_v = static_cast<uint16_t*>(cache_v);
  p.table_mode = g4::kTableDescriptor, p.slot_mode = g4::kSlotDescriptor, p.mr = d_rows;
  p.rows = rows, p.Hq = 0, p.Hk = Hk, p.d = d, p.stride = stride, p.rotate_k = 0;
  return g4::launch(fn, p);
}

}  // extern "C"

namespace granite4 {

int prefill_rope_split_append(const std::uint16_t* qkv, const float* cos_tbl, const float* sin_tbl,
                              int base_pos, int rows, int Hq, int Hk, int d, int stride,
                              std::uint16_t* q_rot, std::uint16_t* cache_k, std::uint16_t* cache_v,
                              const int* d_pt) {
  return granite4_prefill_rope_split_append(qkv, cos_tbl, sin_tbl, base_pos, rows, Hq, Hk, d, stride,
                                            q_rot, cache_k, cache_v, d_pt);
}

int gpu_multi_rope(const std::uint16_t* x, const float* cos_tbl, const float* sin_tbl,
                   const GpuMultiRows* d_rows, int rows, int heads, int d, std::uint16_t* out) {
  return granite4_gpu_multi_rope(x, cos_tbl, sin_tbl,
                                 reinterpret_cast<const granite4_multi_rows*>(d_rows), rows, heads, d,
                                 out);
}

int gpu_multi_kv_append(const std::uint16_t* k, const std::uint16_t* v, int bits, void* cache_k,
                        void* cache_v, float* k_scale, float* v_scale, const GpuMultiRows* d_rows,
                        int rows, int stride, int Hk, int d) {
  return granite4_gpu_multi_kv_append(k, v, bits, cache_k, cache_v, k_scale, v_scale,
                                      reinterpret_cast<const granite4_multi_rows*>(d_rows), rows,
                                      stride, Hk, d);
}

}  // namespace granite4
