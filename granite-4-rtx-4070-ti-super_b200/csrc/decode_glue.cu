// The rest of the decode step's glue: greedy pick over the logits with device-
// side token chaining, and the KV row moves that follow an accepted draft path.
//
// Greedy pick (reference: engine/src/forward_gpu.cu:280-333 argmax_rows_kernel,
// engine/src/eagle_gpu.cu:155-178 argmax_map_kernel; host rule
// engine/src/kernel_math.h:592-601): the first index of the row maximum of bf16
// logits [rows][V]; NaN never wins; a row with nothing above -inf gives 0. With
// d_pos (one row) the id goes to out[*d_pos + 1] and *d_pos advances, which
// chains captured decode steps; with a vocabulary map the id is map[index].
//
// This is a pure read: 2 V bytes per row (200 704 at V = 100352). Each thread
// streams its 128-bit chunks through a packed bf16 max (one instruction per two
// logits) and only the threads whose maximum equals the row's go back for the
// index, so the sweep is a load loop. Large batches take one CTA per row; a
// decode or verify step (<= 16 rows) cuts each row over the CTAs of a thread-
// block cluster, which combine (max, index) through distributed shared memory,
// so that a single row is read by several SMs at once.
//
// Token chaining (engine/src/forward_gpu.cu:758-764) and KV moves
// (engine/src/forward_gpu.cu:3473-3536) are tiny; the move handles every layer
// in one launch where the reference launches once per layer.
#include "g4_cluster.cuh"
#include "g4_host.h"
#include "g4_math.cuh"

#include "../../include/granite4_b200.h"

#include <cuda_bf16.h>

namespace g4 {
namespace {

constexpr int kArgmaxThreads = 1024;
constexpr int kArgmaxUnroll = 4;

struct ArgmaxParams {
  const uint16_t* logits;
  int32_t* out;
  int* d_pos;
  const int32_t* map;
  granite4_multi_rows* advance;  // non-NULL: the pick also becomes the row's next token and its position advances
  int V;
  int rows;
  int ctas_per_row;
};

__device__ __forceinline__ uint32_t bf16x2_max(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));  // a NaN operand loses
  return d;
}
__device__ __forceinline__ float pair_max(uint32_t m) {
  return fmaxf(__uint_as_float(m << 16), __uint_as_float(m & 0xffff0000u));
}

// VEC: V % 8 == 0 and 16-byte aligned rows. CLUSTER: the grid is cut into clusters of
// ctas_per_row CTAs, one cluster per row.
template <bool VEC, bool CLUSTER>
__global__ void __launch_bounds__(kArgmaxThreads) argmax_rows_kernel(const ArgmaxParams p) {
  pdl_begin();
  if (CLUSTER) cluster_announce();
  const int T = blockDim.x, t = threadIdx.x, lane = t & 31, warp = t >> 5, nwarps = T >> 5;
  const int C = CLUSTER ? p.ctas_per_row : 1;
  const int row = CLUSTER ? static_cast<int>(blockIdx.x) / C : blockIdx.x;
  const int part = CLUSTER ? static_cast<int>(blockIdx.x) % C : 0;
  const uint16_t* x = p.logits + static_cast<size_t>(row) * p.V;
  // this CTA's slice, in units (chunks of 8 when VEC, else elements)
  const int units = VEC ? p.V / 8 : p.V;
  const int per = (units + C - 1) / C;
  const int u0 = min(part * per, units), u1 = min(u0 + per, units);

  // ---- sweep 1: the maximum ----------------------------------------------------------
  float tmax = -INFINITY;
  if (VEC) {
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    uint32_t m = 0xff80ff80u;  // (-inf, -inf)
    int u = u0 + t;
    for (; u + (kArgmaxUnroll - 1) * T < u1; u += kArgmaxUnroll * T) {
      uint4 v[kArgmaxUnroll];
#pragma unroll
      for (int k = 0; k < kArgmaxUnroll; ++k) v[k] = ld_stream(xv + u + k * T);
#pragma unroll
      for (int k = 0; k < kArgmaxUnroll; ++k)
        m = bf16x2_max(bf16x2_max(m, bf16x2_max(v[k].x, v[k].y)), bf16x2_max(v[k].z, v[k].w));
    }
    for (; u < u1; u += T) {
      const uint4 v = ld_stream(xv + u);
      m = bf16x2_max(bf16x2_max(m, bf16x2_max(v.x, v.y)), bf16x2_max(v.z, v.w));
    }
    tmax = pair_max(m);
  } else {
    for (int u = u0 + t; u < u1; u += T) tmax = fmaxf(tmax, bf16_to_f32(x[u]));  // fmaxf drops NaN
  }
  __shared__ float s_max[32];
  __shared__ int s_idx[32];
  float wmax = tmax;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wmax = fmaxf(wmax, __shfl_xor_sync(0xffffffffu, wmax, o));
  if (lane == 0) s_max[warp] = wmax;
  __syncthreads();
  float M = -INFINITY;
  for (int i = 0; i < nwarps; ++i) M = fmaxf(M, s_max[i]);

  // ---- sweep 2: the first index that holds it (few threads; their data is cache-hot) -----
  int idx = INT_MAX;
  if (tmax == M && M > -INFINITY) {
    if (VEC) {
      const uint4* xv = reinterpret_cast<const uint4*>(x);
      for (int u = u0 + t; u < u1 && idx == INT_MAX; u += T) {
        float f[8];
        unpack8(__ldg(xv + u), f);
#pragma unroll
        for (int e = 7; e >= 0; --e)
          if (f[e] == M) idx = u * 8 + e;  // descending e: the lowest match stays
      }
    } else {
      for (int u = u0 + t; u < u1; u += T)
        if (bf16_to_f32(x[u]) == M) {
          idx = u;
          break;
        }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) idx = min(idx, __shfl_xor_sync(0xffffffffu, idx, o));
  if (lane == 0) s_idx[warp] = idx;
  __syncthreads();
  if (CLUSTER) cluster_all_started();  // before the stores into CTA 0's shared memory below
  __shared__ float s_cmax[kMaxClusterCtas];
  __shared__ int s_cidx[kMaxClusterCtas];
  if (t == 0) {
    int best = INT_MAX;
    for (int i = 0; i < nwarps; ++i) best = min(best, s_idx[i]);
    if (CLUSTER) {
      namespace cg = cooperative_groups;
      cg::cluster_group cluster = cg::this_cluster();
      *cluster.map_shared_rank(s_cmax + part, 0) = M;
      *cluster.map_shared_rank(s_cidx + part, 0) = best;
    } else {
      s_cmax[0] = M, s_cidx[0] = best;
    }
  }
  if (CLUSTER) cooperative_groups::this_cluster().sync();  // every thread of every CTA, once
  if (part == 0 && t == 0) {
    float bm = s_cmax[0];
    int bi = s_cidx[0];
    for (int c = 1; c < C; ++c)
      if (s_cmax[c] > bm || (s_cmax[c] == bm && s_cidx[c] < bi)) bm = s_cmax[c], bi = s_cidx[c];
    int best = (bi == INT_MAX || !(bm > -INFINITY)) ? 0 : bi;
    if (p.map != nullptr) best = p.map[best];
    if (p.advance != nullptr) {
      // multi_scatter_advance_kernel of the reference (engine/src/forward_gpu.cu:758-764), folded in
      const int pos = p.advance->pos[row];
      p.advance->tok[row][pos + 1] = best;
      p.advance->pos[row] = pos + 1;
      if (p.out != nullptr) p.out[row] = best;
    } else if (p.d_pos != nullptr) {
      const int pos = *p.d_pos;
      p.out[pos + 1] = best;
      *p.d_pos = pos + 1;
    } else {
      p.out[row] = best;
    }
  }
}

// Row r's greedy id becomes its session's next token; positions advance
// (engine/src/forward_gpu.cu:758-764).
__global__ void multi_scatter_advance_kernel(granite4_multi_rows* mr, const int32_t* ids) {
  const int r = threadIdx.x;
  if (r >= mr->n || r >= GRANITE4_MAX_VERIFY_ROWS) return;
  const int pos = mr->pos[r];
  mr->tok[r][pos + 1] = ids[r];
  mr->pos[r] = pos + 1;
}

// Embedding rows of a multi-session step: row r takes the token its session holds at the row's slot
// (engine/src/forward_gpu.cu:359-378, embed_multi_v8_kernel): out[r] = bf16(mult * emb[tok[r][slot]]),
// slot = pos[r], or slot[r] for tree rows. One CTA per row, 128-bit accesses.
__global__ void __launch_bounds__(256) multi_embed_kernel(const granite4_multi_rows* mr, const uint4* emb,
                                                         int vocab, float mult, uint4* out, int H8) {
  pdl_begin();
  const int r = blockIdx.x;
  const int slot = mr->tree ? mr->slot[r] : mr->pos[r];
  const int tok = mr->tok[r][slot];
  const bool known = tok >= 0 && tok < vocab;  // an id outside the table gives a zero row
  for (int c = threadIdx.x; c < H8; c += blockDim.x) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (known) {
      float f[8];
      unpack8(__ldg(emb + static_cast<size_t>(tok) * H8 + c), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __fmul_rn(mult, f[e]);
      v = pack8(f);
    }
    out[static_cast<size_t>(r) * H8 + c] = v;
  }
}

struct KvMoveParams {
  int n;
  int src[GRANITE4_MAX_TREE_DEPTH], dst[GRANITE4_MAX_TREE_DEPTH];  // physical pool rows
  uint8_t* k;
  uint8_t* v;
  float* ks;
  float* vs;
  int row_bytes;  // d for int8 codes, 2 d for bf16
  long long stride;
  int Hk;
};

// One CTA per (kv head, layer); the moves run in order, as the reference's do: a later move may
// read a row an earlier one wrote.
__global__ void __launch_bounds__(128) kv_move_kernel(const KvMoveParams p) {
  const size_t head = static_cast<size_t>(blockIdx.y) * p.Hk + blockIdx.x;  // [layer][hkv]
  const int words = p.row_bytes / 4;
  for (int i = 0; i < p.n; ++i) {
    const size_t so = head * p.stride + p.src[i], dd = head * p.stride + p.dst[i];
    const uint32_t* ksrc = reinterpret_cast<const uint32_t*>(p.k + so * p.row_bytes);
    const uint32_t* vsrc = reinterpret_cast<const uint32_t*>(p.v + so * p.row_bytes);
    uint32_t* kdst = reinterpret_cast<uint32_t*>(p.k + dd * p.row_bytes);
    uint32_t* vdst = reinterpret_cast<uint32_t*>(p.v + dd * p.row_bytes);
    for (int w = threadIdx.x; w < words; w += blockDim.x) kdst[w] = ksrc[w], vdst[w] = vsrc[w];
    if (p.ks != nullptr && threadIdx.x == 0) p.ks[dd] = p.ks[so], p.vs[dd] = p.vs[so];
    __syncthreads();
  }
}

}  // namespace
}  // namespace g4

extern "C" {

}  // extern "C"

namespace g4 {
namespace {
int launch_argmax(const char* fn, ArgmaxParams p) {
  p.ctas_per_row = 1;
  cudaStream_t st = current_stream();
  const bool vec = p.V % 8 == 0 && aligned16(p.logits);
  // A step of at most 16 rows: several CTAs per row, as one cluster per row.
  if (vec && p.rows <= GRANITE4_MAX_VERIFY_ROWS && p.V >= 8 * 1024 && cluster_enabled()) {
    p.ctas_per_row = 8;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(p.rows * p.ctas_per_row));
    cfg.blockDim = dim3(512);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(p.ctas_per_row);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    void (*kernel)(ArgmaxParams) = argmax_rows_kernel<true, true>;
    if (cluster_fits(reinterpret_cast<const void*>(kernel), cfg, p.ctas_per_row, 512)) {
      cfg.numAttrs = pdl_enabled() ? 2 : 1;
      G4_CUDA_TRY(fn, cudaLaunchKernelEx(&cfg, kernel, p));
      return 0;
    }
    p.ctas_per_row = 1;
  }
  const dim3 grid(static_cast<unsigned>(p.rows)), block(kArgmaxThreads);
  if (vec) G4_LAUNCH_PDL(fn, argmax_rows_kernel<true, false>, grid, block, 0, st, p);
  else G4_LAUNCH_PDL(fn, argmax_rows_kernel<false, false>, grid, block, 0, st, p);
  return 0;
}
}  // namespace
}  // namespace g4

extern "C" {

int granite4_kernel_argmax_rows(const uint16_t* d_logits, int rows, int V, int32_t* d_out,
                                int* d_pos, const int32_t* d_vocab_map) {
  const char* fn = "granite4_kernel_argmax_rows";
  if (d_logits == nullptr || d_out == nullptr || rows <= 0 || V <= 0 ||
      (d_pos != nullptr && rows != 1))
    return g4::fail(fn, "invalid arguments");
  g4::ArgmaxParams p{};
  p.logits = d_logits, p.out = d_out, p.d_pos = d_pos, p.map = d_vocab_map, p.V = V, p.rows = rows;
  return g4::launch_argmax(fn, p);
}

int granite4_kernel_argmax_advance(const uint16_t* d_logits, int rows, int V, granite4_multi_rows* d_rows,
                                   int32_t* d_ids_out) {
  const char* fn = "granite4_kernel_argmax_advance";
  if (d_logits == nullptr || d_rows == nullptr || rows <= 0 || rows > GRANITE4_MAX_VERIFY_ROWS || V <= 0)
    return g4::fail(fn, "invalid arguments");
  g4::ArgmaxParams p{};
  p.logits = d_logits, p.out = d_ids_out, p.advance = d_rows, p.V = V, p.rows = rows;
  return g4::launch_argmax(fn, p);
}

int granite4_kernel_multi_scatter_advance(granite4_multi_rows* d_rows, const int32_t* d_ids) {
  const char* fn = "granite4_kernel_multi_scatter_advance";
  if (d_rows == nullptr || d_ids == nullptr) return g4::fail(fn, "invalid arguments");
  g4::multi_scatter_advance_kernel<<<1, 32, 0, g4::current_stream()>>>(d_rows, d_ids);
  G4_LAUNCH_CHECK(fn);
  return 0;
}

int granite4_gpu_multi_embed(const granite4_multi_rows* d_rows, int rows, const uint16_t* d_emb, int vocab,
                             float mult, uint16_t* d_out, int H) {
  const char* fn = "granite4_gpu_multi_embed";
  if (d_rows == nullptr || d_emb == nullptr || d_out == nullptr || rows < 1 || rows > GRANITE4_MAX_VERIFY_ROWS ||
      vocab <= 0 || H <= 0 || H % 8 != 0 || !std::isfinite(mult) || !g4::aligned16(d_emb) || !g4::aligned16(d_out))
    return g4::fail(fn, "invalid arguments");
  G4_LAUNCH_PDL(fn, g4::multi_embed_kernel, dim3(static_cast<unsigned>(rows)), dim3(256), 0, g4::current_stream(),
                d_rows, reinterpret_cast<const uint4*>(d_emb), vocab, mult, reinterpret_cast<uint4*>(d_out), H / 8);
  return 0;
}

int granite4_kernel_kv_move(const int* src_rows, const int* dst_rows, int n, int bits, void* d_cache_k,
                            void* d_cache_v, float* d_k_scale, float* d_v_scale, int layers, int Hk,
                            int stride, int d) {
  const char* fn = "granite4_kernel_kv_move";
  if (n < 0 || n > GRANITE4_MAX_TREE_DEPTH || src_rows == nullptr || dst_rows == nullptr) return -1;
  if (n == 0) return 0;
  if (d_cache_k == nullptr || d_cache_v == nullptr || layers <= 0 || Hk <= 0 || stride <= 0 ||
      d <= 0 || (bits != 8 && bits != 16) || (bits == 8 && (d_k_scale == nullptr || d_v_scale == nullptr)))
    return g4::fail(fn, "invalid arguments (bits must be 8 or 16)");
  g4::KvMoveParams p{};
  p.n = n;
  for (int i = 0; i < n; ++i) {
    // engine/src/forward_gpu.cu:3514-3519: rows in range, never moved to a later row, and no
    // later move reads what an earlier one overwrote
    if (src_rows[i] < 0 || dst_rows[i] < 0 || src_rows[i] >= stride || dst_rows[i] >= stride)
      return g4::fail(fn, "row outside the pool");
    for (int j = i + 1; j < n; ++j)
      if (src_rows[j] == dst_rows[i]) return g4::fail(fn, "a later move reads a row an earlier one overwrites");
    p.src[i] = src_rows[i], p.dst[i] = dst_rows[i];
  }
  p.k = static_cast<uint8_t*>(d_cache_k), p.v = static_cast<uint8_t*>(d_cache_v);
  p.ks = bits == 8 ? d_k_scale : nullptr, p.vs = bits == 8 ? d_v_scale : nullptr;
  p.row_bytes = bits == 16 ? 2 * d : d;
  if (p.row_bytes % 4 != 0 || (reinterpret_cast<uintptr_t>(d_cache_k) & 3u) != 0 ||
      (reinterpret_cast<uintptr_t>(d_cache_v) & 3u) != 0)
    return g4::fail(fn, "rows must be whole 4-byte words");
  p.stride = stride, p.Hk = Hk;
  g4::kv_move_kernel<<<dim3(static_cast<unsigned>(Hk), static_cast<unsigned>(layers)), 128, 0,
                       g4::current_stream()>>>(p);
  G4_LAUNCH_CHECK(fn);
  return 0;
}

}  // extern "C"
