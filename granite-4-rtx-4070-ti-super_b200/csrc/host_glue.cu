// Host side of the layer glue: one call per layer over device buffers, and the
// same layer over HOST buffers with the transfers pipelined.
//
// The reference's forward pass issues the glue launches one by one between its
// GEMMs (engine/src/forward_gpu.cu:2786-2845) with activations that never leave
// the device. granite4_glue_layer is that call sequence for the glue alone.
// granite4_host_glue_* is for callers that hold activations in host memory: it
// stages them through device buffers it owns. The PCIe link, not the kernels,
// bounds that path (87 KB go in and 37 KB come out per token and layer at
// Granite sizes), so the design goal is only to keep both directions of the
// link busy: three streams (in, compute, out), two staging sets, events
// between them, no host synchronisation except when a third call would reuse
// a set that is still in flight.
#include "g4_host.h"

#include "../../include/granite4_b200.h"

#include <new>

extern "C" int granite4_glue_layer(const granite4_glue_layer_args* a) {
  const char* fn = "granite4_glue_layer";
  if (a == nullptr) return g4::fail(fn, "invalid arguments");
  float* sc = a->scales;
  if (sc == nullptr) return g4::fail(fn, "scales buffer missing");
  // One memset clears the {scale, amax} slots of all three FP8 ops, so that the seven kernels of
  // the layer follow one another on the stream with no other operation between them (each is
  // staged while its predecessor drains, g4_host.h launch_pdl).
  G4_CUDA_TRY(fn, cudaMemsetAsync(sc, 0, 6 * sizeof(float), g4::current_stream()));
  struct Prezeroed {
    Prezeroed() { g4::set_amax_prezeroed(true); }
    ~Prezeroed() { g4::set_amax_prezeroed(false); }
  } prezeroed;
  if (granite4_kernel_add_rmsnorm_fp8(a->y_attn, 0, a->hidden, 0, a->w_attn_norm, a->eps, a->resid_mult,
                                      a->rows, a->hidden_size, a->hidden, nullptr, a->n_attn_fp8, sc,
                                      a->rstd) != 0)
    return -1;
  if (granite4_kernel_rope_kv_int8_paged(a->qkv, a->cos_tbl, a->sin_tbl, a->pos_rows, a->kv_rows, a->rows,
                                         a->q_heads, a->kv_heads, a->head_dim, a->pool_rows, a->max_pos,
                                         0, a->q_rot, a->cache_k, a->cache_v, a->k_scale,
                                         a->v_scale) != 0)
    return -1;
  if (granite4_kernel_add_rmsnorm_fp8(a->y_mlp, 0, a->hidden, 0, a->w_mlp_norm, a->eps, a->resid_mult,
                                      a->rows, a->hidden_size, a->hidden, nullptr, a->n_mlp_fp8, sc + 2,
                                      a->rstd) != 0)
    return -1;
  if (granite4_kernel_swiglu_fp8(a->gate, a->up, 0, a->intermediate, a->rows, a->intermediate, a->act_ws,
                                 a->act_fp8, sc + 4) != 0)
    return -1;
  return 0;
}

// ------------------------------------------------------------------------------------------------

namespace {

struct StagingSet {
  // inputs
  uint16_t *y_attn, *y_mlp, *qkv, *gate, *up, *w_attn, *w_mlp;
  int *pos_rows, *kv_rows;
  // outputs
  uint8_t *n_attn, *n_mlp, *act;
  uint16_t* q_rot;
  float* scales;
  // scratch
  float* rstd;
  uint16_t* act_ws;
  cudaEvent_t in_done, compute_done, out_done;
  bool busy;
};

}  // namespace

struct granite4_host_glue {
  int max_rows, hidden, inter, q_heads, kv_heads, head_dim, layers, pool_rows, max_pos;
  int device;
  StagingSet set[2];
  int next;  // set the next call uses
  int8_t *cache_k, *cache_v;  // [layers][kv_heads][pool_rows][head_dim]
  float *k_scale, *v_scale;   // [layers][kv_heads][pool_rows]
  float *cos_tbl, *sin_tbl;
  // The residual stream stays on the device between layer calls (context state, like the KV
  // pool); a call uploads it only when it is given hidden_in and reads it back only when it
  // is given hidden_out.
  uint16_t* resid;              // [max_rows][hidden]
  cudaEvent_t hidden_read_back;  // the last read-back of `resid` has finished
  bool hidden_read_pending;
  cudaEvent_t last_compute;      // the last layer enqueued on s_compute has finished
  bool any_compute;
  cudaStream_t s_in, s_compute, s_out;
};

namespace {

template <typename T>
bool dev_alloc(T** p, size_t count) {
  *p = nullptr;
  return cudaMalloc(reinterpret_cast<void**>(p), count * sizeof(T)) == cudaSuccess;
}

void free_set(StagingSet& s) {
  void* ptrs[] = {s.y_attn, s.y_mlp, s.qkv, s.gate, s.up, s.w_attn, s.w_mlp, s.pos_rows,
                  s.kv_rows, s.n_attn, s.n_mlp, s.act, s.q_rot, s.scales, s.rstd, s.act_ws};
  for (void* p : ptrs)
    if (p != nullptr) cudaFree(p);
  if (s.in_done) cudaEventDestroy(s.in_done);
  if (s.compute_done) cudaEventDestroy(s.compute_done);
  if (s.out_done) cudaEventDestroy(s.out_done);
}

bool alloc_set(StagingSet& s, const granite4_host_glue& c) {
  const size_t R = c.max_rows, H = c.hidden, I = c.inter;
  const size_t QKV = static_cast<size_t>(c.q_heads + 2 * c.kv_heads) * c.head_dim;
  const size_t Q = static_cast<size_t>(c.q_heads) * c.head_dim;
  bool ok = dev_alloc(&s.y_attn, R * H) && dev_alloc(&s.y_mlp, R * H) && dev_alloc(&s.qkv, R * QKV) &&
            dev_alloc(&s.gate, R * I) && dev_alloc(&s.up, R * I) &&
            dev_alloc(&s.w_attn, H) && dev_alloc(&s.w_mlp, H) && dev_alloc(&s.pos_rows, R) &&
            dev_alloc(&s.kv_rows, R) && dev_alloc(&s.n_attn, R * H) && dev_alloc(&s.n_mlp, R * H) &&
            dev_alloc(&s.act, R * I) && dev_alloc(&s.q_rot, R * Q) && dev_alloc(&s.scales, 6) &&
            dev_alloc(&s.rstd, R) && dev_alloc(&s.act_ws, R * I);
  ok = ok && cudaEventCreateWithFlags(&s.in_done, cudaEventDisableTiming) == cudaSuccess &&
       cudaEventCreateWithFlags(&s.compute_done, cudaEventDisableTiming) == cudaSuccess &&
       cudaEventCreateWithFlags(&s.out_done, cudaEventDisableTiming) == cudaSuccess;
  s.busy = false;
  return ok;
}

}  // namespace

extern "C" {

void granite4_host_glue_destroy(granite4_host_glue* c) {
  if (c == nullptr) return;
  cudaSetDevice(c->device);
  if (c->s_in) cudaStreamSynchronize(c->s_in);
  if (c->s_compute) cudaStreamSynchronize(c->s_compute);
  if (c->s_out) cudaStreamSynchronize(c->s_out);
  free_set(c->set[0]);
  free_set(c->set[1]);
  void* ptrs[] = {c->cache_k, c->cache_v, c->k_scale, c->v_scale, c->cos_tbl, c->sin_tbl, c->resid};
  for (void* p : ptrs)
    if (p != nullptr) cudaFree(p);
  if (c->hidden_read_back) cudaEventDestroy(c->hidden_read_back);
  if (c->last_compute) cudaEventDestroy(c->last_compute);
  if (c->s_in) cudaStreamDestroy(c->s_in);
  if (c->s_compute) cudaStreamDestroy(c->s_compute);
  if (c->s_out) cudaStreamDestroy(c->s_out);
  delete c;
}

granite4_host_glue* granite4_host_glue_create(int max_rows, int hidden_size, int intermediate,
                                              int q_heads, int kv_heads, int head_dim, int layers,
                                              int pool_rows, int max_pos, double rope_theta) {
  const char* fn = "granite4_host_glue_create";
  if (max_rows <= 0 || hidden_size <= 0 || hidden_size % 8 != 0 || intermediate <= 0 ||
      intermediate % 8 != 0 || q_heads <= 0 || kv_heads <= 0 || head_dim != 128 || layers <= 0 ||
      pool_rows <= 0 || max_pos <= 0) {
    g4::fail(fn, "invalid arguments");
    return nullptr;
  }
  granite4_host_glue* c = new (std::nothrow) granite4_host_glue();
  if (c == nullptr) return nullptr;
  *c = granite4_host_glue{};
  c->max_rows = max_rows, c->hidden = hidden_size, c->inter = intermediate, c->q_heads = q_heads;
  c->kv_heads = kv_heads, c->head_dim = head_dim, c->layers = layers, c->pool_rows = pool_rows;
  c->max_pos = max_pos;
  bool ok = cudaGetDevice(&c->device) == cudaSuccess;
  const size_t pool = static_cast<size_t>(layers) * kv_heads * pool_rows;
  ok = ok && alloc_set(c->set[0], *c) && alloc_set(c->set[1], *c) &&
       dev_alloc(&c->cache_k, pool * head_dim) && dev_alloc(&c->cache_v, pool * head_dim) &&
       dev_alloc(&c->k_scale, pool) && dev_alloc(&c->v_scale, pool) &&
       dev_alloc(&c->resid, static_cast<size_t>(max_rows) * hidden_size) &&
       cudaMemset(c->resid, 0, static_cast<size_t>(max_rows) * hidden_size * 2) == cudaSuccess &&
       cudaEventCreateWithFlags(&c->hidden_read_back, cudaEventDisableTiming) == cudaSuccess &&
       cudaEventCreateWithFlags(&c->last_compute, cudaEventDisableTiming) == cudaSuccess;
  ok = ok && cudaMemset(c->cache_k, 0, pool * head_dim) == cudaSuccess &&
       cudaMemset(c->cache_v, 0, pool * head_dim) == cudaSuccess &&
       cudaMemset(c->k_scale, 0, pool * sizeof(float)) == cudaSuccess &&
       cudaMemset(c->v_scale, 0, pool * sizeof(float)) == cudaSuccess;
  ok = ok && granite4_rope_tables_build(rope_theta, head_dim, max_pos, &c->cos_tbl, &c->sin_tbl) == 0;
  ok = ok && cudaStreamCreateWithFlags(&c->s_in, cudaStreamNonBlocking) == cudaSuccess &&
       cudaStreamCreateWithFlags(&c->s_compute, cudaStreamNonBlocking) == cudaSuccess &&
       cudaStreamCreateWithFlags(&c->s_out, cudaStreamNonBlocking) == cudaSuccess;
  if (!ok) {
    g4::fail(fn, "allocation failed");
    granite4_host_glue_destroy(c);
    return nullptr;
  }
  return c;
}

long long granite4_host_glue_h2d_bytes(const granite4_host_glue* c, int rows) {
  if (c == nullptr) return 0;
  const long long qkv = static_cast<long long>(c->q_heads + 2 * c->kv_heads) * c->head_dim;
  // without the optional upload of the residual stream (2 * hidden bytes per row more)
  return static_cast<long long>(rows) * (2LL * (2LL * c->hidden + qkv + 2LL * c->inter) + 8) +
         4LL * c->hidden;
}
long long granite4_host_glue_d2h_bytes(const granite4_host_glue* c, int rows) {
  if (c == nullptr) return 0;
  const long long q = static_cast<long long>(c->q_heads) * c->head_dim;
  // without the optional read-back of the residual stream (2 * hidden bytes per row more)
  return static_cast<long long>(rows) * (2LL * c->hidden + 2LL * q + c->inter) + 24;
}

int granite4_host_glue_layer(granite4_host_glue* c, int layer, const granite4_host_layer_io* io) {
  const char* fn = "granite4_host_glue_layer";
  if (c == nullptr || io == nullptr || layer < 0 || layer >= c->layers || io->rows <= 0 ||
      io->rows > c->max_rows)
    return g4::fail(fn, "invalid arguments");
  if (io->y_attn == nullptr || io->y_mlp == nullptr || io->qkv == nullptr || io->gate == nullptr ||
      io->up == nullptr || io->w_attn_norm == nullptr || io->w_mlp_norm == nullptr ||
      io->pos_rows == nullptr || io->kv_rows == nullptr || io->n_attn_fp8 == nullptr ||
      io->n_mlp_fp8 == nullptr ||
      io->q_rot == nullptr || io->act_fp8 == nullptr || io->scales == nullptr)
    return g4::fail(fn, "NULL host buffer");
  G4_CUDA_TRY(fn, cudaSetDevice(c->device));
  StagingSet& s = c->set[c->next];
  c->next ^= 1;
  if (s.busy) G4_CUDA_TRY(fn, cudaEventSynchronize(s.out_done));  // its previous outputs have left
  s.busy = true;
  const size_t R = io->rows, H = c->hidden, I = c->inter;
  const size_t QKV = static_cast<size_t>(c->q_heads + 2 * c->kv_heads) * c->head_dim;
  const size_t Q = static_cast<size_t>(c->q_heads) * c->head_dim;
  auto h2d = [&](void* d, const void* h, size_t bytes) {
    return cudaMemcpyAsync(d, h, bytes, cudaMemcpyHostToDevice, c->s_in);
  };
  G4_CUDA_TRY(fn, h2d(s.y_attn, io->y_attn, R * H * 2));
  if (io->hidden_in != nullptr) {
    // overwrite the resident residual stream: not before the layer that still uses it is done
    if (c->any_compute) G4_CUDA_TRY(fn, cudaStreamWaitEvent(c->s_in, c->last_compute, 0));
    if (c->hidden_read_pending) G4_CUDA_TRY(fn, cudaStreamWaitEvent(c->s_in, c->hidden_read_back, 0));
    G4_CUDA_TRY(fn, h2d(c->resid, io->hidden_in, R * H * 2));
  }
  G4_CUDA_TRY(fn, h2d(s.w_attn, io->w_attn_norm, H * 2));
  G4_CUDA_TRY(fn, h2d(s.w_mlp, io->w_mlp_norm, H * 2));
  G4_CUDA_TRY(fn, h2d(s.pos_rows, io->pos_rows, R * 4));
  G4_CUDA_TRY(fn, h2d(s.kv_rows, io->kv_rows, R * 4));
  G4_CUDA_TRY(fn, h2d(s.qkv, io->qkv, R * QKV * 2));
  G4_CUDA_TRY(fn, h2d(s.y_mlp, io->y_mlp, R * H * 2));
  G4_CUDA_TRY(fn, h2d(s.gate, io->gate, R * I * 2));
  G4_CUDA_TRY(fn, h2d(s.up, io->up, R * I * 2));
  G4_CUDA_TRY(fn, cudaEventRecord(s.in_done, c->s_in));

  G4_CUDA_TRY(fn, cudaStreamWaitEvent(c->s_compute, s.in_done, 0));
  if (c->hidden_read_pending) {  // the previous read-back of the residual stream must finish first
    G4_CUDA_TRY(fn, cudaStreamWaitEvent(c->s_compute, c->hidden_read_back, 0));
    c->hidden_read_pending = false;
  }
  const size_t pool_off = static_cast<size_t>(layer) * c->kv_heads * c->pool_rows;
  granite4_glue_layer_args a{};
  a.y_attn = s.y_attn, a.y_mlp = s.y_mlp, a.qkv = s.qkv, a.gate = s.gate, a.up = s.up;
  a.w_attn_norm = s.w_attn, a.w_mlp_norm = s.w_mlp, a.cos_tbl = c->cos_tbl, a.sin_tbl = c->sin_tbl;
  a.pos_rows = s.pos_rows, a.kv_rows = s.kv_rows, a.hidden = c->resid;
  a.n_attn_fp8 = s.n_attn, a.n_mlp_fp8 = s.n_mlp, a.q_rot = s.q_rot;
  a.cache_k = c->cache_k + pool_off * c->head_dim, a.cache_v = c->cache_v + pool_off * c->head_dim;
  a.k_scale = c->k_scale + pool_off, a.v_scale = c->v_scale + pool_off;
  a.act_fp8 = s.act, a.scales = s.scales, a.rstd = s.rstd, a.act_ws = s.act_ws;
  a.rows = io->rows, a.hidden_size = c->hidden, a.intermediate = c->inter, a.q_heads = c->q_heads;
  a.kv_heads = c->kv_heads, a.head_dim = c->head_dim, a.pool_rows = c->pool_rows, a.max_pos = c->max_pos;
  a.eps = io->eps, a.resid_mult = io->resid_mult;
  cudaStream_t prev = g4::current_stream();
  g4::set_current_stream(c->s_compute);
  const int rc = granite4_glue_layer(&a);
  g4::set_current_stream(prev == cudaStreamPerThread ? nullptr : prev);
  if (rc != 0) return -1;
  G4_CUDA_TRY(fn, cudaEventRecord(s.compute_done, c->s_compute));
  G4_CUDA_TRY(fn, cudaEventRecord(c->last_compute, c->s_compute));
  c->any_compute = true;

  G4_CUDA_TRY(fn, cudaStreamWaitEvent(c->s_out, s.compute_done, 0));
  auto d2h = [&](void* h, const void* d, size_t bytes) {
    return cudaMemcpyAsync(h, d, bytes, cudaMemcpyDeviceToHost, c->s_out);
  };
  if (io->hidden_out != nullptr) {
    G4_CUDA_TRY(fn, d2h(io->hidden_out, c->resid, R * H * 2));
    G4_CUDA_TRY(fn, cudaEventRecord(c->hidden_read_back, c->s_out));
    c->hidden_read_pending = true;
  }
  G4_CUDA_TRY(fn, d2h(io->n_attn_fp8, s.n_attn, R * H));
  G4_CUDA_TRY(fn, d2h(io->n_mlp_fp8, s.n_mlp, R * H));
  G4_CUDA_TRY(fn, d2h(io->q_rot, s.q_rot, R * Q * 2));
  G4_CUDA_TRY(fn, d2h(io->act_fp8, s.act, R * I));
  G4_CUDA_TRY(fn, d2h(io->scales, s.scales, 6 * sizeof(float)));
  G4_CUDA_TRY(fn, cudaEventRecord(s.out_done, c->s_out));
  return 0;
}

int granite4_host_glue_final_norm(granite4_host_glue* c, const uint16_t* h_w, float eps, int rows,
                                  uint16_t* h_out) {
  const char* fn = "granite4_host_glue_final_norm";
  if (c == nullptr || h_w == nullptr || h_out == nullptr || rows <= 0 || rows > c->max_rows)
    return g4::fail(fn, "invalid arguments");
  G4_CUDA_TRY(fn, cudaSetDevice(c->device));
  StagingSet& s = c->set[c->next];
  c->next ^= 1;
  if (s.busy) G4_CUDA_TRY(fn, cudaEventSynchronize(s.out_done));
  s.busy = true;
  const size_t H = c->hidden;
  G4_CUDA_TRY(fn, cudaMemcpyAsync(s.w_attn, h_w, H * 2, cudaMemcpyHostToDevice, c->s_in));
  G4_CUDA_TRY(fn, cudaEventRecord(s.in_done, c->s_in));
  G4_CUDA_TRY(fn, cudaStreamWaitEvent(c->s_compute, s.in_done, 0));
  cudaStream_t prev = g4::current_stream();
  g4::set_current_stream(c->s_compute);
  // the staging set's y_attn buffer receives the normed rows
  const int rc = granite4_kernel_rmsnorm(c->resid, s.w_attn, eps, rows, c->hidden, s.y_attn);
  g4::set_current_stream(prev == cudaStreamPerThread ? nullptr : prev);
  if (rc != 0) return -1;
  G4_CUDA_TRY(fn, cudaEventRecord(s.compute_done, c->s_compute));
  G4_CUDA_TRY(fn, cudaEventRecord(c->last_compute, c->s_compute));
  c->any_compute = true;
  G4_CUDA_TRY(fn, cudaStreamWaitEvent(c->s_out, s.compute_done, 0));
  G4_CUDA_TRY(fn, cudaMemcpyAsync(h_out, s.y_attn, static_cast<size_t>(rows) * H * 2,
                                  cudaMemcpyDeviceToHost, c->s_out));
  G4_CUDA_TRY(fn, cudaEventRecord(s.out_done, c->s_out));
  return 0;
}

int granite4_host_glue_sync(granite4_host_glue* c) {
  const char* fn = "granite4_host_glue_sync";
  if (c == nullptr) return g4::fail(fn, "invalid arguments");
  G4_CUDA_TRY(fn, cudaSetDevice(c->device));
  G4_CUDA_TRY(fn, cudaStreamSynchronize(c->s_out));
  c->set[0].busy = c->set[1].busy = false;
  return 0;
}

}  // extern "C"
