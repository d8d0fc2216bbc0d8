/* C ABI of libgranite4_b200.so: the Granite 4.2 8B per-layer glue kernels for
 * NVIDIA B200 (sm_100a).
 *
 * Conventions, identical to the reference engine's launchers
 * (engine/src/kernels_phase2.cu:822-836): every pointer named d_* is
 * caller-owned device memory on the current device; a launcher validates its
 * arguments, enqueues its kernels on the calling thread's stream (see
 * granite4_b200_set_stream) and returns without synchronising; it returns 0 on
 * success and -1 on invalid arguments or a launch error, with one diagnostic
 * line on stderr. Nothing here allocates unless its comment says so. bf16
 * tensors are passed as uint16_t bit patterns, FP8 e4m3 as uint8_t.
 *
 * "Kept" entry points have the reference's name, argument list and error
 * behaviour, so the reference's forward pass and tests link against this
 * library unchanged; the citation is the reference definition each replaces.
 * "Added" entry points cover fusions the reference does not have (its FP8
 * activation path is future work, docs/phases.md:714-715); they follow the same
 * conventions.
 */
#ifndef GRANITE4_B200_H
#define GRANITE4_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------ */
/* Library status (kept: engine/src/capi.h:18-66, engine/src/capi.cc:44-75)  */
/* ------------------------------------------------------------------------ */
typedef enum {
  granite4_status_ok = 0,
  granite4_unimplemented = 1,
  granite4_no_device = 2,
  granite4_unavailable = 3,
} granite4_status_code;

typedef struct {
  const char* model_id;
  long num_layers;
  long hidden_size;
  long intermediate_size;
  long num_attention_heads;
  long num_key_value_heads;
  long head_dim;
  long vocab_size;
  long max_context_length;
  const char* gpu_target; /* "sm_100a" here; the reference reports "sm_89" */
} granite4_model_info;

typedef struct {
  granite4_status_code status;
  int cuda_device_present;
  const char* status_text;
  const char* message; /* e.g. "device is sm_90, engine targets sm_100a" */
} granite4_status_info;

/* engine/src/capi.cc:44-58. NULL-tolerant, static strings, no allocation. */
void granite4_get_model_info(granite4_model_info* out);
/* engine/src/capi.cc:60-75 with the arch check of :17-36 retargeted to 10.0. */
void granite4_status(granite4_status_info* out);

/* ------------------------------------------------------------------------ */
/* Stream selection (added)                                                  */
/* ------------------------------------------------------------------------ */
/* Launch stream for the calling host thread, as a cudaStream_t. The default
 * (and the meaning of NULL) is the per-thread default stream the reference
 * build uses (engine/CMakeLists.txt:43-48). Always returns 0. */
int granite4_b200_set_stream(void* cuda_stream);
/* Reads the library's device status word on the current device into *out
 * (blocking device-to-host copy). 0 means no kernel has reported a problem;
 * bit 0: the embedding kernel gave up waiting for a bulk copy, bits 1-3: the
 * same for the norm, SwiGLU and RoPE kernels. A set bit means the outputs of
 * that launch are incomplete. Returns 0, or -1 if the word cannot be read. */
int granite4_b200_device_status(unsigned int* out);
/* cudaFree() for hosts that do not link the CUDA runtime themselves (ctypes,
 * cgo): releases a buffer granite4_rope_tables_build returned. 0 / -1. */
int granite4_b200_free(void* d_ptr);

/* ------------------------------------------------------------------------ */
/* a1. Embedding gather x embedding_multiplier                               */
/* ------------------------------------------------------------------------ */
/* Kept: granite4::prefill_embed_rows, engine/src/prefill_gemm.h:42-43,
 * engine/src/prefill_gemm.cu:1300-1309.
 * out[r][:] = bf16(mult * emb[d_tokens[start + r]][:]), r in [0, rows).
 * -1 when rows <= 0, rows > 65535 or H <= 0 (the reference's limits). */
int granite4_prefill_embed_rows(const int32_t* d_tokens, int start, int rows, const uint16_t* emb,
                                float mult, uint16_t* out, int H);
/* Added: the same gather without the 65535-row limit and with the vocabulary
 * size known: a row whose id is outside [0, vocab) is written as zeros instead
 * of reading out of bounds. */
int granite4_kernel_embed_gather(const int32_t* d_tokens, long long rows, const uint16_t* d_emb,
                                 int vocab, float mult, uint16_t* d_out, int H);

/* ------------------------------------------------------------------------ */
/* a2 / a5. Residual add + RMSNorm, bf16 and FP8 outputs                     */
/* ------------------------------------------------------------------------ */
/* Kept: engine/src/kernels_phase2.cu:910-920.
 * d_out[r][c] = bf16(x * r * w), r = 1 / sqrt(mean(x^2) + eps); -1 on NULL
 * pointers, non-finite or non-positive eps, rows or cols <= 0, or
 * rows * cols > INT_MAX. */
int granite4_kernel_rmsnorm(const uint16_t* d_x, const uint16_t* d_w, float eps, int rows, int cols,
                            uint16_t* d_out);
/* Kept: engine/src/kernels_phase2.cu:922-936 (additionally rows <= 16). */
int granite4_kernel_rmsnorm_batched(const uint16_t* d_x, const uint16_t* d_w, float eps, int rows,
                                    int cols, uint16_t* d_out);
/* Added: the residual add the reference does in its GEMM epilogues
 * (engine/src/prefill_gemm.cu:81-88, engine/src/forward_gpu.cu:988-995) fused
 * with the norm that follows it (engine/src/kernels_phase2.cu:51-132) and with a
 * per-tensor FP8 e4m3 quantisation of the normed output (the reference's weight
 * quantiser rule, engine/src/checkpoint_main.cc:118-122, :702-723):
 *   h = bf16(res + resid_mult * y)         (d_res == NULL: h = bf16(y))
 *   n = bf16(h * r * w)
 *   amax = max |n| over all rows, scale = float(amax / 448),
 *   code = e4m3(n / scale)                 (scale == 0: e4m3(n))
 * d_y is bf16 (y_is_f32 == 0) or f32; d_res likewise. Outputs, each optional:
 * d_h_out [rows][cols] bf16 (may alias d_res), d_n_bf16, d_n_fp8.
 * d_scale_amax: float[2] = {scale, amax}, required when d_n_fp8 is given.
 * d_rstd: optional float[rows]; receives r of every row. It is also scratch:
 * with it (and d_h_out) the second sweep that writes the codes is a plain
 * streaming pass over h instead of a second reduction per row.
 * cols must be a multiple of 8, at most 32768, and every row 16-byte aligned.
 * With d_n_fp8 this enqueues a 8-byte memset and two kernels (the scale depends
 * on every row, so the codes are written by a second sweep); with at most 16
 * rows and cols <= 8192 it is a single launch of one thread-block cluster that
 * keeps the rows in registers (same bits). */
int granite4_kernel_add_rmsnorm_fp8(const void* d_y, int y_is_f32, const void* d_res,
                                    int res_is_f32, const uint16_t* d_w, float eps,
                                    float resid_mult, int rows, int cols, uint16_t* d_h_out,
                                    uint16_t* d_n_bf16, uint8_t* d_n_fp8, float* d_scale_amax,
                                    float* d_rstd);
/* Added; no counterpart in the reference. The same op (h and FP8 codes out) for
 * callers that cannot allocate device memory at call time and so have no
 * d_rstd buffer to offer: an engine that gave the whole card to its arenas at
 * start-up, or a foreign-language binding that loads this library without the
 * CUDA runtime and has no cudaMalloc to call. The per-row scratch lives in a
 * 256 KB array inside the library instead (held by every GPU that loads it,
 * until the process exits), which limits rows to 65536; more rows are refused
 * with -1 and a message. The first call on a device resolves the array's
 * device address; make it before any stream capture. All calls on a device
 * share the array, so calls whose kernels may overlap on the GPU race on it;
 * nothing in it needs clearing between calls. Calls no allocator. */
int granite4_kernel_add_rmsnorm_fp8_noalloc(const void* d_y, int y_is_f32, const void* d_res,
                                            int res_is_f32, const uint16_t* d_w, float eps,
                                            float resid_mult, int rows, int cols,
                                            uint16_t* d_h_out, uint8_t* d_n_fp8,
                                            float* d_scale_amax);
/* Added: per-tensor FP8 quantisation of a bf16 tensor of n elements (n % 8 ==
 * 0) with the same rule; d_scale_amax as above. */
int granite4_kernel_fp8_quant(const uint16_t* d_x, long long n, uint8_t* d_codes,
                              float* d_scale_amax);

/* ------------------------------------------------------------------------ */
/* a3. RoPE on Q/K + int8 paged KV write                                     */
/* ------------------------------------------------------------------------ */
/* Kept: engine/src/kernels_phase2.cu:868-908. Builds the [max_pos][head_dim/2]
 * f32 cos and sin tables in double on the host and uploads them. ALLOCATES two
 * device buffers with cudaMalloc; the caller cudaFree()s them. Synchronous. */
int granite4_rope_tables_build(double theta, int head_dim, int max_pos, float** d_cos,
                               float** d_sin);
/* Kept: engine/src/kernels_phase2.cu:938-951. Row r of [rows][head_dim] is
 * rotated with table row r. */
int granite4_kernel_rope(const uint16_t* d_x, const float* d_cos, const float* d_sin, int rows,
                         int head_dim, uint16_t* d_out);
/* Kept: engine/src/kernels_phase2.cu:1107-1131. Quantise bf16 K/V rows
 * [rows][Hk][d] to int8 + per-(row, head) f32 scale and store them at pool rows
 * d_pt[base_pos + r] (d_pt == NULL: base_pos + r). rows <= 16. */
int granite4_kernel_kv_append_int8_batched(const uint16_t* d_src_k, const uint16_t* d_src_v,
                                           int8_t* d_cache_k, int8_t* d_cache_v,
                                           float* d_cache_k_scale, float* d_cache_v_scale,
                                           int base_pos, int rows, int stride, int Hk, int d,
                                           const int* d_pt);
/* Kept: granite4::prefill_rope_split_append_int8, engine/src/prefill_gemm.h:58-64,
 * engine/src/prefill_gemm.cu:1328-1346. Token-major qkv [rows][(Hq+2Hk) d] at
 * positions base_pos + r: RoPE(q) -> q_rot bf16; RoPE(k) (kept in f32) and raw
 * v quantised per (row, kv head) into the [Hk][stride][d] int8 caches with
 * [Hk][stride] f32 scales at pool row d_pt[pos] (NULL: pos). d must be 128,
 * rows <= 65535, stride >= base_pos + rows. */
int granite4_prefill_rope_split_append_int8(const uint16_t* qkv, const float* cos_tbl,
                                            const float* sin_tbl, int base_pos, int rows, int Hq,
                                            int Hk, int d, int stride, uint16_t* q_rot,
                                            int8_t* cache_k, int8_t* cache_v,
                                            float* cache_k_scale, float* cache_v_scale,
                                            const int* d_pt);
/* Device row descriptor of a multi-session step; layout of
 * granite4::GpuMultiRows, engine/src/forward_gpu_api.h:162-182. */
#define GRANITE4_MAX_VERIFY_ROWS 16
#define GRANITE4_MAX_TREE_DEPTH 8
typedef struct granite4_multi_rows {
  int n;
  int pos[GRANITE4_MAX_VERIFY_ROWS];
  const int* pt[GRANITE4_MAX_VERIFY_ROWS];
  int32_t* tok[GRANITE4_MAX_VERIFY_ROWS];
  int grp[GRANITE4_MAX_VERIFY_ROWS];
  int tree;
  int slot[GRANITE4_MAX_VERIFY_ROWS];
  int tbase[GRANITE4_MAX_VERIFY_ROWS];
  int tail[GRANITE4_MAX_VERIFY_ROWS][GRANITE4_MAX_TREE_DEPTH];
} granite4_multi_rows;
/* Kept: granite4::gpu_multi_rope_append, engine/src/forward_gpu_api.h:219-229,
 * engine/src/forward_gpu.cu:598-665, :3907-3914. Decode / verify form: separate
 * q [rows][Hq d], k, v [rows][Hk d]; row r's RoPE position is d_rows->pos[r] and
 * its pool row d_rows->pt[r][slot] (slot = pos, or d_rows->slot[r] for tree
 * rows). K is rounded to bf16 after the rotation and then quantised (bits == 8,
 * d == 128) or stored as bf16 (bits == 16, any even d <= 256; the scale
 * pointers are not used). The reference's 4- and 5-bit cache formats are not
 * built here: they return -1, which the reference's callers treat as "use the
 * unfused path". rows <= 16. */
int granite4_gpu_multi_rope_append(const uint16_t* q, const uint16_t* k, const uint16_t* v,
                                   const float* cos_tbl, const float* sin_tbl,
                                   const granite4_multi_rows* d_rows, int rows, int Hq, int Hk,
                                   int d, int bits, void* cache_k, void* cache_v, float* k_scale,
                                   float* v_scale, int stride, uint16_t* q_rot);
/* Kept: granite4::gpu_multi_rope, engine/src/forward_gpu_api.h:219-220,
 * engine/src/forward_gpu.cu:380-407, :3898-3906. x [rows][heads d]; row r is
 * rotated with table row d_rows->pos[r]. The descriptor's page tables are not
 * read. rows <= 16, d even. */
int granite4_gpu_multi_rope(const uint16_t* x, const float* cos_tbl, const float* sin_tbl,
                            const granite4_multi_rows* d_rows, int rows, int heads, int d,
                            uint16_t* out);
/* Kept: granite4::gpu_multi_kv_append, engine/src/forward_gpu_api.h:227-229,
 * engine/src/forward_gpu.cu:3915-3936. Appends K / V rows [rows][Hk d] as they
 * are at pool row d_rows->pt[r][slot]: bits == 8 quantises to int8 + f32 scales,
 * bits == 16 copies bf16 (scale pointers unused). Other formats return -1. */
int granite4_gpu_multi_kv_append(const uint16_t* k, const uint16_t* v, int bits, void* cache_k,
                                 void* cache_v, float* k_scale, float* v_scale,
                                 const granite4_multi_rows* d_rows, int rows, int stride, int Hk,
                                 int d);
/* Kept: engine/src/forward_gpu.cu:796-821, :3814-3826. One position: every head
 * of x [heads][d] is rotated with d_cos / d_sin, which point at that position's
 * own [d/2] table row. d even, <= 256. */
#define GRANITE4_MAX_HEAD_DIM 256
int granite4_kernel_rope_at_pos(const uint16_t* d_x, const float* d_cos, const float* d_sin,
                                int heads, int d, uint16_t* d_out);
/* Kept: engine/src/forward_gpu.cu:824-854, :3828-3842. Row r of x [rows][heads d]
 * is rotated with row r of the table pointers passed (the caller offsets them
 * to the first position). rows <= 16. */
int granite4_kernel_rope_at_pos_batched(const uint16_t* d_x, const float* d_cos,
                                        const float* d_sin, int rows, int heads, int d,
                                        uint16_t* d_out);
/* Kept: engine/src/kernels_phase2.cu:381-400, :1087-1105. bf16 cache form of the
 * batched append: K / V rows [rows][Hk d] copied to [Hk][stride][d] at pool row
 * d_pt[base_pos + r] (NULL: base_pos + r). rows <= 16; d must be even here (the
 * reference also takes odd d, which no RoPE model has). */
int granite4_kernel_kv_append_batched(const uint16_t* d_src_k, const uint16_t* d_src_v,
                                      uint16_t* d_cache_k, uint16_t* d_cache_v, int base_pos,
                                      int rows, int stride, int Hk, int d, const int* d_pt);
/* Kept: engine/src/forward_gpu.cu:3844-3874. Verify staging for a bf16 cache:
 * RoPE(q) -> d_q_rot, RoPE(k) -> d_k_rot, then d_k_rot and raw v appended at pool
 * rows d_pt[base_pos + r]. Row r uses row r of the table pointers passed. The
 * reference issues three launches; this is one. rows <= 16. */
int granite4_kernel_verify_qkv_stage(const uint16_t* d_q, const uint16_t* d_k, const uint16_t* d_v,
                                     const float* d_cos, const float* d_sin, int base_pos, int rows,
                                     int Hq, int Hk, int d, int cache_stride, uint16_t* d_q_rot,
                                     uint16_t* d_k_rot, uint16_t* d_cache_k, uint16_t* d_cache_v,
                                     const int* d_pt);
/* Kept: granite4::prefill_rope_split_append, engine/src/prefill_gemm.h:48-52,
 * engine/src/prefill_gemm.cu:306-347, :1310-1324. bf16 cache form of the prefill
 * step: token-major qkv at positions base_pos + r; RoPE(q) -> q_rot, RoPE(k) and
 * raw v into the [Hk][stride][d] bf16 caches at pool row d_pt[pos] (NULL: pos).
 * Any even d; rows <= 65535. */
int granite4_prefill_rope_split_append(const uint16_t* qkv, const float* cos_tbl,
                                       const float* sin_tbl, int base_pos, int rows, int Hq, int Hk,
                                       int d, int stride, uint16_t* q_rot, uint16_t* cache_k,
                                       uint16_t* cache_v, const int* d_pt);
/* Added: the prefill form with per-row positions and pool rows, for batches
 * whose rows are not one consecutive run of positions (several sequences,
 * offsets, permuted page tables). d_pos_rows[r] in [0, max_pos) indexes the
 * RoPE tables; d_kv_rows[r] in [0, stride) is the pool row (page_id * 16 + pos %
 * 16 under 16-token pages, engine/src/kv_pool.cc:285-298); rows with an index
 * outside those ranges are skipped. k_from_bf16 selects the decode kernels'
 * rounding of K (1) or the prefill kernel's (0). d must be 128. */
int granite4_kernel_rope_kv_int8_paged(const uint16_t* d_qkv, const float* d_cos,
                                       const float* d_sin, const int* d_pos_rows,
                                       const int* d_kv_rows, int rows, int Hq, int Hk, int d,
                                       int stride, int max_pos, int k_from_bf16,
                                       uint16_t* d_q_rot, int8_t* d_cache_k, int8_t* d_cache_v,
                                       float* d_k_scale, float* d_v_scale);

/* ------------------------------------------------------------------------ */
/* Decode-step glue around the path: greedy pick, token chaining, KV moves   */
/* ------------------------------------------------------------------------ */
/* Added (the reference keeps these kernels private to its forward pass:
 * argmax_rows_kernel engine/src/forward_gpu.cu:280-333, argmax_map_kernel
 * engine/src/eagle_gpu.cu:155-178). d_out[r] = first index of the maximum of
 * bf16 logits row r ([rows][V]); NaN never wins, a row with nothing above -inf
 * gives 0. d_vocab_map (optional): the id written is d_vocab_map[index]. d_pos
 * (optional, rows must be 1): the id goes to d_out[*d_pos + 1] and *d_pos is
 * advanced, which chains captured decode steps on the device. */
int granite4_kernel_argmax_rows(const uint16_t* d_logits, int rows, int V, int32_t* d_out,
                                int* d_pos, const int32_t* d_vocab_map);
/* Added: the greedy pick of a multi-session step fused with the token scatter
 * that follows it in the reference's decode graph (argmax_rows_kernel then
 * multi_scatter_advance_kernel, engine/src/forward_gpu.cu:2617, :758-764): for
 * r < rows, id = first index of the maximum of logits row r;
 * d_rows->tok[r][pos[r] + 1] = id; d_rows->pos[r] += 1; d_ids_out[r] = id when
 * d_ids_out is given. rows <= 16. */
int granite4_kernel_argmax_advance(const uint16_t* d_logits, int rows, int V,
                                   granite4_multi_rows* d_rows, int32_t* d_ids_out);
/* Added (embed_multi_v8_kernel, engine/src/forward_gpu.cu:359-378, private to the
 * reference's forward pass): the embedding rows of a multi-session step.
 * d_out[r] = bf16(mult * d_emb[tok]) with tok = d_rows->tok[r][slot], slot =
 * d_rows->pos[r] (d_rows->slot[r] for tree rows); an id outside [0, vocab)
 * gives a zero row. rows <= 16, H a multiple of 8. Reads the token on the
 * device, so a captured decode step follows the positions as they advance. */
int granite4_gpu_multi_embed(const granite4_multi_rows* d_rows, int rows, const uint16_t* d_emb,
                             int vocab, float mult, uint16_t* d_out, int H);
/* Added (multi_scatter_advance_kernel, engine/src/forward_gpu.cu:758-764): for
 * r < d_rows->n: d_rows->tok[r][pos[r] + 1] = d_ids[r]; pos[r] += 1. */
int granite4_kernel_multi_scatter_advance(granite4_multi_rows* d_rows, const int32_t* d_ids);
/* Added (kv_move_kernel / gpu_ctx_kv_move, engine/src/forward_gpu.cu:3473-3536):
 * copy KV rows src_rows[i] -> dst_rows[i], i in order, in every layer and kv
 * head of a [layers][Hk][stride][d] pool (int8 codes + [layers][Hk][stride]
 * scales for bits == 8, bf16 for bits == 16). src_rows / dst_rows are HOST
 * arrays of n <= 8 physical pool rows (the caller maps logical positions
 * through its row table, as gpu_ctx_kv_move does). A later move must not read a
 * row an earlier one overwrites (-1). One launch for all layers. */
int granite4_kernel_kv_move(const int* src_rows, const int* dst_rows, int n, int bits,
                            void* d_cache_k, void* d_cache_v, float* d_k_scale, float* d_v_scale,
                            int layers, int Hk, int stride, int d);

/* ------------------------------------------------------------------------ */
/* Host-side paged KV pool (no device work)                                  */
/* ------------------------------------------------------------------------ */
/* Added; the reference's granite4::PagedKV (engine/src/kv_pool.h:102-199,
 * engine/src/kv_pool.cc) behind a C interface: 16-token pages (any page size),
 * dense per-sequence block tables, a prefix cache over full pages keyed by the
 * chained FNV-1a hash of the token prefix (verified against the stored token
 * ids), reference counts, least-recently-used eviction of cached pages nobody
 * references. Same page ids, row tables and counts as the reference for the same
 * sequence of calls, with one deliberate difference: truncate_sequence always
 * shortens the token record of the last kept page to what is left of it (the
 * reference leaves it long when no page is dropped, after which a further
 * reserve on that sequence records more than a page's worth of ids for it).
 * Returns: create_sequence the new id or -1; match_prefix the number of leading
 * tokens now covered by shared cached pages (a multiple of the page size; only
 * on a sequence that holds nothing yet); reserve / mark_written / row_table 1 on
 * success, 0 otherwise. row_table writes out[p] = page * tokens_per_page + p %
 * tokens_per_page for p < n <= the sequence's token count: the d_pt / kv_rows
 * table of the KV-write and attention entry points. Not thread-safe. */
typedef struct granite4_kv_pool granite4_kv_pool;
enum {
  GRANITE4_KV_POOL_FREE_PAGES = 0,
  GRANITE4_KV_POOL_USED_PAGES = 1,
  GRANITE4_KV_POOL_SHARED_PAGES = 2,   /* reference count > 1 */
  GRANITE4_KV_POOL_CACHED_PAGES = 3,   /* entries of the prefix cache */
  GRANITE4_KV_POOL_EVICTED_PAGES = 4,  /* evictions so far */
  GRANITE4_KV_POOL_RETAINED_PAGES = 5, /* cached, reference count 0 */
  GRANITE4_KV_POOL_LIVE_SEQUENCES = 6
};
granite4_kv_pool* granite4_kv_pool_create(int num_pages, int tokens_per_page);
void granite4_kv_pool_destroy(granite4_kv_pool* pool);
int granite4_kv_pool_create_sequence(granite4_kv_pool* pool);
long long granite4_kv_pool_match_prefix(granite4_kv_pool* pool, int seq, const uint32_t* tokens,
                                        long long n);
int granite4_kv_pool_reserve(granite4_kv_pool* pool, int seq, long long token_count,
                             const uint32_t* tokens, long long n);
int granite4_kv_pool_mark_written(granite4_kv_pool* pool, int seq, long long page_index);
int granite4_kv_pool_row_table(const granite4_kv_pool* pool, int seq, long long n, int* out);
void granite4_kv_pool_reset_sequence(granite4_kv_pool* pool, int seq);
void granite4_kv_pool_truncate_sequence(granite4_kv_pool* pool, int seq, long long n_tokens);
void granite4_kv_pool_release(granite4_kv_pool* pool, int seq);
void granite4_kv_pool_clear(granite4_kv_pool* pool);
long long granite4_kv_pool_count(const granite4_kv_pool* pool, int which);
long long granite4_kv_pool_sequence_tokens(const granite4_kv_pool* pool, int seq);
/* Writes min(capacity, pages) page ids to out (may be NULL); returns the number of pages. */
long long granite4_kv_pool_block_table(const granite4_kv_pool* pool, int seq, int* out,
                                       long long capacity);
int granite4_kv_pool_ref_count(const granite4_kv_pool* pool, int page);
int granite4_kv_pool_page_in_cache(const granite4_kv_pool* pool, int page);
/* The host half of gpu_ctx_kv_move (engine/src/forward_gpu.cu:3508-3522): maps n
 * <= 8 logical (src, dst) positions of a sequence to pool rows for
 * granite4_kernel_kv_move, with the reference's checks (positions inside the
 * sequence's pages, dst <= src, no later move reading a row an earlier one
 * overwrites). 0, or -1 if a check fails. */
int granite4_kv_pool_move_rows(const granite4_kv_pool* pool, int seq, const int* src_pos,
                               const int* dst_pos, int n, int* src_rows, int* dst_rows);

/* ------------------------------------------------------------------------ */
/* Serve-loop controller over the pool: session slots (no device work)       */
/* ------------------------------------------------------------------------ */
/* Added; the reference's granite4::KvPoolController
 * (engine/src/kv_pool_controller.h:32-112, engine/src/kv_pool_controller.cc)
 * behind a C interface. It owns one pool and maps session slots (one per
 * concurrent request; at most num_pages of them) to pool sequences. Same slot
 * ids, return values, row tables and pool counts as the reference for the same
 * sequence of calls.
 *   new_slot      a slot id, or -1 when the pool has no sequence left. An idle
 *                 slot (released earlier) is recycled first, lowest id first,
 *                 and stays idle until prefill or open_slot puts it in use.
 *   release_slot  ends a session: private pages freed, published pages stay
 *                 cached; the id can be reused.
 *   shutdown      frees everything and empties the cache; all slot ids die.
 *   prefill       starts a request on a slot: drops what the slot held, adopts
 *                 the cached page-aligned prefix of prompt[0..n), reserves the
 *                 rest, publishes every full page. Returns 1 and writes the
 *                 pool sequence id and the number of leading tokens whose KV
 *                 is already in the pool rows the row table names (the GPU may
 *                 skip them) to *seq_out / *reused_out (either may be NULL);
 *                 0 when the pool cannot hold the prompt (the slot is left
 *                 idle and clean, *seq_out = -1, *reused_out = 0).
 *   commit        after a generated token, with the session's full id list:
 *                 grows by a page at page boundaries, publishes pages as they
 *                 fill; no effect when n does not exceed what is committed.
 *   open_slot / ensure / trim / drop / pages_missing / slot_pages: resident
 *                 sessions that never share pages - make a slot live, grow it
 *                 to n_tokens (1, or 0 and nothing changed), hand back the
 *                 pages past n_tokens, drop all pages, pages still needed for
 *                 n_tokens, pages held.
 *   row_table     out[p] = pool row of position p for p < n <= committed(slot):
 *                 the d_pt / kv_rows table of the KV-write and attention entry
 *                 points; rows of committed positions never move. 1 / 0.
 *   count         granite4_kv_pool_count of the pool underneath (same enum);
 *                 granite4_kv_ctl_pool exposes that pool for inspection and
 *                 for granite4_kv_pool_move_rows (it stays owned by the
 *                 controller). Not thread-safe. */
typedef struct granite4_kv_ctl granite4_kv_ctl;
granite4_kv_ctl* granite4_kv_ctl_create(int num_pages, int tokens_per_page);
void granite4_kv_ctl_destroy(granite4_kv_ctl* ctl);
void granite4_kv_ctl_shutdown(granite4_kv_ctl* ctl);
granite4_kv_pool* granite4_kv_ctl_pool(granite4_kv_ctl* ctl);
int granite4_kv_ctl_new_slot(granite4_kv_ctl* ctl);
void granite4_kv_ctl_release_slot(granite4_kv_ctl* ctl, int slot);
int granite4_kv_ctl_prefill(granite4_kv_ctl* ctl, int slot, const uint32_t* prompt, long long n,
                            int* seq_out, long long* reused_out);
void granite4_kv_ctl_commit(granite4_kv_ctl* ctl, int slot, const uint32_t* all_tokens, long long n);
int granite4_kv_ctl_open_slot(granite4_kv_ctl* ctl);
int granite4_kv_ctl_ensure(granite4_kv_ctl* ctl, int slot, long long n_tokens);
void granite4_kv_ctl_trim(granite4_kv_ctl* ctl, int slot, long long n_tokens);
void granite4_kv_ctl_drop(granite4_kv_ctl* ctl, int slot);
long long granite4_kv_ctl_slot_pages(const granite4_kv_ctl* ctl, int slot);
long long granite4_kv_ctl_pages_missing(const granite4_kv_ctl* ctl, int slot, long long n_tokens);
int granite4_kv_ctl_row_table(const granite4_kv_ctl* ctl, int slot, long long n, int* out);
long long granite4_kv_ctl_committed(const granite4_kv_ctl* ctl, int slot);
long long granite4_kv_ctl_last_reused(const granite4_kv_ctl* ctl, int slot);
long long granite4_kv_ctl_max_slots(const granite4_kv_ctl* ctl);
long long granite4_kv_ctl_count(const granite4_kv_ctl* ctl, int which);

/* ------------------------------------------------------------------------ */
/* Decode / verify attention over the int8 paged pool                        */
/* ------------------------------------------------------------------------ */
/* Added; the int8 multi-sequence mode of granite4::attn_split
 * (engine/src/attention_gpu.h:15-68) as a C entry point. Row r of d_q
 * [rows][Hq 128] (bf16, already rotated) is at position d_row_pos[r] of its
 * sequence and attends to cache positions 0..d_row_pos[r]; position t of that
 * sequence lives in pool row table[t], where table is d_row_pt[r] when
 * d_row_pt is given (a device array of per-row device tables), else d_pt for
 * every row, else the identity. rows_per_group (1..4) consecutive rows belong
 * to ONE sequence (a verify step's rows; they share the first row's table) and
 * read each cache tile once; use 1 for independent decode rows. The pool is
 * what granite4_kernel_rope_kv_int8_paged writes: codes [Hk][stride][128] int8,
 * scales [Hk][stride] f32. logits = scale * q . k. d_out [rows][Hq 128] bf16.
 * max_len bounds every position + 1 (it sizes the split of the cache range and
 * the scratch): d_scratch must hold granite4_attn_decode_scratch_bytes(...)
 * bytes, 16-byte aligned (may be NULL when that returns a plan of one split,
 * i.e. for short contexts with many rows). Only d == 128 and Hq == 4 Hk are
 * built; anything else returns -1 like the reference's kernel. A row with a
 * negative position gets zeros. */
long long granite4_attn_decode_scratch_bytes(int rows, int rows_per_group, int Hk, int max_len);
int granite4_kernel_attn_decode_int8_paged(const uint16_t* d_q, const int8_t* d_cache_k,
                                           const int8_t* d_cache_v, const float* d_k_scale,
                                           const float* d_v_scale, const int* d_row_pos,
                                           const int* const* d_row_pt, const int* d_pt, int rows,
                                           int rows_per_group, int Hq, int Hk, int d, int stride,
                                           int max_len, float scale, void* d_scratch,
                                           long long scratch_bytes, uint16_t* d_out);

/* The reference's split-KV contract (granite4::attn_split, engine/src/attention_gpu.h:15-68)
 * for the int8 cache, argument for argument (the bf16 / int4 cache pointers and
 * flags of that signature are left out; the C++ symbol granite4::attn_split
 * with the full signature is exported too and returns -1 for those formats):
 *   rows 1..16 query rows d_q [rows][Hq 128].
 *   d_row_pos NULL: the rows are consecutive positions p, p + 1, ... of ONE
 *     sequence, p = *d_pos (read on the device) when d_pos is given, else
 *     kv_base; position t lives in pool row d_pt[t] (NULL: t).
 *   d_row_pos / d_row_pt (both or neither): row r is at position d_row_pos[r]
 *     and reads through its own table d_row_pt[r]; every row is a sequence of
 *     its own unless d_row_grp says otherwise.
 *   d_row_grp / ngroups: group z owns rows [w & 0xff, + (w >> 8)) (at most 4)
 *     of one sequence, which then read each cache tile once and share the
 *     first row's table.
 *   d_row_tbase / d_row_tail (both or neither; need d_row_pos): draft-tree
 *     rows. Logical positions up to tbase = d_row_tbase[first row of the
 *     group] are the sequence's own; position tbase + 1 + j of row r is the
 *     slot d_row_tail[r * 8 + j] (an ancestor of r in the tree), looked up
 *     through the table like any position; at most 8 such positions per row.
 *   window > 0: a row attends to its last `window` positions only,
 *     (pos - window, pos].
 *   max_len (0 = stride) bounds every position + 1 and sizes the split of the
 *     cache range; d_scratch must hold granite4_attn_split_scratch_bytes(Hq,
 *     rows, max_len) bytes (an upper bound over every grouping of the rows).
 * Results are those of one single-row call per row at its position. -1 on
 * invalid arguments and for shapes other than d == 128, Hq == 4 Hk. */
long long granite4_attn_split_scratch_bytes(int Hq, int rows, int max_len);
int granite4_attn_split_int8(const uint16_t* d_q, const int8_t* d_cache_k8, const int8_t* d_cache_v8,
                             const float* d_k_scale, const float* d_v_scale, float scale, int Hq,
                             int Hk, int d, int kv_base, const int* d_pos, int rows, int stride,
                             void* d_scratch, long long scratch_bytes, uint16_t* d_out, const int* d_pt,
                             int max_len, const int* d_row_pos, const int* const* d_row_pt,
                             const int* d_row_grp, int ngroups, const int* d_row_tbase,
                             const int* d_row_tail, int window);

/* ------------------------------------------------------------------------ */
/* a4. SwiGLU, bf16 and FP8 outputs                                          */
/* ------------------------------------------------------------------------ */
/* Kept: granite4::prefill_silu_mul, engine/src/prefill_gemm.h:105,
 * engine/src/prefill_gemm.cu:1468-1474. gu is f32 [rows][2 I] (gate columns
 * first); act[r][i] = bf16(silu(gu[r][i]) * gu[r][I + i]). */
int granite4_prefill_silu_mul(const float* gu, int I, int rows, uint16_t* act);
/* Added: SwiGLU on bf16 (in_is_f32 == 0) or f32 gate / up rows of pitch ld
 * elements, with optional bf16 output and optional per-tensor FP8 output:
 *   a = bf16(silu(g) * u), amax = max |a|, scale = float(amax / 448),
 *   code = e4m3(a / scale).
 * d_scale_amax: float[2] = {scale, amax}, required with d_act_fp8. I must be
 * a multiple of 8, rows 16-byte aligned. With d_act_fp8 this enqueues an 8-byte
 * memset and two kernels. */
/* Added. The second half of a per-tensor FP8 quantisation whose first half (the
 * max |x|) another kernel already did: d_scale_amax[1] holds the max |x| of
 * the bf16 tensor d_x (n elements, n % 8 == 0, 16-byte aligned), the call
 * writes the scale to d_scale_amax[0] and the e4m3 codes to d_codes. One sweep:
 * 2 bytes read, 1 written per element. */
int granite4_kernel_fp8_encode_with_amax(const uint16_t* d_x, long long n, uint8_t* d_codes,
                                         float* d_scale_amax);
int granite4_kernel_swiglu_fp8(const void* d_gate, const void* d_up, int in_is_f32, long long ld,
                               int rows, int I, uint16_t* d_act_bf16, uint8_t* d_act_fp8,
                               float* d_scale_amax);

/* ------------------------------------------------------------------------ */
/* One layer's glue in one call (added)                                      */
/* ------------------------------------------------------------------------ */
/* The four glue launches of one transformer layer, in the order the
 * reference's prefill path issues them between its GEMMs
 * (engine/src/forward_gpu.cu:2786-2845): residual add + norm -> FP8 on the
 * attention output, RoPE + int8 paged KV write on the QKV output, residual add
 * + norm -> FP8 on the MLP output, SwiGLU -> FP8 on the gate/up output. It only
 * saves host launch overhead: results are those of the four entry points above.
 * Every pointer is device memory. */
typedef struct granite4_glue_layer_args {
  /* stand-ins for GEMM / attention outputs, bf16 */
  const uint16_t* y_attn; /* [rows][hidden]  O-projection output   */
  const uint16_t* y_mlp;  /* [rows][hidden]  down-projection output */
  const uint16_t* qkv;    /* [rows][(q_heads + 2 kv_heads) head_dim] */
  const uint16_t* gate;   /* [rows][intermediate] */
  const uint16_t* up;     /* [rows][intermediate] */
  /* weights and tables */
  const uint16_t* w_attn_norm; /* [hidden] bf16, norm after the attention block */
  const uint16_t* w_mlp_norm;  /* [hidden] bf16, norm after the MLP block */
  const float* cos_tbl;        /* [max_pos][head_dim / 2] */
  const float* sin_tbl;
  const int* pos_rows; /* [rows] RoPE position of each row */
  const int* kv_rows;  /* [rows] pool row of each row */
  /* residual stream, updated in place twice */
  uint16_t* hidden; /* [rows][hidden] bf16 */
  /* outputs */
  uint8_t* n_attn_fp8; /* [rows][hidden] e4m3: norm after the attention block (input of the MLP GEMMs) */
  uint8_t* n_mlp_fp8;  /* [rows][hidden] e4m3: norm after the MLP block (input of the next QKV GEMM) */
  uint16_t* q_rot;     /* [rows][q_heads head_dim] bf16 */
  int8_t* cache_k;     /* [kv_heads][pool_rows][head_dim] */
  int8_t* cache_v;
  float* k_scale; /* [kv_heads][pool_rows] */
  float* v_scale;
  uint8_t* act_fp8; /* [rows][intermediate] e4m3 */
  float* scales;    /* [3][2]: {scale, amax} of n_attn, n_mlp, act */
  /* optional scratch between the two sweeps of the FP8 ops (may be NULL) */
  float* rstd;      /* [rows] */
  uint16_t* act_ws; /* [rows][intermediate] bf16 */
  int rows, hidden_size, intermediate, q_heads, kv_heads, head_dim, pool_rows, max_pos;
  float eps, resid_mult;
} granite4_glue_layer_args;
int granite4_glue_layer(const granite4_glue_layer_args* a);

/* ------------------------------------------------------------------------ */
/* The same layer through HOST buffers (added)                               */
/* ------------------------------------------------------------------------ */
/* For callers whose activations live in host memory: a context owns device
 * staging for max_rows rows (two sets, so the copies of one call overlap the
 * kernels and the read-back of the previous one), the int8 KV pool of every
 * layer, the RoPE tables, three streams and their events.
 * granite4_host_glue_create ALLOCATES (cudaMalloc, streams, events);
 * granite4_host_glue_destroy frees. */
typedef struct granite4_host_glue granite4_host_glue;
granite4_host_glue* granite4_host_glue_create(int max_rows, int hidden_size, int intermediate,
                                              int q_heads, int kv_heads, int head_dim, int layers,
                                              int pool_rows, int max_pos, double rope_theta);
void granite4_host_glue_destroy(granite4_host_glue* ctx);
/* Host-side arguments of one layer call; every pointer is HOST memory (pinned
 * memory makes the copies asynchronous; pageable memory works but serialises). */
typedef struct granite4_host_layer_io {
  const uint16_t* y_attn;
  const uint16_t* y_mlp;
  const uint16_t* qkv;
  const uint16_t* gate;
  const uint16_t* up;
  const uint16_t* w_attn_norm;
  const uint16_t* w_mlp_norm;
  const int* pos_rows;
  const int* kv_rows;
  /* The residual stream is context state that stays on the device from one layer call to
   * the next. hidden_in (optional): upload it before this layer (the first layer's input);
   * hidden_out (optional): read it back after this layer (the last layer's output). */
  const uint16_t* hidden_in; /* [rows][hidden] or NULL */
  uint16_t* hidden_out;      /* [rows][hidden] or NULL */
  uint8_t* n_attn_fp8;
  uint8_t* n_mlp_fp8;
  uint16_t* q_rot;
  uint8_t* act_fp8;
  float* scales; /* [3][2] */
  int rows;
  float eps, resid_mult;
} granite4_host_layer_io;
/* Enqueues: host -> device copies of the inputs, the layer's kernels, device ->
 * host copies of the outputs (the KV pool stays on the device; it is the
 * context's state, as in the reference). Returns as soon as everything is
 * enqueued; the outputs are valid after granite4_host_glue_sync. At most two
 * calls are in flight: a third call first waits for the oldest one. */
int granite4_host_glue_layer(granite4_host_glue* ctx, int layer, const granite4_host_layer_io* io);
/* The final norm (a5) of the resident residual stream with the HOST weights h_w
 * [hidden]; the normed rows are copied to the HOST buffer h_out [rows][hidden].
 * Asynchronous like granite4_host_glue_layer. */
int granite4_host_glue_final_norm(granite4_host_glue* ctx, const uint16_t* h_w, float eps, int rows,
                                  uint16_t* h_out);
int granite4_host_glue_sync(granite4_host_glue* ctx);
/* Bytes one call copies host -> device and device -> host for `rows` rows, not
 * counting the optional transfers of the residual stream. */
long long granite4_host_glue_h2d_bytes(const granite4_host_glue* ctx, int rows);
long long granite4_host_glue_d2h_bytes(const granite4_host_glue* ctx, int rows);

/* granite4::prefill_attention with the int8 cache (engine/src/prefill_gemm.h:86-101)
 * as a C entry point: causal attention of the query rows at positions
 * [base_pos, base_pos + rows) of ONE sequence (d_q_rot [rows][Hq 128] bf16, as
 * the RoPE kernels write it) over cache positions [0, position], position t in
 * pool row d_pt[t] (NULL: t). Chunks of 32 rows or more run as a flash kernel
 * (32 query positions x 4 heads per CTA share each K / V tile; no scratch);
 * shorter ones on the decode kernel as groups of four consecutive rows, where
 * d_scratch / scratch_bytes (optional,
 * granite4_attn_decode_scratch_bytes(rows, 4, Hk, base_pos + rows) bytes) let a
 * short chunk at a long context split the context over CTAs; without it the
 * range is walked in one piece. -1 as granite4_kernel_attn_decode_int8_paged. */
int granite4_prefill_attention_int8(const uint16_t* d_q_rot, float scale, int Hq, int Hk, int d,
                                    int base_pos, int rows, int stride, uint16_t* d_out,
                                    const int8_t* d_cache_k8, const int8_t* d_cache_v8,
                                    const float* d_k_scale, const float* d_v_scale, const int* d_pt,
                                    void* d_scratch, long long scratch_bytes);

/* ------------------------------------------------------------------------ */
/* FP8 x FP8 GEMM consuming the glue's FP8 outputs                            */
/* ------------------------------------------------------------------------ */
/* Added; the FP8-activation counterpart of granite4::prefill_gemm
 * (engine/src/prefill_gemm.h:12-36). C[M][N] = a_scale * w_scale(n) * A[M][K] x
 * W[N][K]^T with A e4m3 codes of row pitch lda bytes (what
 * granite4_kernel_add_rmsnorm_fp8 / _swiglu_fp8 write), W e4m3 row-major (the
 * reference's weight layout) and f32 accumulation on the tensor cores. The
 * activation scale is read from DEVICE memory (d_a_scale, slot 0 of the glue's
 * {scale, amax} pair; NULL = 1), the weight scales are passed by value like the
 * reference's GemmEpilogue: w_scale(n) = w_scale0 for n < seg1, w_scale1 for
 * n < seg2, else w_scale2. Output kinds as GemmOut: bf16(y), f32 y, or
 * bf16(residual + resid_scale * y) (d_residual may alias d_out_bf16).
 * GRANITE4_GEMM_OUT_SWIGLU folds prefill_silu_mul (engine/src/prefill_gemm.h:105)
 * into the epilogue of the gate|up projection: W holds the I = N / 2 gate rows,
 * then the I up rows (the reference's stacked layout), d_out_bf16 [M][I] gets
 * a = bf16(silu(y_gate) * y_up) computed from the f32 sums (as the reference
 * does from its f32 GEMM output), and max |a| is written to
 * d_out_scale_amax[1] (cleared by the call), so that
 * granite4_kernel_fp8_encode_with_amax turns a into FP8 codes in one sweep;
 * the 4 I bytes per row of gate|up output never exist.
 * Needs K % 16 == 0, lda % 16 == 0, 16-byte aligned A and W; any M >= 0, any N.
 * d_ws / ws_bytes, as the ws / ws_bytes of prefill_gemm: with a few rows a
 * GEMM has too few output tiles to occupy the card and splits K across CTAs,
 * which add their partial sums in a fixed order (the result does not depend on
 * scheduling). Up to 16 rows the slices of a tile are the CTAs of one
 * thread-block cluster and exchange their sums through its shared memory: no
 * workspace is wanted. The older forms (selected by G4_GEMM_DECODE=0 in the
 * environment, or where the device cannot co-schedule the cluster) split
 * through d_ws. granite4_gemm_fp8_workspace_bytes(M, N, K) is the size that
 * allows the planned split (0: none wanted); the buffer must be zeroed once
 * before its first use (every call leaves its first bytes, the tile counters,
 * zero again) and belongs to one call at a time. The counters return to zero
 * only when a call runs to completion: after granite4_b200_device_status
 * reported a non-zero word (a bounded wait ran out and the kernel left early),
 * or after a failed launch, zero the buffer again before reusing it, or later
 * calls sum stale partials without reporting anything. NULL or a smaller
 * buffer: no split. d_w must not be written by the operation just before this call on
 * the stream: with at most 128 rows the kernel starts fetching weights while
 * that operation drains (weights are constants of a loaded model). Returns 0,
 * or -1 on bad arguments or a launch error. */
enum {
  GRANITE4_GEMM_OUT_BF16 = 0,
  GRANITE4_GEMM_OUT_F32 = 1,
  GRANITE4_GEMM_OUT_RESIDUAL = 2,
  GRANITE4_GEMM_OUT_SWIGLU = 3
};
typedef struct granite4_gemm_fp8_epilogue {
  const float* d_a_scale;
  float w_scale0, w_scale1, w_scale2;
  int seg1, seg2;
  uint16_t* d_out_bf16;
  float* d_out_f32;
  const uint16_t* d_residual;
  float resid_scale;
  int ldc; /* output (and residual) row pitch, elements */
  float* d_out_scale_amax; /* GRANITE4_GEMM_OUT_SWIGLU only: {scale, amax} of the activations */
} granite4_gemm_fp8_epilogue;
long long granite4_gemm_fp8_workspace_bytes(int M, int N, int K);
int granite4_kernel_gemm_fp8(int out_kind, const uint8_t* d_a, long long lda, const uint8_t* d_w, int M,
                             int N, int K, const granite4_gemm_fp8_epilogue* ep, void* d_ws,
                             long long ws_bytes);

#ifdef __cplusplus
}
#endif
#endif /* GRANITE4_B200_H */
