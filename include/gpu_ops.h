/*
 * gpu_ops.h -- C ABI of libgpu_ops.so: the attention hot path of llm_simple
 * (RoPE, KV-cache append, causal prefill attention, grouped-query decode) as
 * hand-written CUDA kernels for NVIDIA B200 (sm_100a).
 *
 * Every entry point replaces one operator of the reference's
 * prebuild/npu_ops.h (cited per function) or is a fused form of several.
 * Differences from the reference's calling convention, all deliberate:
 *   - C linkage; the stream is a cudaStream_t passed by value as an opaque
 *     pointer (the reference passes `aclrtStream&`);
 *   - every function returns an int status: 0 on success, a negative
 *     GPU_OPS_E_* code otherwise (the reference returns void and logs);
 *     gpu_ops_last_error_string() describes the last failure of the calling
 *     thread;
 *   - all arguments are validated on the host before anything is launched; no
 *     kernel traps or asserts;
 *   - `dt` is the reference's DataType value: 4 = fp16, 5 = bf16
 *     (prebuild/defs.hpp:8-18).  Accumulation is always fp32.
 *
 * All pointers are device pointers unless a parameter is documented as host
 * memory.  Calls are asynchronous on `stream`.  head_dim must be 128 (every
 * model the reference supports has head_dim 128); other values are rejected
 * with GPU_OPS_E_UNSUPPORTED.
 */
#ifndef LLM_SIMPLE_GPU_OPS_H_
#define LLM_SIMPLE_GPU_OPS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *gpu_stream_t; /* a cudaStream_t; NULL is the default stream */

enum {
  GPU_OPS_OK = 0,
  GPU_OPS_E_INVALID = -1,     /* null pointer, non-positive extent, inconsistent arguments */
  GPU_OPS_E_UNSUPPORTED = -2, /* dtype / head_dim / shape outside what the kernels cover */
  GPU_OPS_E_WORKSPACE = -3,   /* workspace missing or too small */
  GPU_OPS_E_CUDA = -4         /* a CUDA runtime call or launch failed */
};

enum { GPU_DT_FLOAT16 = 4, GPU_DT_BFLOAT16 = 5 };

/* ------------------------------------------------------------------------
 * Reference-shaped operators.  Same argument order and meaning as the
 * reference; K/V are token-major [n][kv_heads][head_dim] (the layout of the
 * reference's caches, src/llama2_layer_npu.cpp:325-338, :1148-1149).
 * ------------------------------------------------------------------------ */

/* Replaces npu_flash_attn_layer (prebuild/npu_ops.h:6-8).
 * q [m][head_num][head_dim], k/v [n][head_num][head_dim] (first n rows valid),
 * out [m][head_num*head_dim].  Row r attends to columns c <= r + offset
 * (tests/flash_attn_test.cpp:124-132); scale 1/sqrt(head_dim). */
int gpu_flash_attn_layer(void *output_dev, const void *q_dev, const void *k_dev,
                         const void *v_dev, int m, int n, int offset, int head_num,
                         int head_dim, int dt, gpu_stream_t stream);

/* Replaces npu_flash_attn_gqa_layer (prebuild/npu_ops.h:10-13).
 * q [m][kv_head_num*group_size][head_dim], k/v [n][kv_head_num][head_dim];
 * query head h reads KV head h / group_size (call site
 * src/llama2_layer_npu.cpp:866-869). */
int gpu_flash_attn_gqa_layer(void *output_dev, const void *q_dev, const void *k_dev,
                             const void *v_dev, int m, int n, int offset, int group_size,
                             int kv_head_num, int head_dim, int dt, gpu_stream_t stream);

/* Replaces npu_flash_attn_opt_prefill_layer (prebuild/npu_ops.h:15-18); the
 * reference uses it for prefill and for decode (m = 1) alike
 * (src/llama2_layer_npu.cpp:371-374).  Same contract as gpu_flash_attn_layer. */
int gpu_flash_attn_opt_prefill_layer(void *output_dev, const void *q_dev, const void *k_dev,
                                     const void *v_dev, int m, int n, int offset,
                                     int head_num, int head_dim, int dt, gpu_stream_t stream);

/* Replaces npu_rope_layer (prebuild/npu_ops.h:39-42): rotates Q and K
 * ([cur_size][n_heads][hidden_dim/n_heads] each) with table rows
 * start_pos .. start_pos+cur_size-1.  freqs_cis is fp32 [max_seq][D/2][2] =
 * (cos, sin) as built by ModelBase::InitFreqCIS (src/model_base.cpp:27-83).
 * Pairs are (2f, 2f+1), or (f, f+D/2) when is_neox_style != 0
 * (tests/rope_single_layer_test.cpp:86-91).  Results are bit-identical to the
 * reference tests' golden: fp32 products, one subtraction / addition, one
 * rounding to the dtype. */
int gpu_rope_layer(void *output_q_dev, void *output_k_dev, const void *freqs_cis_dev,
                   const void *input_q_dev, const void *input_k_dev, int start_pos,
                   int cur_size, int n_heads, int hidden_dim, int is_neox_style, int dt,
                   gpu_stream_t stream);

/* Replaces npu_rope_single_layer (prebuild/npu_ops.h:44-47); hidden_dim is
 * n_heads*head_dim of the tensor being rotated (src/llama2_layer_npu.cpp:790-798). */
int gpu_rope_single_layer(void *output_x_dev, const void *freqs_cis_dev,
                          const void *input_x_dev, int start_pos, int cur_size, int n_heads,
                          int hidden_dim, int is_neox_style, int dt, gpu_stream_t stream);

/* Replaces npu_split_qkv_layer (prebuild/npu_ops.h:27-30; declared there, not
 * called by the reference's layers): input_qkv [batch][q_dim + k_dim + v_dim]
 * is split row by row into three dense tensors.  Each dim must be a multiple
 * of 128 elements.  A plain copy: bit-exact. */
int gpu_split_qkv_layer(void *output_q_dev, void *output_k_dev, void *output_v_dev,
                        const void *input_qkv, int batch, int q_dim, int k_dim, int v_dim,
                        int dt, gpu_stream_t stream);

/* ------------------------------------------------------------------------
 * Fused operators: the same path with a batch dimension, explicit strides
 * (token-major and head-major caches) and RoPE + append in the same pass.
 * ------------------------------------------------------------------------ */

/* Geometry shared by the fused operators.  All strides are in ELEMENTS.
 *   q / out element (seq b, token t, head h, d):  b*seq_stride + t*tok_stride + h*head_dim + d
 *   raw k / v input element (b, t, kv_head, d):   b*kv_in_seq_stride + t*kv_in_tok_stride + kv_head*head_dim + d
 *   cache element (b, kv_head, pos, d):           b*cache_seq_stride + kv_head*cache_head_stride + pos*cache_pos_stride + d
 * The K and V caches have the same geometry.  Token-major (reference) cache:
 * head_stride = head_dim, pos_stride = n_kv_heads*head_dim.  Head-major cache
 * [kv_head][max_pos][head_dim]: head_stride = max_pos*head_dim, pos_stride = head_dim.
 * cache_pos_stride and cache_head_stride must be multiples of 8 elements. */
typedef struct gpu_attn_desc {
  int32_t dtype;         /* GPU_DT_FLOAT16 / GPU_DT_BFLOAT16 */
  int32_t batch;         /* independent sequences */
  int32_t n_heads;       /* query heads = n_kv_heads * group size */
  int32_t n_kv_heads;
  int32_t head_dim;      /* 128 */
  int32_t is_neox_style; /* RoPE pairing */
  int64_t q_seq_stride, q_tok_stride;
  int64_t kv_in_seq_stride, kv_in_tok_stride;
  int64_t out_seq_stride, out_tok_stride;
  int64_t cache_seq_stride, cache_head_stride, cache_pos_stride;
  int64_t total_kv_len;  /* scheduling hint for gpu_attn_decode_layer: sum over the batch of the cache
                            positions the call reads per KV head (kv_len[b] + append_new); 0 = unknown.
                            Only the split size depends on it, never the result's meaning. */
} gpu_attn_desc;

/* RoPE(Q) -> q_out, RoPE(K) -> k_cache, V -> v_cache for m new tokens of every
 * sequence, in one pass.  Fuses npu_rope_layer / 2 x npu_rope_single_layer with
 * the two cache-append copies (src/llama2_layer_npu.cpp:284, :325-338;
 * :790-798, :830-843).  start_pos_dev: int32 [batch], tokens already cached
 * (= table row of the first new token); if NULL, `start_pos` is used for all.
 * q_out may alias q_in. */
int gpu_rope_kv_append_layer(const gpu_attn_desc *desc, void *q_out, void *k_cache,
                             void *v_cache, const void *q_in, const void *k_in,
                             const void *v_in, const void *freqs_cis_dev,
                             const int32_t *start_pos_dev, int start_pos, int m,
                             gpu_stream_t stream);

/* The same pass fed from a FUSED projection output: each token row holds
 * [n_heads*128 q | n_kv_heads*128 k | n_kv_heads*128 v] (row stride
 * qkv_tok_stride >= that width, sequence stride qkv_seq_stride, in elements).
 * qkv_bias: one row of the same width and dtype, or NULL.  With a bias every
 * element becomes round_dtype(float(x) + float(bias)) before the rotation -- the
 * rounding point of a projection whose epilogue adds the bias
 * (npu_matmul_bias_nz_layer, prebuild/npu_ops.h:90-92, used by the Qwen2
 * q/k/v projections, src/llama2_layer_npu.cpp:1020-1055, :1174-1177).
 * Replaces npu_split_qkv_layer (prebuild/npu_ops.h:27-30) + the two RoPE calls
 * + the two cache copies with one read of the row.  q_out is written with the
 * descriptor's q strides; the descriptor's kv_in strides are not used. */
int gpu_qkv_rope_kv_append_layer(const gpu_attn_desc *desc, void *q_out, void *k_cache,
                                 void *v_cache, const void *qkv_in, int64_t qkv_seq_stride,
                                 int64_t qkv_tok_stride, const void *qkv_bias,
                                 const void *freqs_cis_dev, const int32_t *start_pos_dev,
                                 int start_pos, int m, gpu_stream_t stream);

/* output[r][c] = round_dtype(float(input[r][c]) + float(bias[c])) for rows x width
 * elements, rows row_stride elements apart in both tensors (in place allowed);
 * width a multiple of 128.  The bias step of gpu_qkv_rope_kv_append_layer on
 * its own, for the one-token step, where the rotation happens inside
 * gpu_attn_decode_layer.  No counterpart in prebuild/npu_ops.h: the reference
 * adds the bias inside its projection (npu_matmul_bias_nz_layer, :90-92). */
int gpu_bias_add_layer(void *output_dev, const void *input_dev, const void *bias_dev, int rows,
                       int width, int64_t row_stride, int dt, gpu_stream_t stream);

/* Causal attention of m new (already rotated) query rows per sequence over
 * cache positions [0, offset + m); row r sees positions <= offset + r.  The
 * batched, strided form of gpu_flash_attn_gqa_layer. */
int gpu_attn_prefill_layer(const gpu_attn_desc *desc, void *out, const void *q,
                           const void *k_cache, const void *v_cache, int m, int offset,
                           gpu_stream_t stream);

/* One fused decode step for every sequence: rotate the new token's Q and K,
 * append K and V at cache position kv_len[b], attend over positions
 * [0, kv_len[b]] with the cache split into chunks, merge the chunks.
 *   q_in [batch][n_heads][D], k_in/v_in [batch][n_kv_heads][D]: raw (unrotated)
 *   kv_len_dev   int32 [batch]: tokens already in the cache of sequence b
 *   rope_pos_dev int32 [batch] or NULL: table row used for the rotation
 *                (NULL: kv_len[b]); differs from kv_len when the cache holds
 *                only a slice of the sequence
 *   append_new   1: append and attend to the new token; 0: attend to
 *                [0, kv_len[b]) only and leave the cache untouched (k_in/v_in
 *                may be NULL)
 *   max_kv_len   host upper bound of kv_len[b] + append_new over the batch (sizes the grid)
 *   workspace    device scratch of at least gpu_attn_decode_workspace_bytes()
 * Output: out [batch][n_heads*D] in the dtype; if o_partial/lse_partial are not
 * NULL the kernel instead writes the normalised fp32 result [batch][n_heads][D]
 * and its log-sum-exp [batch][n_heads] (natural log; -inf for an empty slice),
 * for a merge across devices with gpu_attn_merge_lse_layer. */
int gpu_attn_decode_layer(const gpu_attn_desc *desc, void *out, float *o_partial,
                          float *lse_partial, const void *q_in, const void *k_in,
                          const void *v_in, void *k_cache, void *v_cache,
                          const void *freqs_cis_dev, const int32_t *kv_len_dev,
                          const int32_t *rope_pos_dev, int append_new, int max_kv_len,
                          void *workspace, size_t workspace_bytes, gpu_stream_t stream);

/* The same fused decode step for callers that may not allocate device memory
 * (no counterpart in the reference: its operators leave allocation to the
 * caller's pool, src/device_npu.cpp:22-67).  Some hosts cannot call cudaMalloc
 * when a decode step runs: a serving process that reserved all of the GPU's
 * memory for its own KV-cache pool at start-up, a plug-in slot that must not
 * allocate after initialisation, a latency-critical loop that cannot afford
 * cudaMalloc's device-wide synchronisation.  They have no way to supply
 * gpu_attn_decode_layer's workspace.  This entry point
 * needs none: its split-KV scratch is a fixed 16 MiB array in the library's own
 * device image.  It calls no cudaMalloc / cudaFree and no allocating routine.
 *   - Splits are always 512 positions; a call needs batch * n_heads *
 *     ceil(max_kv_len / 512) * 516 bytes of scratch and is rejected with
 *     GPU_OPS_E_WORKSPACE (nothing launched) when that exceeds 16 MiB.
 *   - The array's device address is looked up on the first use per device (with
 *     that device current), by gpu_attn_decode_noalloc_prepare() or by the first
 *     call of the entry point.  With CUDA's lazy module loading that look-up is
 *     also when the device takes the 16 MiB, which it then holds until the
 *     process exits: do it at start-up, BEFORE the host reserves the rest of the
 *     device memory and before any stream capture (or run with
 *     CUDA_MODULE_LOADING=EAGER, which takes the memory when the library loads).
 *   - All calls on a device share the array, which keeps the previous call's
 *     contents; nothing in it needs clearing, but calls whose kernels overlap on
 *     the GPU race on it: order them on one stream or with events.
 * Arguments as gpu_attn_decode_layer, without the partial outputs and workspace. */
int gpu_attn_decode_noalloc_prepare(void);
int gpu_attn_decode_layer_noalloc(const gpu_attn_desc *desc, void *out, const void *q_in,
                                  const void *k_in, const void *v_in, void *k_cache,
                                  void *v_cache, const void *freqs_cis_dev,
                                  const int32_t *kv_len_dev, const int32_t *rope_pos_dev,
                                  int append_new, int max_kv_len, gpu_stream_t stream);

/* Scratch bytes gpu_attn_decode_layer needs for this geometry and bound. */
size_t gpu_attn_decode_workspace_bytes(const gpu_attn_desc *desc, int max_kv_len);

/* ------------------------------------------------------------------------
 * Planned decode.  The reference's generation loop knows every cache length on
 * the host (InferenceCtx::cur_pos / prev_pos, src/model_base.hpp:40-48, passed
 * to the operators as the host integers m, n, offset); with a batch of
 * sequences the host passes them as an array and the library cuts the step's
 * work ONCE: all (sequence, KV head) caches laid end to end in 64-position
 * tiles, one contiguous equally expensive share per CTA.  The plan is the same
 * for every layer of the step.  The planned entry point runs the same fused
 * step as gpu_attn_decode_layer on persistent CTAs whose K/V tiles arrive by
 * TMA, so that the SMs finish together whatever the individual lengths are.
 *
 *   1. gpu_attn_decode_plan(desc, kv_len_host, append_new, 0, plan_host, bytes)
 *      fills plan_host (host memory of gpu_attn_decode_plan_bytes(desc, 0) bytes;
 *      pinned if it is to be copied asynchronously);
 *   2. the caller copies gpu_attn_decode_plan_size(plan_host) bytes to device
 *      memory (16-byte aligned), ordered before the layers on the stream;
 *   3. gpu_attn_decode_planned_layer(...) once per layer, with scratch of
 *      gpu_attn_decode_plan_workspace_bytes(plan_host) bytes.
 * Only desc->batch, n_heads, n_kv_heads matter to the plan.  n_ctas: 0 = three
 * quarters of the CTAs the current device holds at once (the rest of the slots
 * lets the next call's CTAs move in early); a positive value (<= 1024) fixes it.
 * ------------------------------------------------------------------------ */
size_t gpu_attn_decode_plan_bytes(const gpu_attn_desc *desc, int n_ctas);
int gpu_attn_decode_plan(const gpu_attn_desc *desc, const int32_t *kv_len_host, int append_new, int n_ctas,
                         void *plan_host, size_t plan_bytes);
size_t gpu_attn_decode_plan_size(const void *plan_host);
size_t gpu_attn_decode_plan_workspace_bytes(const void *plan_host);

/* One fused decode step driven by a plan: arguments as gpu_attn_decode_layer,
 * with the lengths, append_new and the bound taken from the plan (plan_host: the
 * host copy, read during the call; plan_dev: the device copy, read by the
 * kernels; one upload serves every layer of the step).  pages: NULL for a flat cache, else the page description and
 * k_cache / v_cache are the pools.  Sequences with an empty cache and no new
 * token get a zero output (log-sum-exp -inf).  Honours
 * gpu_attn_set_decode_early_prefetch, whose condition then also covers the
 * device copy of the plan and the page table. */
int gpu_attn_decode_planned_layer(const gpu_attn_desc *desc, const struct gpu_kv_pages *pages,
                                  const void *plan_host, const void *plan_dev, void *out,
                                  float *o_partial, float *lse_partial, const void *q_in,
                                  const void *k_in, const void *v_in, void *k_cache, void *v_cache,
                                  const void *freqs_cis_dev, const int32_t *rope_pos_dev,
                                  void *workspace, size_t workspace_bytes, gpu_stream_t stream);

/* ------------------------------------------------------------------------
 * Cross-device split-KV decode: exchange and merge of the ranks' partials in
 * ONE kernel over NVLink peer memory (plain peer stores, system-scope fence,
 * flags; no collective library call).  The reference is single-device and has
 * no counterpart.
 *
 * Every rank owns one exchange buffer of gpu_attn_xchg_buffer_bytes(world, rows)
 * bytes, zero-filled, visible to its peers (gpu_peer_buffer_alloc / _open, CUDA
 * IPC; one process per GPU).  Per decode step (epoch = 1, 2, 3, ... identical on
 * all ranks): gpu_attn_decode_layer writes this rank's partial to
 * gpu_attn_xchg_local_slot(...) (o_partial = the returned pointer, lse_partial =
 * that + rows*head_dim), then gpu_attn_xchg_merge_layer copies it into every
 * peer's buffer, waits (bounded: about a second, then gpu_ops_kernel_status()
 * turns non-zero and the output is left unwritten) for the peers' partials of
 * the same epoch and merges them: out [rows][head_dim], every rank gets the
 * full result, bit-identical to all-gather + gpu_attn_merge_packed_layer.
 * Consecutive epochs use the two halves of the buffer alternately; a rank may
 * run at most one step ahead of its slowest peer, which the protocol enforces.
 * ------------------------------------------------------------------------ */
size_t gpu_attn_xchg_buffer_bytes(int world, int rows);
float *gpu_attn_xchg_local_slot(void *local_buffer, int world, int rank, uint32_t epoch, int rows);
/* peer_buffers: host array [world] of device addresses of the ranks' buffers as
 * mapped in THIS process (entry [rank] is not used). */
int gpu_attn_xchg_merge_layer(void *out, void *local_buffer, void *const *peer_buffers, int world,
                              int rank, uint32_t epoch, int rows, int head_dim, int dt,
                              gpu_stream_t stream);

/* gpu_attn_decode_layer and gpu_attn_xchg_merge_layer as one call of two launches:
 * the decode kernel leaves this rank's partial split along the cache in the
 * workspace, and the exchange kernel merges a row's splits, pushes the row to
 * the peers and merges the ranks' rows -- one launch less than decode + local
 * merge + exchange, same bits.  Arguments as for the two functions. */
int gpu_attn_decode_xchg_layer(const gpu_attn_desc *desc, void *out, const void *q_in,
                               const void *k_in, const void *v_in, void *k_cache, void *v_cache,
                               const void *freqs_cis_dev, const int32_t *kv_len_dev,
                               const int32_t *rope_pos_dev, int append_new, int max_kv_len,
                               void *workspace, size_t workspace_bytes, void *local_buffer,
                               void *const *peer_buffers, int world, int rank, uint32_t epoch,
                               gpu_stream_t stream);

/* Device memory that other processes of the node can map: cudaMalloc + zero
 * fill + IPC export (handle64: 64 bytes to hand to the peers), import, unmap,
 * free.  Allocation helpers, not operators: call them at start-up. */
int gpu_peer_buffer_alloc(size_t bytes, void **ptr, unsigned char *handle64);
int gpu_peer_buffer_open(const unsigned char *handle64, void **ptr);
int gpu_peer_buffer_close(void *ptr);
int gpu_peer_buffer_free(void *ptr);

/* ------------------------------------------------------------------------
 * Paged KV cache.  The reference allocates one flat block per layer
 * (src/llama2_layer_npu.cpp:1148-1149); for batched serving the cache is a
 * pool of fixed-size pages and a per-sequence page table instead.
 * ------------------------------------------------------------------------ */

/* Position pos of sequence b lives in page page_table[b*table_stride + pos/page_size]
 * of the pool, at in-page position pos % page_size.  Inside a page the
 * descriptor's cache_head_stride / cache_pos_stride apply (head-major page
 * [kv_head][page_size][D]: head stride page_size*D, position stride D);
 * cache_seq_stride is not used.  page_size: a power of two >= 64.  All strides
 * in elements.  Pages named by the table for positions the call touches must
 * exist; the table is read by the kernels, never written. */
typedef struct gpu_kv_pages {
  const int32_t *page_table; /* device, int32 [batch][table_stride] */
  int32_t table_stride;
  int32_t page_size;
  int64_t page_stride;       /* elements between consecutive pages of the pool */
  int32_t n_pages;           /* pages in the pool (every table entry the call uses is below it) */
  int32_t reserved;          /* 0 */
} gpu_kv_pages;

/* gpu_rope_kv_append_layer writing K and V through the page table. */
int gpu_rope_kv_append_paged_layer(const gpu_attn_desc *desc, const gpu_kv_pages *pages,
                                   void *q_out, void *k_pool, void *v_pool, const void *q_in,
                                   const void *k_in, const void *v_in, const void *freqs_cis_dev,
                                   const int32_t *start_pos_dev, int start_pos, int m,
                                   gpu_stream_t stream);

/* gpu_attn_prefill_layer over a paged cache.  The tcgen05 kernel reads K and V in
 * tiles of 128 positions and so needs pages of at least 128; smaller pages run
 * on the mma.sync kernel. */
int gpu_attn_prefill_paged_layer(const gpu_attn_desc *desc, const gpu_kv_pages *pages, void *out,
                                 const void *q, const void *k_pool, const void *v_pool, int m,
                                 int offset, gpu_stream_t stream);

/* gpu_attn_decode_layer over a paged cache (final output only; same workspace
 * sizing, same split and merge kernels; the page of position kv_len[b] must be
 * in the table when append_new is set). */
int gpu_attn_decode_paged_layer(const gpu_attn_desc *desc, const gpu_kv_pages *pages, void *out,
                                const void *q_in, const void *k_in, const void *v_in,
                                void *k_pool, void *v_pool, const void *freqs_cis_dev,
                                const int32_t *kv_len_dev, int append_new, int max_kv_len,
                                void *workspace, size_t workspace_bytes, gpu_stream_t stream);

/* Merge n_parts partial results: o_parts fp32 [n_parts][rows][head_dim]
 * (normalised), lse_parts fp32 [n_parts][rows] (natural log).
 * out[row] = sum_p exp(lse_p - M) o_p / sum_p exp(lse_p - M), M = max_p lse_p,
 * written in the dtype as [rows][head_dim]. */
int gpu_attn_merge_lse_layer(void *out, const float *o_parts, const float *lse_parts,
                             int n_parts, int rows, int head_dim, int dt,
                             gpu_stream_t stream);

/* The same merge on the receive buffer of an all-gather: part p (one per rank)
 * is one contiguous block of rows*(head_dim+1) floats, first the rows*head_dim
 * normalised outputs, then the rows log-sum-exps -- what a rank gets when it
 * points gpu_attn_decode_layer's o_partial at its send buffer and lse_partial
 * at send buffer + rows*head_dim.  The partial (O, LSE) exchange has no
 * counterpart in the reference, which is single-device. */
int gpu_attn_merge_packed_layer(void *out, const float *parts, int n_parts, int rows, int head_dim,
                                int dt, gpu_stream_t stream);

/* Scratch for the reference-shaped attention operators on the CURRENT device.
 * They take no workspace argument (the reference's signatures have none) and
 * never allocate; with scratch registered, decode-shaped calls (m * group_size
 * <= 16) split long caches across CTAs, without it they run unsplit.  The
 * library keeps the pointer, not the memory: pass NULL before freeing it.
 * Calls that share the scratch must be ordered on one stream. */
int gpu_ops_set_workspace(void *workspace, size_t bytes);

/* 1: gpu_attn_decode_layer (flat or paged) requests its first K/V tiles BEFORE
 * the kernels that precede it on the stream have finished, which hides its
 * start-up latency behind their tail.  Allowed when neither kv_len_dev nor the
 * cache rows below kv_len[b] of a call are written by the TWO kernels preceding
 * it on the stream -- the case when consecutive calls work on different layers'
 * caches and the lengths change once per step.  Everything else the call reads
 * (q, the new token, the scratch) is still ordered after those kernels.
 * Process-wide, off by default. */
int gpu_attn_set_decode_early_prefetch(int on);

/* Positions per split used by gpu_attn_decode_layer; 0 restores the built-in
 * choice.  A multiple of 64.  Process-wide tuning knob. */
int gpu_attn_set_decode_chunk(int positions);

/* Which kernel gpu_attn_prefill_layer and the reference-shaped operators use
 * for rows beyond the small-m path: 0 = automatic, 1 = mma.sync kernel,
 * 2 = tcgen05 kernel, one CTA per 256 query rows, 3 = tcgen05 kernel in
 * persistent form (one CTA per SM that takes work items from a counter, output
 * through a TMA tensor store; same bits as 2, measured slower, opt-in only; not
 * on a capturing stream; its first call on a device allocates 2 KB of counters).  Automatic = 2, else 1 where the tensor maps cannot
 * describe the geometry.  Process-wide; for tests and measurements. */
int gpu_attn_set_prefill_kernel(int which);

/* The tcgen05 prefill kernel starts its CTAs chunk by chunk of (sequence, head)
 * pairs, and inside a chunk the longest row block of every pair first, so that
 * the last CTAs to start are the shortest while a chunk's K and V stay in L2
 * together.  bytes = the K/V a chunk may hold (0 restores the built-in 40 MB,
 * chosen for the 126 MB L2 of a B200).  Results do not depend on it.
 * Process-wide tuning knob. */
int gpu_attn_set_prefill_l2_window(size_t bytes);

/* Which kernel served the calling thread's last prefill-shaped call: 1 = mma.sync
 * kernel, 2 = tcgen05 kernel, 3 = persistent tcgen05 kernel, 0 = none yet.  The automatic choice falls back to
 * the mma.sync kernel when the tcgen05 kernel's tensor maps cannot describe a
 * geometry (a stride that is no multiple of 16 bytes, pages below 128
 * positions); a caller that counts on the faster kernel can check here. */
int gpu_attn_last_prefill_kernel(void);

/* 0, or the code a kernel on the current device recorded: every device-side
 * wait (mbarrier polls, flags of other ranks) is bounded to about a second,
 * after which the kernel stores a code (1 .. 39) here, ends normally and leaves
 * the context usable; 40 = a sequence of gpu_attn_decode_layer was longer than
 * max_kv_len, so that its last positions -- the new token among them -- were not
 * covered (the output and cache of that sequence are wrong, nothing is read or
 * written out of bounds).  Read it after synchronising. */
int gpu_ops_kernel_status(void);
/* Resets that status to 0 (call with no kernel of the library in flight on the device). */
int gpu_ops_clear_kernel_status(void);

/* Number of kernels launched by this library on the calling thread since the
 * last call with reset != 0. */
long gpu_ops_launch_count(int reset);

/* Description of the last non-zero status returned on the calling thread. */
const char *gpu_ops_last_error_string(void);

#ifdef __cplusplus
}
#endif
#endif /* LLM_SIMPLE_GPU_OPS_H_ */
