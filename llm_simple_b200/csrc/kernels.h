// Host-visible parameter blocks and launchers of the CUDA kernels.  Internal to
// the library: the public surface is include/gpu_ops.h.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200attn {

// Record the message gpu_ops_last_error_string() returns on the calling thread.
void set_last_error(const char *msg);
// Add to the calling thread's gpu_ops_launch_count().
void add_launch_count(int launches);

// ---- paged KV cache --------------------------------------------------------
// Optional indirection of cache positions: with table != nullptr, position pos of
// sequence b lives in page table[b * table_stride + (pos >> page_shift)] of a pool of
// pages page_stride elements apart, at in-page position pos & ((1 << page_shift) - 1);
// the geometry's head / position strides then address inside a page and its sequence
// stride is not used.  Pages hold a power of two >= 64 positions, so that a tile of 64
// (decode) never straddles two pages.
struct KvPaging {
  const int32_t *table;
  long page_stride;
  int table_stride;
  int page_shift;
  int n_pages; // pages in the pool
};

// ---- RoPE + append ---------------------------------------------------------
// One of up to three tensors handled by a rope_append launch (Q, K, V).
struct RopeStream {
  const void *src; // [batch][m][heads][128], strides below
  void *dst;
  int heads;       // 0 disables the stream
  int rotate;      // 1: apply RoPE, 0: copy
  int dst_at_pos;  // 1: destination token index is start_pos + t (cache), 0: t
  const void *bias; // [heads][128] of the element type added before the rotation, or null
  long src_seq, src_tok;
  long dst_seq, dst_tok, dst_head;
};

struct RopeParams {
  RopeStream s[3];
  const float *freqs_cis; // [max_seq][64][2]
  const int32_t *start_pos_dev;
  int start_pos;
  int batch, m, slots; // slots = sum of heads
  int is_neox;
  KvPaging pg;         // applies to the streams with dst_at_pos
};

cudaError_t launch_rope_append(const RopeParams &p, bool bf16, cudaStream_t stream);

// ---- attention (shared geometry) -------------------------------------------
struct AttnGeom {
  int batch, n_heads, n_kv_heads, group;
  long q_seq, q_tok;       // rotated or raw q
  long out_seq, out_tok;
  long c_seq, c_head, c_pos; // cache strides (K and V alike)
};

// ---- small-m / decode kernel (split-KV, mma.sync) ----------------------------
struct DecodeParams {
  AttnGeom g;
  void *out;            // dtype [batch][m][H*128] (strided) when final
  float *o_partial;     // optional fp32 final [batch*m*H][128] + lse_partial (natural log)
  float *lse_partial;
  const void *q;        // raw (rotate_q) or rotated
  const void *k_new;    // raw new-token K/V (append)
  const void *v_new;
  long kv_in_seq;       // stride between sequences of k_new / v_new
  void *k_cache;
  void *v_cache;
  const float *freqs_cis;
  const int32_t *kv_len_dev; // tokens already cached per sequence, or NULL
  const int32_t *rope_pos_dev;
  int kv_len;           // used when kv_len_dev == NULL
  int m;                // query tokens per sequence; m * group <= 16
  int offset;           // causal: row r sees positions < min(total, offset + r + 1); <0 disables
  int append;           // 1: rotate + append the new token (m == 1)
  int rotate_q;
  int is_neox;
  int chunk;            // positions per split (multiple of 64)
  int max_splits;       // grid.x
  float *ws_o;          // [rows][max_splits][128] fp32, rows = batch*m*H
  float *ws_lse;        // [rows][max_splits] (log2 domain)
  float scale_log2;
  KvPaging pg;
  int early_kv;         // 1: fetch the first K/V tiles before waiting for the preceding kernels
  int no_merge;         // 1: leave the split partials in (ws_o, ws_lse); the caller merges them
  int *error_flag;      // status word (host-mapped), or NULL
};

// Status codes the kernels store in the host-visible status word (besides the codes of waits that
// gave up): a sequence was longer than the bound the launch was sized for.
constexpr int kStatusLengthBeyondBound = 40;

cudaError_t launch_attn_decode(const DecodeParams &p, bool bf16, cudaStream_t stream, int *launches);

// merge of split results held in (ws_o, ws_lse); also used for cross-device parts
struct MergeParams {
  void *out;               // dtype, element (row, d) at row_off(row) + d; may be NULL
  float *o_partial;        // fp32 [rows][128] or NULL
  float *lse_partial;      // natural log
  const float *parts_o;    // [rows][max_parts][128] (part_major == 0) or part i at parts_o + i*part_stride_o
  const float *parts_lse;
  int part_major;
  long part_stride_o, part_stride_lse; // part_major: elements between consecutive parts
  int lse_is_log2;         // workspace partials are in the log2 domain
  int rows, max_parts;
  // number of valid parts per row: fixed n_parts, or ceil(total_b / chunk)
  int n_parts;
  const int32_t *kv_len_dev;
  int kv_len, append, chunk;
  int rows_per_seq;        // m * H
  int n_heads, m;
  long out_seq, out_tok;   // output strides
};

cudaError_t launch_attn_merge(const MergeParams &p, bool bf16, cudaStream_t stream);

// ---- planned decode (persistent CTAs, TMA-fed ring) -------------------------------
// The host cuts the step's work -- every (sequence, KV head) cache laid end to end in tiles of
// 64 positions -- into one contiguous, equally expensive share per CTA and stores the result as a
// "plan": a blob of 32-bit words that is identical in host and device memory.
//   header (PlanHeader) | cta_begin[n_ctas + 1] | items[n_items] | groups[n_groups]
// CTA c works through items [cta_begin[c], cta_begin[c + 1]).  A cache that was cut leaves one
// partial result per piece in consecutive scratch slots; its pieces form a merge group.
constexpr uint32_t kPlanMagic = 0x504c414eu; // "PLAN"

struct PlanHeader { // 64 bytes
  uint32_t magic;
  int32_t n_ctas, n_items, n_groups;
  int32_t n_slots;       // partial-result slots the plan uses (scratch = n_slots * group * 129 floats)
  int32_t batch, n_kv_heads, group;
  int32_t append;        // 1: every sequence gets its new token appended at kv_len[b]
  int32_t max_total;     // max over the batch of kv_len[b] + append
  int32_t off_cta_begin, off_items, off_groups; // byte offsets from the start of the blob
  int32_t total_bytes;
  int32_t total_tiles;
  int32_t max_parts;     // pieces of the most-cut cache
};
static_assert(sizeof(PlanHeader) == 64, "plan header layout");

struct PlanItem { // 32 bytes: one contiguous piece of one (sequence, KV head) cache
  int32_t b, kvh;
  int32_t pos0, pos_end; // cache positions [pos0, pos_end); pos0 a multiple of 64; the new token counts when it falls inside
  int32_t len_old;       // tokens cached before this step
  int32_t slot;          // >= 0: the piece is one of several, its partial result goes to this slot; -1: it is the whole cache
  int32_t has_new;       // 1: the piece contains position len_old, the token appended by this step
  int32_t reserved;
};
static_assert(sizeof(PlanItem) == 32, "plan item layout");

struct PlanGroup { // 16 bytes: the pieces of one cut (sequence, KV head) cache, slots first_slot .. first_slot + n_parts - 1
  int32_t first_slot, n_parts;
  int32_t b, kvh;
};
static_assert(sizeof(PlanGroup) == 16, "plan group layout");

struct PlannedDecodeParams {
  AttnGeom g;
  void *out;            // dtype [batch][H*128] (strided), or NULL with the partial pair below
  float *o_partial;     // fp32 [batch*H][128] + lse_partial (natural log), for a merge across devices
  float *lse_partial;
  const void *q;        // raw query rows, rotated here
  const void *k_new;    // raw new-token K / V (plan built with append)
  const void *v_new;
  long kv_in_seq;
  void *k_cache;
  void *v_cache;
  const float *freqs_cis;
  const int32_t *rope_pos_dev; // table row per sequence, or NULL: the cached length
  int is_neox;
  float scale_log2;
  const unsigned char *plan;   // the blob in device memory
  int n_ctas, n_groups, n_slots, max_total, max_parts;
  int off_cta_begin, off_items, off_groups;
  float *ws_o;          // [n_slots][group][128] fp32 (normalised partial outputs)
  float *ws_lse;        // [n_slots][group] (log2 domain)
  KvPaging pg;
  int early_kv;         // 1: K/V tiles may be requested before the preceding kernels have finished
  int *error_flag;
};

cudaError_t launch_attn_decode_planned(const PlannedDecodeParams &p, bool bf16, cudaStream_t stream, int *launches);

// Host-side plan builder (decode_plan.cpp).  kv_len: tokens cached per sequence (host memory).
// n_ctas: CTAs to cut the work for.  Returns the
// number of bytes written to `blob`, or 0 if `capacity` is too small / the arguments are invalid.
size_t decode_plan_capacity(int batch, int n_kv_heads, int n_ctas);
size_t build_decode_plan(void *blob, size_t capacity, const int32_t *kv_len, int batch, int n_kv_heads, int group,
                         int append, int n_ctas);
// CTAs of attn_decode_tma_kernel that the current device can hold at once; 0 on failure.
int decode_planned_max_ctas();

// ---- general causal attention (mma.sync, any m/n/offset) -----------------------
struct PrefillParams {
  AttnGeom g;
  void *out;
  const void *q; // rotated
  const void *k_cache;
  const void *v_cache;
  int m, n, offset;
  float scale_log2;
  KvPaging pg;    // tcgen05 kernel: pages of at least 128 positions
  long l2_window; // tcgen05 kernel: bytes of K and V a chunk of (sequence, head) pairs may share in L2; 0 = default
};

cudaError_t launch_attn_prefill_mma(const PrefillParams &p, bool bf16, cudaStream_t stream);

// tcgen05 / TMEM / TMA kernel; same contract.  Returns cudaErrorNotSupported if
// the geometry cannot be described by its tensor maps.
cudaError_t launch_attn_prefill_tc5(const PrefillParams &p, bool bf16, cudaStream_t stream);
// The same kernel in persistent form (one CTA per SM, work items handed out through a counter in
// global memory, epilogue through a TMA tensor store); same contract.  Also returns
// cudaErrorNotSupported on a capturing stream.
cudaError_t launch_attn_prefill_tc5p(const PrefillParams &p, bool bf16, cudaStream_t stream);
// Tensor maps are pure functions of (base, geometry): a small per-thread cache of the most recent
// ones saves the driver call on repeated launches (a layer calls with the same buffers every step).
struct TensorMapKey {
  const void *base;
  uint64_t n1, n2, n3;
  long s1, s2, s3;
  uint32_t box1, box2, bf16, pad; // no padding bytes: compared with memcmp
};
// Non-zero once a bounded wait inside a kernel on the current device has given up.
int attn_tc5_error_status();
void attn_clear_error_status();
// Device address of that status word (host-mapped), or nullptr.
int *kernel_error_word_dev();

// ---- cross-device (O, LSE) exchange + merge over peer memory ------------------
constexpr int kMaxPeers = 8;
struct XchgParams {
  void *out;                      // dtype [rows][128]
  const float *slots;             // local buffer half of this step: [world][rows*129] fp32
  const uint32_t *flags;          // local flags of this step's half: [world]
  float *peer_slot[kMaxPeers];    // this rank's slot inside peer p's buffer half
  uint32_t *peer_flag[kMaxPeers]; // this rank's flag inside peer p's buffer half
  uint32_t epoch;                 // step counter, never 0
  int world, rank, rows;
  int *error_flag;
  // Optional: this rank's partial is still split along the cache (decode kernel launched with
  // no_merge): [rows][max_splits][128] fp32 + [rows][max_splits] log2-domain log-sum-exps; the
  // kernel merges the splits of a row, pushes the row to the peers and goes on to the final merge.
  const float *ws_o, *ws_lse;
  int max_splits, chunk, append, rows_per_seq;
  const int32_t *kv_len_dev;
};
cudaError_t launch_attn_xchg_merge(const XchgParams &p, bool bf16, cudaStream_t stream);

} // namespace b200attn
