// C ABI of libgpu_ops.so (declared in include/gpu_ops.h): argument validation
// on the host, geometry set-up and kernel dispatch.  No entry point allocates
// device memory.
#include "gpu_ops.h"
#include "kernels.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <string>
#include <cstdlib>
#include <cstring>

using namespace b200attn;

namespace {

thread_local std::string g_last_error;
thread_local long g_launches = 0;
thread_local int g_last_prefill_kernel = 0; // 1 mma.sync, 2 tcgen05, 3 tcgen05 persistent
std::atomic<int> g_decode_chunk{0};
std::atomic<int> g_prefill_kernel{0};
std::atomic<long> g_prefill_l2_window{0};
std::atomic<int> g_decode_early{0};

// caller-registered scratch for the reference-shaped operators, per device
struct RegisteredWorkspace {
  void *ptr = nullptr;
  size_t bytes = 0;
};
std::mutex g_ws_mutex;
RegisteredWorkspace g_ws[64];

int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

int cuda_fail(cudaError_t e, const char *what) {
  return fail(GPU_OPS_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

bool dt_ok(int dt) { return dt == GPU_DT_FLOAT16 || dt == GPU_DT_BFLOAT16; }

int check_common(int dt, int head_dim) {
  if (!dt_ok(dt)) return fail(GPU_OPS_E_UNSUPPORTED, "dtype %d: only fp16 (4) and bf16 (5) are supported", dt);
  if (head_dim != 128) return fail(GPU_OPS_E_UNSUPPORTED, "head_dim %d: only 128 is supported", head_dim);
  return GPU_OPS_OK;
}

int check_desc(const gpu_attn_desc *d) {
  if (!d) return fail(GPU_OPS_E_INVALID, "desc is NULL");
  if (int rc = check_common(d->dtype, d->head_dim)) return rc;
  if (d->batch <= 0 || d->n_heads <= 0 || d->n_kv_heads <= 0 || d->n_heads % d->n_kv_heads)
    return fail(GPU_OPS_E_INVALID, "batch %d, n_heads %d, n_kv_heads %d", d->batch, d->n_heads, d->n_kv_heads);
  if (d->cache_pos_stride % 8 || d->cache_head_stride % 8 || d->cache_seq_stride % 8 || d->q_tok_stride % 8 ||
      d->q_seq_stride % 8 || d->kv_in_tok_stride % 8 || d->kv_in_seq_stride % 8 || d->out_tok_stride % 8 ||
      d->out_seq_stride % 8)
    return fail(GPU_OPS_E_INVALID, "strides must be multiples of 8 elements (16-byte accesses)");
  return GPU_OPS_OK;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

AttnGeom geom_from_desc(const gpu_attn_desc *d) {
  AttnGeom g{};
  g.batch = d->batch;
  g.n_heads = d->n_heads;
  g.n_kv_heads = d->n_kv_heads;
  g.group = d->n_heads / d->n_kv_heads;
  g.q_seq = d->q_seq_stride;
  g.q_tok = d->q_tok_stride;
  g.out_seq = d->out_seq_stride;
  g.out_tok = d->out_tok_stride;
  g.c_seq = d->cache_seq_stride;
  g.c_head = d->cache_head_stride;
  g.c_pos = d->cache_pos_stride;
  return g;
}

float scale_log2_of(int head_dim) {
  return (1.0f / sqrtf(static_cast<float>(head_dim))) * 1.4426950408889634f;
}

// Positions per split of the decode kernel.  total_len is the number of cache
// positions the call reads per KV head, summed over the batch (<= 0: unknown,
// taken as 5/8 of batch * max_len).  Two regimes, both measured on B200 with
// 148 SMs x 2 resident CTAs = 296 slots:
//   - the work fits one wave: the smallest split for which the expected CTA
//     count (full splits plus about half a ragged split per sequence and head)
//     stays within the slots -- no CTA waits for a slot and the merge stays small;
//   - otherwise about 1024 positions (512 KB of K+V) per CTA: per-CTA set-up and
//     pipeline fill cost about 3 us, so shorter splits lose more than they balance.
// The floor of 128 positions applies to calls too small to fill the GPU (one short sequence):
// they are bound by latency, and two tiles per CTA measured best there (7.0 us per layer at 640
// positions against 8.1 with 256 and 7.6 with 64).
constexpr int kMinChunk = 128;
int pick_chunk(int batch, int kv_heads, long total_len, int max_len) {
  const int forced = g_decode_chunk.load();
  if (forced > 0) return forced;
  const long slots = 296, fill = 256; // resident CTAs, and how many of them to aim for
  const long units = static_cast<long>(batch) * kv_heads;
  if (total_len <= 0) total_len = static_cast<long>(batch) * max_len * 5 / 8;
  const long positions = total_len * kv_heads; // over all (sequence, KV head) pairs
  long chunk = 1024;
  if (units / 2 < fill) {
    const long single = (positions + (fill - units / 2) - 1) / (fill - units / 2);
    if (single <= 1536 || units <= slots) chunk = single;
    // nearly whole sequences: do not split at all (no partials, no merge launch)
    if (units <= slots && single * 4 >= static_cast<long>(max_len) * 3) chunk = max_len;
  }
  chunk = ((chunk + 63) / 64) * 64;
  if (chunk < kMinChunk) chunk = kMinChunk;
  const long cap = ((static_cast<long>(max_len) + 63) / 64) * 64;
  if (chunk > cap) chunk = cap;
  return static_cast<int>(chunk);
}

size_t decode_ws_bytes(long rows, int splits) {
  return static_cast<size_t>(rows) * splits * (128 + 1) * sizeof(float);
}

// q rows handled by the split decode kernel: m * group <= 16
bool small_m(int m, int group) { return static_cast<long>(m) * group <= 16; }

int run_prefill(const PrefillParams &p, bool bf16, cudaStream_t stream) {
  const int which = g_prefill_kernel.load();
  cudaError_t e;
  if (which == 3) {   // opt-in: measured slower than the kernel below at every size tried
    e = launch_attn_prefill_tc5p(p, bf16, stream);
    if (e == cudaSuccess) {
      g_launches += 1;
      g_last_prefill_kernel = 3;
      return GPU_OPS_OK;
    }
    if (e != cudaErrorNotSupported || which == 3) return cuda_fail(e, "persistent tcgen05 prefill attention launch");
    (void)cudaGetLastError();
  }
  if (which != 1) {
    e = launch_attn_prefill_tc5(p, bf16, stream);
    if (e == cudaSuccess) {
      g_launches += 1;
      g_last_prefill_kernel = 2;
      return GPU_OPS_OK;
    }
    if (e != cudaErrorNotSupported || which == 2) return cuda_fail(e, "tcgen05 prefill attention launch");
    (void)cudaGetLastError();
  }
  e = launch_attn_prefill_mma(p, bf16, stream);
  if (e != cudaSuccess) return cuda_fail(e, "prefill attention launch");
  g_launches += 1;
  g_last_prefill_kernel = 1;
  return GPU_OPS_OK;
}

int ref_attention(void *out, const void *q, const void *k, const void *v, int m, int n, int offset, int group,
                  int kv_heads, int head_dim, int dt, gpu_stream_t stream) {
  if (int rc = check_common(dt, head_dim)) return rc;
  if (!out || !q || !k || !v) return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  if (m <= 0 || n <= 0 || offset < 0 || group <= 0 || kv_heads <= 0)
    return fail(GPU_OPS_E_INVALID, "m %d, n %d, offset %d, group_size %d, kv_head_num %d", m, n, offset, group,
                kv_heads);
  if (!aligned16(out) || !aligned16(q) || !aligned16(k) || !aligned16(v))
    return fail(GPU_OPS_E_INVALID, "tensor pointers must be 16-byte aligned");
  const bool bf16 = dt == GPU_DT_BFLOAT16;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  AttnGeom g{};
  g.batch = 1;
  g.n_kv_heads = kv_heads;
  g.group = group;
  g.n_heads = kv_heads * group;
  g.q_tok = g.out_tok = static_cast<long>(g.n_heads) * head_dim;
  g.q_seq = g.out_seq = 0;
  g.c_seq = 0;
  g.c_head = head_dim;
  g.c_pos = static_cast<long>(kv_heads) * head_dim;
  if (small_m(m, group)) {
    DecodeParams p{};
    p.g = g;
    p.out = out;
    p.q = q;
    p.k_cache = const_cast<void *>(k);
    p.v_cache = const_cast<void *>(v);
    p.kv_len = n;
    p.m = m;
    p.offset = offset;
    p.scale_log2 = scale_log2_of(head_dim);
    p.error_flag = kernel_error_word_dev();
    // split only if the caller registered scratch for this device
    p.chunk = ((n + 63) / 64) * 64;
    p.max_splits = 1;
    int dev = 0;
    cudaGetDevice(&dev);
    {
      std::lock_guard<std::mutex> lk(g_ws_mutex);
      if (dev >= 0 && dev < 64 && g_ws[dev].ptr) {
        const int chunk = pick_chunk(1, kv_heads, n, n);
        const int splits = (n + chunk - 1) / chunk;
        const long rows = static_cast<long>(m) * g.n_heads;
        if (splits > 1 && decode_ws_bytes(rows, splits) <= g_ws[dev].bytes) {
          p.chunk = chunk;
          p.max_splits = splits;
          p.ws_o = static_cast<float *>(g_ws[dev].ptr);
          p.ws_lse = p.ws_o + rows * splits * 128;
        }
      }
    }
    int launches = 0;
    cudaError_t e = launch_attn_decode(p, bf16, s, &launches);
    g_launches += launches;
    if (e != cudaSuccess) return cuda_fail(e, "decode attention launch");
    return GPU_OPS_OK;
  }
  PrefillParams p{};
  p.g = g;
  p.out = out;
  p.q = q;
  p.k_cache = k;
  p.v_cache = v;
  p.m = m;
  p.n = n;
  p.offset = offset;
  p.scale_log2 = scale_log2_of(head_dim);
  p.l2_window = g_prefill_l2_window.load();
  return run_prefill(p, bf16, s);
}

int ref_rope(void *out_q, void *out_k, const void *freqs, const void *in_q, const void *in_k, int start_pos,
             int cur_size, int n_heads, int hidden_dim, int is_neox, int dt, gpu_stream_t stream) {
  if (!dt_ok(dt)) return fail(GPU_OPS_E_UNSUPPORTED, "dtype %d: only fp16 (4) and bf16 (5) are supported", dt);
  if (n_heads <= 0 || hidden_dim <= 0 || hidden_dim % n_heads)
    return fail(GPU_OPS_E_INVALID, "n_heads %d, hidden_dim %d", n_heads, hidden_dim);
  if (hidden_dim / n_heads != 128)
    return fail(GPU_OPS_E_UNSUPPORTED, "head_dim %d: only 128 is supported", hidden_dim / n_heads);
  if (!out_q || !freqs || !in_q || (out_k && !in_k)) return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  if (start_pos < 0 || cur_size < 0) return fail(GPU_OPS_E_INVALID, "start_pos %d, cur_size %d", start_pos, cur_size);
  if (!aligned16(out_q) || !aligned16(in_q) || !aligned16(out_k) || !aligned16(in_k) || !aligned16(freqs))
    return fail(GPU_OPS_E_INVALID, "tensor pointers must be 16-byte aligned");
  if (cur_size == 0) return GPU_OPS_OK;
  RopeParams p{};
  auto set = [&](RopeStream &st, const void *src, void *dst) {
    st.src = src;
    st.dst = dst;
    st.heads = n_heads;
    st.rotate = 1;
    st.dst_at_pos = 0;
    st.src_seq = st.dst_seq = 0;
    st.src_tok = st.dst_tok = hidden_dim;
    st.dst_head = 128;
  };
  set(p.s[0], in_q, out_q);
  p.slots = n_heads;
  if (out_k) {
    set(p.s[1], in_k, out_k);
    p.slots += n_heads;
  }
  p.freqs_cis = static_cast<const float *>(freqs);
  p.start_pos = start_pos;
  p.batch = 1;
  p.m = cur_size;
  p.is_neox = is_neox ? 1 : 0;
  cudaError_t e = launch_rope_append(p, dt == GPU_DT_BFLOAT16, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "rope launch");
  g_launches += 1;
  return GPU_OPS_OK;
}

} // namespace

namespace b200attn {
void set_last_error(const char *msg) { g_last_error = msg ? msg : ""; }
void add_launch_count(int launches) { g_launches += launches; }
} // namespace b200attn

namespace {

// Validates a page description and converts it; pages == nullptr means a flat cache.
int paging_from(const gpu_kv_pages *pages, KvPaging *pg) {
  *pg = KvPaging{};
  if (!pages) return GPU_OPS_OK;
  if (!pages->page_table) return fail(GPU_OPS_E_INVALID, "null page table");
  const int ps = pages->page_size;
  if (ps < 64 || (ps & (ps - 1))) return fail(GPU_OPS_E_UNSUPPORTED, "page size %d: a power of two >= 64", ps);
  if (pages->table_stride <= 0 || pages->page_stride <= 0 || pages->page_stride % 8 || pages->n_pages <= 0)
    return fail(GPU_OPS_E_INVALID, "table stride %d, page stride %lld, pages %d", pages->table_stride,
                static_cast<long long>(pages->page_stride), pages->n_pages);
  pg->table = pages->page_table;
  pg->page_stride = pages->page_stride;
  pg->table_stride = pages->table_stride;
  pg->n_pages = pages->n_pages;
  int shift = 0;
  while ((1 << shift) < ps) ++shift;
  pg->page_shift = shift;
  return GPU_OPS_OK;
}

// Sources of one RoPE + append pass: three tensors with their own strides, or three
// column ranges of one fused projection row; bias rows are optional.
struct RopeSources {
  const void *q, *k, *v;
  long q_seq, q_tok, kv_seq, kv_tok;
  const void *bias_q, *bias_k, *bias_v;
};

int rope_append_common(const gpu_attn_desc *desc, const gpu_kv_pages *pages, void *q_out, void *k_cache, void *v_cache,
                       const RopeSources &src, const void *freqs_cis_dev, const int32_t *start_pos_dev, int start_pos,
                       int m, gpu_stream_t stream) {
  const void *q_in = src.q, *k_in = src.k, *v_in = src.v;
  KvPaging pg;
  if (int rc = paging_from(pages, &pg)) return rc;
  if (!k_cache || !v_cache || !k_in || !v_in || !freqs_cis_dev || (q_out && !q_in))
    return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  if (m < 0 || (!start_pos_dev && start_pos < 0)) return fail(GPU_OPS_E_INVALID, "m %d, start_pos %d", m, start_pos);
  if (!aligned16(q_out) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(q_in) || !aligned16(k_in) ||
      !aligned16(v_in) || !aligned16(freqs_cis_dev))
    return fail(GPU_OPS_E_INVALID, "tensor pointers must be 16-byte aligned");
  if (m == 0) return GPU_OPS_OK;
  // With the sequence as the outermost cache dimension the caches lie cache_seq_stride apart: rows
  // appended beyond what that stride holds would land in the next sequence's cache (or behind the last).
  if (!pages && !start_pos_dev && desc->batch > 1 && desc->cache_seq_stride > 0 &&
      desc->cache_seq_stride >= desc->cache_head_stride && desc->cache_seq_stride >= desc->cache_pos_stride &&
      (static_cast<long>(start_pos) + m) * desc->n_kv_heads * desc->head_dim > desc->cache_seq_stride)
    return fail(GPU_OPS_E_INVALID, "positions %d..%ld do not fit the cache (%ld per sequence)", start_pos,
                static_cast<long>(start_pos) + m - 1,
                static_cast<long>(desc->cache_seq_stride / (static_cast<long>(desc->n_kv_heads) * desc->head_dim)));
  RopeParams p{};
  int slots = 0;
  if (q_out) {
    RopeStream &s = p.s[slots];
    s.src = q_in;
    s.dst = q_out;
    s.heads = desc->n_heads;
    s.rotate = 1;
    s.dst_at_pos = 0;
    s.bias = src.bias_q;
    s.src_seq = src.q_seq;
    s.src_tok = src.q_tok;
    s.dst_seq = desc->q_seq_stride;
    s.dst_tok = desc->q_tok_stride;
    s.dst_head = 128;
    ++slots;
  }
  for (int kv = 0; kv < 2; ++kv) {
    RopeStream &s = p.s[slots++];
    s.src = kv == 0 ? k_in : v_in;
    s.dst = kv == 0 ? k_cache : v_cache;
    s.heads = desc->n_kv_heads;
    s.rotate = kv == 0 ? 1 : 0;
    s.dst_at_pos = 1;
    s.bias = kv == 0 ? src.bias_k : src.bias_v;
    s.src_seq = src.kv_seq;
    s.src_tok = src.kv_tok;
    s.dst_seq = desc->cache_seq_stride;
    s.dst_tok = desc->cache_pos_stride;
    s.dst_head = desc->cache_head_stride;
  }
  p.slots = (q_out ? desc->n_heads : 0) + 2 * desc->n_kv_heads;
  p.pg = pg;
  p.freqs_cis = static_cast<const float *>(freqs_cis_dev);
  p.start_pos_dev = start_pos_dev;
  p.start_pos = start_pos;
  p.batch = desc->batch;
  p.m = m;
  p.is_neox = desc->is_neox_style ? 1 : 0;
  cudaError_t e = launch_rope_append(p, desc->dtype == GPU_DT_BFLOAT16, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "rope + append launch");
  g_launches += 1;
  return GPU_OPS_OK;
}

} // namespace

extern "C" {

int gpu_flash_attn_layer(void *output_dev, const void *q_dev, const void *k_dev, const void *v_dev, int m, int n,
                         int offset, int head_num, int head_dim, int dt, gpu_stream_t stream) {
  return ref_attention(output_dev, q_dev, k_dev, v_dev, m, n, offset, 1, head_num, head_dim, dt, stream);
}

int gpu_flash_attn_gqa_layer(void *output_dev, const void *q_dev, const void *k_dev, const void *v_dev, int m,
                             int n, int offset, int group_size, int kv_head_num, int head_dim, int dt,
                             gpu_stream_t stream) {
  return ref_attention(output_dev, q_dev, k_dev, v_dev, m, n, offset, group_size, kv_head_num, head_dim, dt, stream);
}

int gpu_flash_attn_opt_prefill_layer(void *output_dev, const void *q_dev, const void *k_dev, const void *v_dev,
                                     int m, int n, int offset, int head_num, int head_dim, int dt,
                                     gpu_stream_t stream) {
  return ref_attention(output_dev, q_dev, k_dev, v_dev, m, n, offset, 1, head_num, head_dim, dt, stream);
}

int gpu_rope_layer(void *output_q_dev, void *output_k_dev, const void *freqs_cis_dev, const void *input_q_dev,
                   const void *input_k_dev, int start_pos, int cur_size, int n_heads, int hidden_dim,
                   int is_neox_style, int dt, gpu_stream_t stream) {
  if (!output_k_dev || !input_k_dev) return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  return ref_rope(output_q_dev, output_k_dev, freqs_cis_dev, input_q_dev, input_k_dev, start_pos, cur_size, n_heads,
                  hidden_dim, is_neox_style, dt, stream);
}

int gpu_rope_single_layer(void *output_x_dev, const void *freqs_cis_dev, const void *input_x_dev, int start_pos,
                          int cur_size, int n_heads, int hidden_dim, int is_neox_style, int dt,
                          gpu_stream_t stream) {
  return ref_rope(output_x_dev, nullptr, freqs_cis_dev, input_x_dev, nullptr, start_pos, cur_size, n_heads,
                  hidden_dim, is_neox_style, dt, stream);
}

int gpu_rope_kv_append_layer(const gpu_attn_desc *desc, void *q_out, void *k_cache, void *v_cache, const void *q_in,
                             const void *k_in, const void *v_in, const void *freqs_cis_dev,
                             const int32_t *start_pos_dev, int start_pos, int m, gpu_stream_t stream) {
  if (int rc = check_desc(desc)) return rc;
  RopeSources src{q_in, k_in, v_in, desc->q_seq_stride, desc->q_tok_stride, desc->kv_in_seq_stride,
                  desc->kv_in_tok_stride, nullptr, nullptr, nullptr};
  return rope_append_common(desc, nullptr, q_out, k_cache, v_cache, src, freqs_cis_dev, start_pos_dev, start_pos, m,
                            stream);
}

int gpu_rope_kv_append_paged_layer(const gpu_attn_desc *desc, const gpu_kv_pages *pages, void *q_out, void *k_pool,
                                   void *v_pool, const void *q_in, const void *k_in, const void *v_in,
                                   const void *freqs_cis_dev, const int32_t *start_pos_dev, int start_pos, int m,
                                   gpu_stream_t stream) {
  if (int rc = check_desc(desc)) return rc;
  if (!pages) return fail(GPU_OPS_E_INVALID, "null page description");
  RopeSources src{q_in, k_in, v_in, desc->q_seq_stride, desc->q_tok_stride, desc->kv_in_seq_stride,
                  desc->kv_in_tok_stride, nullptr, nullptr, nullptr};
  return rope_append_common(desc, pages, q_out, k_pool, v_pool, src, freqs_cis_dev, start_pos_dev, start_pos, m,
                            stream);
}

int gpu_qkv_rope_kv_append_layer(const gpu_attn_desc *desc, void *q_out, void *k_cache, void *v_cache,
                                 const void *qkv_in, int64_t qkv_seq_stride, int64_t qkv_tok_stride,
                                 const void *qkv_bias, const void *freqs_cis_dev, const int32_t *start_pos_dev,
                                 int start_pos, int m, gpu_stream_t stream) {
  if (int rc = check_desc(desc)) return rc;
  if (!qkv_in) return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  const long q_dim = static_cast<long>(desc->n_heads) * 128, kv_dim = static_cast<long>(desc->n_kv_heads) * 128;
  if (qkv_tok_stride < q_dim + 2 * kv_dim || qkv_tok_stride % 8 || qkv_seq_stride % 8 || qkv_seq_stride < 0)
    return fail(GPU_OPS_E_INVALID, "fused row stride %lld (row holds %ld elements), sequence stride %lld",
                static_cast<long long>(qkv_tok_stride), q_dim + 2 * kv_dim, static_cast<long long>(qkv_seq_stride));
  if (!aligned16(qkv_in) || !aligned16(qkv_bias))
    return fail(GPU_OPS_E_INVALID, "tensor pointers must be 16-byte aligned");
  const size_t eb = 2;
  const char *row = static_cast<const char *>(qkv_in);
  const char *bias = static_cast<const char *>(qkv_bias);
  RopeSources src{row,
                  row + q_dim * eb,
                  row + (q_dim + kv_dim) * eb,
                  qkv_seq_stride,
                  qkv_tok_stride,
                  qkv_seq_stride,
                  qkv_tok_stride,
                  bias,
                  bias ? bias + q_dim * eb : nullptr,
                  bias ? bias + (q_dim + kv_dim) * eb : nullptr};
  return rope_append_common(desc, nullptr, q_out, k_cache, v_cache, src, freqs_cis_dev, start_pos_dev, start_pos, m,
                            stream);
}

int gpu_split_qkv_layer(void *output_q_dev, void *output_k_dev, void *output_v_dev, const void *input_qkv, int batch,
                        int q_dim, int k_dim, int v_dim, int dt, gpu_stream_t stream) {
  if (dt != GPU_DT_FLOAT16 && dt != GPU_DT_BFLOAT16) return fail(GPU_OPS_E_UNSUPPORTED, "dtype %d", dt);
  if (batch < 0 || q_dim < 0 || k_dim < 0 || v_dim < 0)
    return fail(GPU_OPS_E_INVALID, "batch %d, dims %d %d %d", batch, q_dim, k_dim, v_dim);
  if (q_dim % 128 || k_dim % 128 || v_dim % 128)
    return fail(GPU_OPS_E_UNSUPPORTED, "dims %d %d %d: each must be a multiple of 128", q_dim, k_dim, v_dim);
  if (batch == 0 || q_dim + k_dim + v_dim == 0) return GPU_OPS_OK; // nothing is read or written
  if (!output_q_dev || !output_k_dev || !output_v_dev || !input_qkv)
    return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  if (!aligned16(output_q_dev) || !aligned16(output_k_dev) || !aligned16(output_v_dev) || !aligned16(input_qkv))
    return fail(GPU_OPS_E_INVALID, "tensor pointers must be 16-byte aligned");
  RopeParams p{};
  const long row = static_cast<long>(q_dim) + k_dim + v_dim;
  const int dims[3] = {q_dim, k_dim, v_dim};
  void *dsts[3] = {output_q_dev, output_k_dev, output_v_dev};
  long col = 0;
  for (int i = 0; i < 3; ++i) {
    RopeStream &st = p.s[i];
    st.src = static_cast<const char *>(input_qkv) + col * 2;
    st.dst = dsts[i];
    st.heads = dims[i] / 128;
    st.src_tok = row;
    st.dst_tok = dims[i];
    st.dst_head = 128;
    col += dims[i];
    p.slots += st.heads;
  }
  p.batch = 1;
  p.m = batch;
  cudaError_t e = launch_rope_append(p, dt == GPU_DT_BFLOAT16, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "split launch");
  g_launches += 1;
  return GPU_OPS_OK;
}


int gpu_bias_add_layer(void *output_dev, const void *input_dev, const void *bias_dev, int rows, int width,
                       int64_t row_stride, int dt, gpu_stream_t stream) {
  if (dt != GPU_DT_FLOAT16 && dt != GPU_DT_BFLOAT16) return fail(GPU_OPS_E_UNSUPPORTED, "dtype %d", dt);
  if (rows < 0 || width < 0 || row_stride < width || row_stride % 8)
    return fail(GPU_OPS_E_INVALID, "rows %d, width %d, row stride %lld", rows, width, static_cast<long long>(row_stride));
  if (width % 128) return fail(GPU_OPS_E_UNSUPPORTED, "width %d: must be a multiple of 128", width);
  if (!output_dev || !input_dev || !bias_dev) return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  if (!aligned16(output_dev) || !aligned16(input_dev) || !aligned16(bias_dev))
    return fail(GPU_OPS_E_INVALID, "tensor pointers must be 16-byte aligned");
  if (rows == 0 || width == 0) return GPU_OPS_OK;
  RopeParams p{};
  RopeStream &st = p.s[0];
  st.src = input_dev;
  st.dst = output_dev;
  st.bias = bias_dev;
  st.heads = width / 128;
  st.src_tok = st.dst_tok = row_stride;
  st.dst_head = 128;
  p.slots = st.heads;
  p.batch = 1;
  p.m = rows;
  cudaError_t e = launch_rope_append(p, dt == GPU_DT_BFLOAT16, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "bias launch");
  g_launches += 1;
  return GPU_OPS_OK;
}

static int prefill_common(const gpu_attn_desc *desc, const gpu_kv_pages *pages, void *out, const void *q,
                          const void *k_cache, const void *v_cache, int m, int offset, gpu_stream_t stream) {
  if (int rc = check_desc(desc)) return rc;
  KvPaging pg;
  if (int rc = paging_from(pages, &pg)) return rc;
  if (!out || !q || !k_cache || !v_cache) return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  if (m <= 0 || offset < 0) return fail(GPU_OPS_E_INVALID, "m %d, offset %d", m, offset);
  if (!aligned16(out) || !aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache))
    return fail(GPU_OPS_E_INVALID, "tensor pointers must be 16-byte aligned");
  const long n_pos = static_cast<long>(offset) + m;
  if (pages) {
    const long entries = (n_pos + pages->page_size - 1) / pages->page_size;
    if (entries > pages->table_stride)
      return fail(GPU_OPS_E_INVALID, "page table rows hold %d entries, %ld needed", pages->table_stride, entries);
  } else if (desc->batch > 1 && desc->cache_seq_stride > 0 && desc->cache_seq_stride >= desc->cache_head_stride &&
             desc->cache_seq_stride >= desc->cache_pos_stride &&
             n_pos * desc->n_kv_heads * desc->head_dim > desc->cache_seq_stride) {
    // sequence outermost: the caches lie cache_seq_stride apart and cannot hold more positions than that
    return fail(GPU_OPS_E_INVALID, "%ld positions do not fit the cache (%ld per sequence)", n_pos,
                static_cast<long>(desc->cache_seq_stride / (static_cast<long>(desc->n_kv_heads) * desc->head_dim)));
  }
  PrefillParams p{};
  p.g = geom_from_desc(desc);
  p.out = out;
  p.q = q;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.m = m;
  p.n = offset + m;
  p.offset = offset;
  p.scale_log2 = scale_log2_of(desc->head_dim);
  p.pg = pg;
  p.l2_window = g_prefill_l2_window.load();
  return run_prefill(p, desc->dtype == GPU_DT_BFLOAT16, static_cast<cudaStream_t>(stream));
}

int gpu_attn_prefill_layer(const gpu_attn_desc *desc, void *out, const void *q, const void *k_cache,
                           const void *v_cache, int m, int offset, gpu_stream_t stream) {
  return prefill_common(desc, nullptr, out, q, k_cache, v_cache, m, offset, stream);
}

int gpu_attn_prefill_paged_layer(const gpu_attn_desc *desc, const gpu_kv_pages *pages, void *out, const void *q,
                                 const void *k_pool, const void *v_pool, int m, int offset, gpu_stream_t stream) {
  if (!pages) return fail(GPU_OPS_E_INVALID, "null page description");
  return prefill_common(desc, pages, out, q, k_pool, v_pool, m, offset, stream);
}

size_t gpu_attn_decode_workspace_bytes(const gpu_attn_desc *desc, int max_kv_len) {
  if (!desc || desc->batch <= 0 || desc->n_kv_heads <= 0 || max_kv_len <= 0) return 0;
  // enough for the shortest split the call may choose, whatever length hint it is given
  const int forced = g_decode_chunk.load();
  const int chunk = forced > 0 ? forced : kMinChunk;
  const int splits = (max_kv_len + chunk - 1) / chunk;
  return decode_ws_bytes(static_cast<long>(desc->batch) * desc->n_heads, splits);
}

// ---- cross-device exchange over peer memory ----------------------------------
namespace {
size_t align16(size_t x) { return (x + 15) & ~static_cast<size_t>(15); }
size_t xchg_slots_bytes(int world, int rows) { return align16(static_cast<size_t>(world) * rows * 129 * 4); }
size_t xchg_half_bytes(int world, int rows) {
  return xchg_slots_bytes(world, rows) + align16(static_cast<size_t>(world) * rows * 4);
}

struct XchgRequest {
  void *local;
  void *const *peers;
  int world, rank;
  uint32_t epoch;
};

// Addresses of one step's buffer half on this rank and on its peers.
int build_xchg(XchgParams *p, const XchgRequest &x, int rows) {
  if (!x.local || !x.peers) return fail(GPU_OPS_E_INVALID, "null pointer");
  if (x.world < 1 || x.world > kMaxPeers || x.rank < 0 || x.rank >= x.world || rows <= 0 || x.epoch == 0)
    return fail(GPU_OPS_E_INVALID, "world %d (1..%d), rank %d, rows %d, epoch %u", x.world, kMaxPeers, x.rank, rows,
                x.epoch);
  *p = XchgParams{};
  const size_t half = (x.epoch & 1u) * xchg_half_bytes(x.world, rows);
  const size_t n = static_cast<size_t>(rows) * 129;
  char *lb = static_cast<char *>(x.local) + half;
  p->slots = reinterpret_cast<const float *>(lb);
  p->flags = reinterpret_cast<const uint32_t *>(lb + xchg_slots_bytes(x.world, rows));
  for (int r = 0; r < x.world; ++r) {
    if (r == x.rank) continue;
    if (!x.peers[r]) return fail(GPU_OPS_E_INVALID, "peer buffer %d is null", r);
    char *pb = static_cast<char *>(x.peers[r]) + half;
    p->peer_slot[r] = reinterpret_cast<float *>(pb) + static_cast<size_t>(x.rank) * n;
    p->peer_flag[r] = reinterpret_cast<uint32_t *>(pb + xchg_slots_bytes(x.world, rows)) + static_cast<size_t>(x.rank) * rows;
  }
  p->epoch = x.epoch;
  p->world = x.world;
  p->rank = x.rank;
  p->rows = rows;
  p->error_flag = kernel_error_word_dev();
  if (!p->error_flag) return fail(GPU_OPS_E_CUDA, "no status word");
  return GPU_OPS_OK;
}
} // namespace

size_t gpu_attn_xchg_buffer_bytes(int world, int rows) {
  if (world <= 0 || rows <= 0) return 0;
  return 2 * xchg_half_bytes(world, rows);
}

float *gpu_attn_xchg_local_slot(void *local_buffer, int world, int rank, uint32_t epoch, int rows) {
  if (!local_buffer || world <= 0 || rank < 0 || rank >= world || rows <= 0) return nullptr;
  char *half = static_cast<char *>(local_buffer) + (epoch & 1u) * xchg_half_bytes(world, rows);
  return reinterpret_cast<float *>(half) + static_cast<size_t>(rank) * rows * 129;
}

int gpu_attn_xchg_merge_layer(void *out, void *local_buffer, void *const *peer_buffers, int world, int rank,
                              uint32_t epoch, int rows, int head_dim, int dt, gpu_stream_t stream) {
  if (int rc = check_common(dt, head_dim)) return rc;
  if (!out) return fail(GPU_OPS_E_INVALID, "null pointer");
  XchgParams p;
  if (int rc = build_xchg(&p, XchgRequest{local_buffer, peer_buffers, world, rank, epoch}, rows)) return rc;
  p.out = out;
  cudaError_t e = launch_attn_xchg_merge(p, dt == GPU_DT_BFLOAT16, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "exchange + merge launch");
  g_launches += 1;
  return GPU_OPS_OK;
}

static int decode_common(const gpu_attn_desc *desc, const gpu_kv_pages *pages, void *out, float *o_partial,
                         float *lse_partial, const void *q_in, const void *k_in, const void *v_in, void *k_cache,
                         void *v_cache, const void *freqs_cis_dev, const int32_t *kv_len_dev,
                         const int32_t *rope_pos_dev, int append_new, int max_kv_len, void *workspace,
                         size_t workspace_bytes, gpu_stream_t stream, const XchgRequest *xchg = nullptr) {
  if (int rc = check_desc(desc)) return rc;
  XchgParams xp;
  if (xchg) {
    // the partial goes to this rank's slot of the exchange buffer, or stays split for the exchange kernel
    if (int rc = build_xchg(&xp, *xchg, desc->batch * desc->n_heads)) return rc;
    o_partial = gpu_attn_xchg_local_slot(xchg->local, xchg->world, xchg->rank, xchg->epoch, desc->batch * desc->n_heads);
    lse_partial = o_partial + static_cast<size_t>(desc->batch) * desc->n_heads * 128;
  }
  KvPaging pg;
  if (int rc = paging_from(pages, &pg)) return rc;
  const int group = desc->n_heads / desc->n_kv_heads;
  if (group > 16) return fail(GPU_OPS_E_UNSUPPORTED, "group size %d: at most 16 query heads per KV head", group);
  if (!q_in || !k_cache || !v_cache || !freqs_cis_dev || !kv_len_dev)
    return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  if ((o_partial == nullptr) != (lse_partial == nullptr))
    return fail(GPU_OPS_E_INVALID, "o_partial and lse_partial go together");
  if (!out && !o_partial) return fail(GPU_OPS_E_INVALID, "no output given");
  if (append_new && (!k_in || !v_in)) return fail(GPU_OPS_E_INVALID, "append_new needs k_in and v_in");
  if (max_kv_len <= 0) return fail(GPU_OPS_E_INVALID, "max_kv_len %d", max_kv_len);
  if (!aligned16(out) || !aligned16(q_in) || !aligned16(k_in) || !aligned16(v_in) || !aligned16(k_cache) ||
      !aligned16(v_cache) || !aligned16(freqs_cis_dev) || !aligned16(workspace))
    return fail(GPU_OPS_E_INVALID, "tensor pointers must be 16-byte aligned");
  DecodeParams p{};
  p.g = geom_from_desc(desc);
  p.out = out;
  p.o_partial = o_partial;
  p.lse_partial = lse_partial;
  p.q = q_in;
  p.k_new = k_in;
  p.v_new = v_in;
  p.kv_in_seq = desc->kv_in_seq_stride;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.freqs_cis = static_cast<const float *>(freqs_cis_dev);
  p.kv_len_dev = kv_len_dev;
  p.rope_pos_dev = rope_pos_dev;
  p.m = 1;
  p.offset = -1;
  p.append = append_new ? 1 : 0;
  p.rotate_q = 1;
  p.is_neox = desc->is_neox_style ? 1 : 0;
  p.scale_log2 = scale_log2_of(desc->head_dim);
  p.pg = pg;
  p.early_kv = g_decode_early.load();
  p.error_flag = kernel_error_word_dev();
  p.chunk = pick_chunk(desc->batch, desc->n_kv_heads, desc->total_kv_len, max_kv_len);
  p.max_splits = (max_kv_len + p.chunk - 1) / p.chunk;
  if (p.max_splits > 1) {
    const long rows = static_cast<long>(desc->batch) * desc->n_heads;
    const size_t need = decode_ws_bytes(rows, p.max_splits);
    if (!workspace || workspace_bytes < need)
      return fail(GPU_OPS_E_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
    p.ws_o = static_cast<float *>(workspace);
    p.ws_lse = p.ws_o + rows * p.max_splits * 128;
  }
  if (xchg) p.no_merge = 1;
  int launches = 0;
  cudaError_t e = launch_attn_decode(p, desc->dtype == GPU_DT_BFLOAT16, static_cast<cudaStream_t>(stream), &launches);
  g_launches += launches;
  if (e != cudaSuccess) return cuda_fail(e, "decode attention launch");
  if (xchg) {
    xp.out = out;
    if (p.max_splits > 1) {
      xp.ws_o = p.ws_o;
      xp.ws_lse = p.ws_lse;
      xp.max_splits = p.max_splits;
      xp.chunk = p.chunk;
      xp.append = p.append;
      xp.rows_per_seq = desc->n_heads;
      xp.kv_len_dev = kv_len_dev;
    }
    e = launch_attn_xchg_merge(xp, desc->dtype == GPU_DT_BFLOAT16, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, "exchange + merge launch");
    g_launches += 1;
  }
  return GPU_OPS_OK;
}

int gpu_attn_decode_xchg_layer(const gpu_attn_desc *desc, void *out, const void *q_in, const void *k_in,
                               const void *v_in, void *k_cache, void *v_cache, const void *freqs_cis_dev,
                               const int32_t *kv_len_dev, const int32_t *rope_pos_dev, int append_new, int max_kv_len,
                               void *workspace, size_t workspace_bytes, void *local_buffer, void *const *peer_buffers,
                               int world, int rank, uint32_t epoch, gpu_stream_t stream) {
  if (!out) return fail(GPU_OPS_E_INVALID, "null pointer");
  const XchgRequest x{local_buffer, peer_buffers, world, rank, epoch};
  return decode_common(desc, nullptr, out, nullptr, nullptr, q_in, k_in, v_in, k_cache, v_cache, freqs_cis_dev,
                       kv_len_dev, rope_pos_dev, append_new, max_kv_len, workspace, workspace_bytes, stream, &x);
}

int gpu_attn_decode_layer(const gpu_attn_desc *desc, void *out, float *o_partial, float *lse_partial,
                          const void *q_in, const void *k_in, const void *v_in, void *k_cache, void *v_cache,
                          const void *freqs_cis_dev, const int32_t *kv_len_dev, const int32_t *rope_pos_dev,
                          int append_new, int max_kv_len, void *workspace, size_t workspace_bytes,
                          gpu_stream_t stream) {
  return decode_common(desc, nullptr, out, o_partial, lse_partial, q_in, k_in, v_in, k_cache, v_cache, freqs_cis_dev,
                       kv_len_dev, rope_pos_dev, append_new, max_kv_len, workspace, workspace_bytes, stream);
}

int gpu_attn_decode_paged_layer(const gpu_attn_desc *desc, const gpu_kv_pages *pages, void *out, const void *q_in,
                                const void *k_in, const void *v_in, void *k_pool, void *v_pool,
                                const void *freqs_cis_dev, const int32_t *kv_len_dev, int append_new, int max_kv_len,
                                void *workspace, size_t workspace_bytes, gpu_stream_t stream) {
  if (!pages) return fail(GPU_OPS_E_INVALID, "null page description");
  return decode_common(desc, pages, out, nullptr, nullptr, q_in, k_in, v_in, k_pool, v_pool, freqs_cis_dev, kv_len_dev,
                       nullptr, append_new, max_kv_len, workspace, workspace_bytes, stream);
}

// ---- planned decode ---------------------------------------------------------------
namespace {
constexpr int kPlanMaxCtas = 1024;

const PlanHeader *plan_header(const void *plan_host) {
  const PlanHeader *h = static_cast<const PlanHeader *>(plan_host);
  return (h && h->magic == kPlanMagic) ? h : nullptr;
}
} // namespace

size_t gpu_attn_decode_plan_bytes(const gpu_attn_desc *desc, int n_ctas) {
  if (!desc || n_ctas < 0 || n_ctas > kPlanMaxCtas) return 0;
  return decode_plan_capacity(desc->batch, desc->n_kv_heads, n_ctas > 0 ? n_ctas : kPlanMaxCtas);
}

int gpu_attn_decode_plan(const gpu_attn_desc *desc, const int32_t *kv_len_host, int append_new, int n_ctas,
                         void *plan_host, size_t plan_bytes) {
  if (int rc = check_desc(desc)) return rc;
  if (!kv_len_host || !plan_host) return fail(GPU_OPS_E_INVALID, "null pointer");
  if (desc->n_heads / desc->n_kv_heads > 16)
    return fail(GPU_OPS_E_UNSUPPORTED, "group size %d: at most 16 query heads per KV head", desc->n_heads / desc->n_kv_heads);
  if (n_ctas < 0 || n_ctas > kPlanMaxCtas) return fail(GPU_OPS_E_INVALID, "n_ctas %d (0 .. %d)", n_ctas, kPlanMaxCtas);
  if (n_ctas == 0) {
    // Three quarters of what the current device holds at once: consecutive calls are launched as
    // programmatic dependents, and the free quarter lets the next call's first CTAs move in and
    // fetch their first tiles while this call still streams (measured on B200, 296 slots: 222 CTAs
    // beat 296 by 0 - 3 % at every size from 87 MB to 694 MB per call).
    const int slots = decode_planned_max_ctas();
    if (slots <= 0) return fail(GPU_OPS_E_CUDA, "no current CUDA device to size the plan for");
    n_ctas = std::min(kPlanMaxCtas, std::max(1, slots * 3 / 4));
  }
  for (int b = 0; b < desc->batch; ++b)
    if (kv_len_host[b] < 0) return fail(GPU_OPS_E_INVALID, "kv_len[%d] = %d", b, kv_len_host[b]);
  const size_t used = build_decode_plan(plan_host, plan_bytes, kv_len_host, desc->batch, desc->n_kv_heads,
                                        desc->n_heads / desc->n_kv_heads, append_new, n_ctas);
  if (!used) return fail(GPU_OPS_E_WORKSPACE, "plan buffer of %zu bytes is too small", plan_bytes);
  return GPU_OPS_OK;
}

size_t gpu_attn_decode_plan_size(const void *plan_host) {
  const PlanHeader *h = plan_header(plan_host);
  return h ? static_cast<size_t>(h->total_bytes) : 0;
}

size_t gpu_attn_decode_plan_workspace_bytes(const void *plan_host) {
  const PlanHeader *h = plan_header(plan_host);
  return h ? static_cast<size_t>(h->n_slots) * h->group * (128 + 1) * sizeof(float) : 0;
}

int gpu_attn_decode_planned_layer(const gpu_attn_desc *desc, const gpu_kv_pages *pages, const void *plan_host,
                                  const void *plan_dev, void *out, float *o_partial, float *lse_partial,
                                  const void *q_in, const void *k_in, const void *v_in, void *k_cache, void *v_cache,
                                  const void *freqs_cis_dev, const int32_t *rope_pos_dev, void *workspace,
                                  size_t workspace_bytes, gpu_stream_t stream) {
  if (int rc = check_desc(desc)) return rc;
  KvPaging pg;
  if (int rc = paging_from(pages, &pg)) return rc;
  const PlanHeader *h = plan_header(plan_host);
  if (!h || !plan_dev) return fail(GPU_OPS_E_INVALID, "not a decode plan");
  const int group = desc->n_heads / desc->n_kv_heads;
  if (h->batch != desc->batch || h->n_kv_heads != desc->n_kv_heads || h->group != group)
    return fail(GPU_OPS_E_INVALID, "plan was built for batch %d, %d KV heads, group %d", h->batch, h->n_kv_heads, h->group);
  if (!q_in || !k_cache || !v_cache || !freqs_cis_dev) return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  if ((o_partial == nullptr) != (lse_partial == nullptr))
    return fail(GPU_OPS_E_INVALID, "o_partial and lse_partial go together");
  if (!out && !o_partial) return fail(GPU_OPS_E_INVALID, "no output given");
  if (h->append && (!k_in || !v_in)) return fail(GPU_OPS_E_INVALID, "the plan appends a token: k_in and v_in are needed");
  if (!aligned16(out) || !aligned16(q_in) || !aligned16(k_in) || !aligned16(v_in) || !aligned16(k_cache) ||
      !aligned16(v_cache) || !aligned16(freqs_cis_dev) || !aligned16(workspace) || !aligned16(plan_dev) ||
      !aligned16(o_partial))
    return fail(GPU_OPS_E_INVALID, "tensor pointers must be 16-byte aligned");
  const size_t need = gpu_attn_decode_plan_workspace_bytes(plan_host);
  if (need && (!workspace || workspace_bytes < need))
    return fail(GPU_OPS_E_WORKSPACE, "workspace of %zu bytes given, %zu needed", workspace_bytes, need);
  if (pages && h->max_total > 0) {
    const long entries = (static_cast<long>(h->max_total) + pages->page_size - 1) / pages->page_size;
    if (entries > pages->table_stride)
      return fail(GPU_OPS_E_INVALID, "page table rows hold %d entries, %ld needed", pages->table_stride, entries);
  }
  // Without paging, and with the sequence as the outermost dimension of the cache, the sequences'
  // caches lie cache_seq_stride apart: a sequence longer than that stride holds would read and
  // (with an appended token) write the next sequence's memory.
  if (!pages && desc->batch > 1 && desc->cache_seq_stride >= desc->cache_head_stride &&
      desc->cache_seq_stride >= desc->cache_pos_stride && desc->cache_seq_stride > 0 &&
      static_cast<long>(h->max_total) * desc->n_kv_heads * desc->head_dim > desc->cache_seq_stride)
    return fail(GPU_OPS_E_INVALID, "the plan's longest sequence (%d positions) does not fit the cache (%ld per sequence)",
                h->max_total, static_cast<long>(desc->cache_seq_stride / (static_cast<long>(desc->n_kv_heads) * desc->head_dim)));
  PlannedDecodeParams p{};
  p.g = geom_from_desc(desc);
  p.out = o_partial ? nullptr : out;
  p.o_partial = o_partial;
  p.lse_partial = lse_partial;
  p.q = q_in;
  p.k_new = k_in;
  p.v_new = v_in;
  p.kv_in_seq = desc->kv_in_seq_stride;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.freqs_cis = static_cast<const float *>(freqs_cis_dev);
  p.rope_pos_dev = rope_pos_dev;
  p.is_neox = desc->is_neox_style ? 1 : 0;
  p.scale_log2 = scale_log2_of(desc->head_dim);
  p.plan = static_cast<const unsigned char *>(plan_dev);
  p.n_ctas = h->n_ctas;
  p.n_groups = h->n_groups;
  p.n_slots = h->n_slots;
  p.max_total = h->max_total > 0 ? h->max_total : 1;
  p.off_cta_begin = h->off_cta_begin;
  p.off_items = h->off_items;
  p.off_groups = h->off_groups;
  p.max_parts = h->max_parts;
  p.ws_o = static_cast<float *>(workspace);
  p.ws_lse = p.ws_o ? p.ws_o + static_cast<size_t>(h->n_slots) * group * 128 : nullptr;
  p.pg = pg;
  p.early_kv = g_decode_early.load();
  p.error_flag = kernel_error_word_dev();
  if (!p.error_flag) return fail(GPU_OPS_E_CUDA, "no status word");
  int launches = 0;
  cudaError_t e = launch_attn_decode_planned(p, desc->dtype == GPU_DT_BFLOAT16, static_cast<cudaStream_t>(stream), &launches);
  g_launches += launches;
  if (e == cudaErrorNotSupported)
    return fail(GPU_OPS_E_UNSUPPORTED, "the cache strides cannot be described by a TMA tensor map");
  if (e != cudaSuccess) return cuda_fail(e, "planned decode launch");
  return GPU_OPS_OK;
}

static int merge_parts(void *out, const float *o_parts, const float *lse_parts, long stride_o, long stride_lse,
                       int n_parts, int rows, int head_dim, int dt, gpu_stream_t stream) {
  if (int rc = check_common(dt, head_dim)) return rc;
  if (!out || !o_parts || !lse_parts) return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  if (n_parts <= 0 || rows < 0) return fail(GPU_OPS_E_INVALID, "n_parts %d, rows %d", n_parts, rows);
  MergeParams p{};
  p.out = out;
  p.parts_o = o_parts;
  p.parts_lse = lse_parts;
  p.part_stride_o = stride_o;
  p.part_stride_lse = stride_lse;
  p.part_major = 1;
  p.lse_is_log2 = 0;
  p.rows = rows;
  p.max_parts = n_parts;
  p.n_parts = n_parts;
  p.rows_per_seq = rows > 0 ? rows : 1;
  p.n_heads = rows > 0 ? rows : 1;
  p.m = 1;
  p.out_seq = 0;
  p.out_tok = 0;
  cudaError_t e = launch_attn_merge(p, dt == GPU_DT_BFLOAT16, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_fail(e, "merge launch");
  g_launches += 1;
  return GPU_OPS_OK;
}

int gpu_attn_merge_lse_layer(void *out, const float *o_parts, const float *lse_parts, int n_parts, int rows,
                             int head_dim, int dt, gpu_stream_t stream) {
  return merge_parts(out, o_parts, lse_parts, static_cast<long>(rows) * 128, rows, n_parts, rows, head_dim, dt, stream);
}

int gpu_attn_merge_packed_layer(void *out, const float *parts, int n_parts, int rows, int head_dim, int dt,
                                gpu_stream_t stream) {
  if (!parts) return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  const long stride = static_cast<long>(rows) * (128 + 1);
  return merge_parts(out, parts, parts + static_cast<long>(rows) * 128, stride, stride, n_parts, rows, head_dim, dt,
                     stream);
}

int gpu_peer_buffer_alloc(size_t bytes, void **ptr, unsigned char *handle64) {
  if (!ptr || !handle64 || bytes == 0) return fail(GPU_OPS_E_INVALID, "null pointer or zero size");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return cuda_fail(e, "peer buffer allocation");
  if ((e = cudaMemset(p, 0, bytes)) != cudaSuccess || (e = cudaDeviceSynchronize()) != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e, "peer buffer clear");
  }
  cudaIpcMemHandle_t h;
  if ((e = cudaIpcGetMemHandle(&h, p)) != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e, "peer buffer export");
  }
  memcpy(handle64, &h, 64);
  *ptr = p;
  return GPU_OPS_OK;
}

int gpu_peer_buffer_open(const unsigned char *handle64, void **ptr) {
  if (!ptr || !handle64) return fail(GPU_OPS_E_INVALID, "null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail(e, "peer buffer import");
  return GPU_OPS_OK;
}

int gpu_peer_buffer_close(void *ptr) {
  if (!ptr) return GPU_OPS_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? GPU_OPS_OK : cuda_fail(e, "peer buffer close");
}

int gpu_peer_buffer_free(void *ptr) {
  if (!ptr) return GPU_OPS_OK;
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? GPU_OPS_OK : cuda_fail(e, "peer buffer free");
}

int gpu_ops_set_workspace(void *workspace, size_t bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(GPU_OPS_E_INVALID, "device index %d", dev);
  if (workspace && !aligned16(workspace)) return fail(GPU_OPS_E_INVALID, "workspace must be 16-byte aligned");
  std::lock_guard<std::mutex> lk(g_ws_mutex);
  g_ws[dev].ptr = workspace;
  g_ws[dev].bytes = workspace ? bytes : 0;
  return GPU_OPS_OK;
}

int gpu_attn_set_decode_chunk(int positions) {
  if (positions < 0 || positions % 64) return fail(GPU_OPS_E_INVALID, "chunk %d: a non-negative multiple of 64", positions);
  g_decode_chunk.store(positions);
  return GPU_OPS_OK;
}

int gpu_attn_set_decode_early_prefetch(int on) {
  g_decode_early.store(on ? 1 : 0);
  return GPU_OPS_OK;
}

int gpu_attn_set_prefill_kernel(int which) {
  if (which < 0 || which > 3) return fail(GPU_OPS_E_INVALID, "prefill kernel selector %d", which);
  g_prefill_kernel.store(which);
  return GPU_OPS_OK;
}

int gpu_attn_set_prefill_l2_window(size_t bytes) {
  if (bytes > (static_cast<size_t>(1) << 40)) return fail(GPU_OPS_E_INVALID, "L2 window of %zu bytes", bytes);
  g_prefill_l2_window.store(static_cast<long>(bytes));
  return GPU_OPS_OK;
}

int gpu_attn_last_prefill_kernel(void) { return g_last_prefill_kernel; }

int gpu_ops_kernel_status(void) { return attn_tc5_error_status(); }

int gpu_ops_clear_kernel_status(void) {
  attn_clear_error_status();
  return GPU_OPS_OK;
}

long gpu_ops_launch_count(int reset) {
  const long n = g_launches;
  if (reset) g_launches = 0;
  return n;
}

const char *gpu_ops_last_error_string(void) { return g_last_error.c_str(); }

} // extern "C"
