// gpu_attn_decode_layer_noalloc: the fused decode step for callers that cannot
// allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc when a decode step runs:
// a serving process that reserved all of the GPU's memory for its own KV-cache
// pool at start-up, so that a later cudaMalloc fails; a plug-in slot whose
// contract forbids allocation after initialisation; a latency-critical loop
// that cannot afford cudaMalloc's device-wide synchronisation, which stalls
// every stream.  The ordinary entry point (gpu_attn_decode_layer) leaves the
// split-KV scratch to the caller, and such a caller has nowhere to get it.
// This one brings its own: a fixed array in device global memory that is part
// of the library image.
//
// Cost and limit: every GPU on which the array has been resolved holds
// kNoAllocScratchBytes (16 MiB) until the process exits, used or not.  With CUDA's
// lazy module loading the array is materialised -- and its 16 MiB taken -- when its
// address is first looked up on a device, not when the library is loaded: a host
// that hands all device memory to its own pool must make that first look-up
// (gpu_attn_decode_noalloc_prepare, or a first call of the entry point) BEFORE it
// reserves its memory, or run with CUDA_MODULE_LOADING=EAGER.  The scratch holds, per query
// head and split, 128 fp32 partial outputs and one log-sum-exp, so a call needs
// batch * n_heads * ceil(max_kv_len / 512) * 516 bytes; a call that needs more
// is rejected with GPU_OPS_E_WORKSPACE before anything is launched.
//
// All calls on a device share the one array and it keeps whatever the last call
// left in it.  Nothing in it has to start at zero: every partial the merge reads
// has been written by the same call's split kernel first (the split count per
// sequence is recomputed from kv_len by both kernels).  Two calls whose kernels
// overlap on the GPU (different streams, no dependency) race on the array and
// give wrong results; order them on one stream or with events.
#include "gpu_ops.h"
#include "kernels.h"

#include <cmath>
#include <cstdio>
#include <mutex>

namespace {

constexpr size_t kNoAllocScratchBytes = 16u << 20;
constexpr int kNoAllocChunk = 512; // positions per split, fixed for this entry point
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code this name is only a stand-in for the
// symbol: its device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

std::mutex g_mutex;
void *g_scratch_ptr[kMaxDevices];
bool g_scratch_ready[kMaxDevices];

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Device address of the scratch array on the current device; looked up on the
// first call for that device (with that device current) and remembered.
cudaError_t scratch_address(void **out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lk(g_mutex);
  if (!g_scratch_ready[dev]) {
    void *ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_ptr[dev] = ptr;
    g_scratch_ready[dev] = true;
  }
  *out = g_scratch_ptr[dev];
  return cudaSuccess;
}

// failures are reported through gpu_ops_last_error_string(), like every other entry point
int fail(int code, const char *msg) {
  b200attn::set_last_error(msg);
  return code;
}

} // namespace

extern "C" {

int gpu_attn_decode_noalloc_prepare(void) {
  void *scratch = nullptr;
  cudaError_t e = scratch_address(&scratch);
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof msg, "cudaGetSymbolAddress of the scratch array: %s", cudaGetErrorString(e));
    return fail(GPU_OPS_E_CUDA, msg);
  }
  return GPU_OPS_OK;
}

int gpu_attn_decode_layer_noalloc(const gpu_attn_desc *desc, void *out, const void *q_in, const void *k_in,
                                  const void *v_in, void *k_cache, void *v_cache, const void *freqs_cis_dev,
                                  const int32_t *kv_len_dev, const int32_t *rope_pos_dev, int append_new,
                                  int max_kv_len, gpu_stream_t stream) {
  using namespace b200attn;
  if (!desc) return fail(GPU_OPS_E_INVALID, "desc is NULL");
  if (desc->dtype != GPU_DT_FLOAT16 && desc->dtype != GPU_DT_BFLOAT16)
    return fail(GPU_OPS_E_UNSUPPORTED, "only fp16 (4) and bf16 (5) are supported");
  if (desc->head_dim != 128) return fail(GPU_OPS_E_UNSUPPORTED, "only head_dim 128 is supported");
  if (desc->batch <= 0 || desc->n_heads <= 0 || desc->n_kv_heads <= 0 || desc->n_heads % desc->n_kv_heads)
    return fail(GPU_OPS_E_INVALID, "batch / n_heads / n_kv_heads are inconsistent");
  const int group = desc->n_heads / desc->n_kv_heads;
  if (group > 16) return fail(GPU_OPS_E_UNSUPPORTED, "at most 16 query heads per KV head");
  if (desc->cache_pos_stride % 8 || desc->cache_head_stride % 8 || desc->cache_seq_stride % 8 ||
      desc->q_seq_stride % 8 || desc->kv_in_seq_stride % 8 || desc->out_seq_stride % 8)
    return fail(GPU_OPS_E_INVALID, "strides must be multiples of 8 elements");
  if (!out || !q_in || !k_cache || !v_cache || !freqs_cis_dev || !kv_len_dev)
    return fail(GPU_OPS_E_INVALID, "null tensor pointer");
  if (append_new && (!k_in || !v_in)) return fail(GPU_OPS_E_INVALID, "append_new needs k_in and v_in");
  if (max_kv_len <= 0) return fail(GPU_OPS_E_INVALID, "max_kv_len must be positive");
  if (!aligned16(out) || !aligned16(q_in) || !aligned16(k_in) || !aligned16(v_in) || !aligned16(k_cache) ||
      !aligned16(v_cache) || !aligned16(freqs_cis_dev))
    return fail(GPU_OPS_E_INVALID, "tensor pointers must be 16-byte aligned");

  const int splits = (max_kv_len + kNoAllocChunk - 1) / kNoAllocChunk;
  const long rows = static_cast<long>(desc->batch) * desc->n_heads;
  const size_t need = static_cast<size_t>(rows) * splits * (128 + 1) * sizeof(float);
  if (splits > 1 && need > kNoAllocScratchBytes) {
    char msg[256];
    snprintf(msg, sizeof msg,
             "batch %d x %d heads x %d splits of %d positions needs %zu bytes of scratch; the built-in array "
             "holds %zu -- use gpu_attn_decode_layer with a caller-provided workspace",
             desc->batch, desc->n_heads, splits, kNoAllocChunk, need, kNoAllocScratchBytes);
    return fail(GPU_OPS_E_WORKSPACE, msg);
  }
  void *scratch = nullptr;
  cudaError_t e = scratch_address(&scratch);
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof msg, "cudaGetSymbolAddress of the scratch array: %s", cudaGetErrorString(e));
    return fail(GPU_OPS_E_CUDA, msg);
  }

  DecodeParams p{};
  p.g.batch = desc->batch;
  p.g.n_heads = desc->n_heads;
  p.g.n_kv_heads = desc->n_kv_heads;
  p.g.group = group;
  p.g.q_seq = desc->q_seq_stride;
  p.g.q_tok = desc->q_tok_stride;
  p.g.out_seq = desc->out_seq_stride;
  p.g.out_tok = desc->out_tok_stride;
  p.g.c_seq = desc->cache_seq_stride;
  p.g.c_head = desc->cache_head_stride;
  p.g.c_pos = desc->cache_pos_stride;
  p.out = out;
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
  p.chunk = kNoAllocChunk;
  p.max_splits = splits;
  p.scale_log2 = (1.0f / sqrtf(128.0f)) * 1.4426950408889634f;
  p.error_flag = kernel_error_word_dev();
  if (splits > 1) {
    p.ws_o = static_cast<float *>(scratch);
    p.ws_lse = p.ws_o + rows * splits * 128;
  }
  int launches = 0;
  e = launch_attn_decode(p, desc->dtype == GPU_DT_BFLOAT16, static_cast<cudaStream_t>(stream), &launches);
  add_launch_count(launches);
  if (e != cudaSuccess) {
    char msg[256];
    snprintf(msg, sizeof msg, "decode attention launch: %s", cudaGetErrorString(e));
    return fail(GPU_OPS_E_CUDA, msg);
  }
  return GPU_OPS_OK;
}

} // extern "C"
