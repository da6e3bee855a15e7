// C ABI over the host layer (declared in include/gpu_layer.h).
#include "gpu_layer.h"

#include <cstdlib>

#include "attention_layer_gpu.hpp"
#include "device.hpp"

namespace {
void *host_alloc(size_t n) { return std::malloc(n); }
void host_free(void *p) { std::free(p); }
AttentionLayerGPUImpl *as_layer(void *h) { return static_cast<AttentionLayerGPUImpl *>(h); }
} // namespace

extern "C" {

void *gpu_allocator_allocate(size_t bytes) { return GPUAllocator::Allocate(bytes); }
void gpu_allocator_deallocate(void *ptr) { GPUAllocator::Deallocate(ptr); }
void gpu_allocator_stats(size_t out[5]) {
  GPUAllocator::Stats s = GPUAllocator::GetStats();
  out[0] = s.backend_bytes;
  out[1] = s.pooled_bytes;
  out[2] = s.backend_allocs;
  out[3] = s.pool_hits;
  out[4] = s.backend_frees;
}
void gpu_allocator_trim(void) { GPUAllocator::Trim(); }
void gpu_allocator_set_limit(size_t bytes) { GPUAllocator::SetLimit(bytes); }
void gpu_allocator_use_host_backend(int on) {
  if (on)
    GPUAllocator::SetBackend(host_alloc, host_free);
  else
    GPUAllocator::SetBackend(nullptr, nullptr);
}

void gpu_init_freq_cis(float *host_out, int head_dim, int max_seq_len, float theta, int dt) {
  InitFreqCIS(host_out, head_dim, max_seq_len, theta, static_cast<DataType>(dt));
}

void *gpu_attention_layer_create(int kind, int n_heads, int n_kv_heads, int head_dim, int max_seq_len, int max_batch,
                                 int dt, float rope_theta, int rope_is_neox_style, int cache_layout,
                                 const float *shared_freq_cis_dev, void *k_cache_ext, void *v_cache_ext) {
  AttentionConfig cfg;
  cfg.n_heads = n_heads;
  cfg.n_kv_heads = n_kv_heads;
  cfg.head_dim = head_dim;
  cfg.max_seq_len = max_seq_len;
  cfg.max_batch = max_batch;
  cfg.data_type = static_cast<DataType>(dt);
  cfg.rope_theta = rope_theta;
  cfg.rope_is_neox_style = rope_is_neox_style != 0;
  cfg.cache_layout = cache_layout == 0 ? CacheLayout::TokenMajor : CacheLayout::HeadMajor;
  AttentionLayerGPUImpl *layer = nullptr;
  if (kind == 0)
    layer = new Llamma2AttentionGPUImpl();
  else if (kind == 1)
    layer = new Qwen2AttentionGPUImpl();
  else
    return nullptr;
  if (!layer->Init(cfg, shared_freq_cis_dev, k_cache_ext, v_cache_ext)) {
    delete layer;
    return nullptr;
  }
  return layer;
}

void gpu_attention_layer_destroy(void *layer) { delete as_layer(layer); }

int gpu_attention_layer_forward(void *layer, void *out, const void *q, const void *k, const void *v, int batch,
                                int cur_pos, int prev_pos, gpu_stream_t stream) {
  if (!layer || cur_pos < prev_pos || prev_pos < 0) return GPU_OPS_E_INVALID;
  InferenceCtx ctx(cur_pos, prev_pos);
  ctx.gpu_stream = static_cast<cudaStream_t>(stream);
  return as_layer(layer)->ForwardRaw(out, q, k, v, ctx, batch);
}

int gpu_attention_layer_decode_ragged(void *layer, void *out, const void *q, const void *k, const void *v,
                                      const int32_t *kv_len_host, int batch, gpu_stream_t stream) {
  if (!layer) return GPU_OPS_E_INVALID;
  return as_layer(layer)->DecodeRagged(out, q, k, v, kv_len_host, batch, static_cast<cudaStream_t>(stream));
}

int gpu_attention_layer_set_shared_lens(void *layer, const int32_t *kv_len_dev, int max_kv_len, long total_kv_len) {
  if (!layer || (kv_len_dev && max_kv_len <= 0)) return GPU_OPS_E_INVALID;
  as_layer(layer)->SetSharedLens(kv_len_dev, max_kv_len, total_kv_len);
  return GPU_OPS_OK;
}

void *gpu_decode_step_create(int max_batch, int n_heads, int n_kv_heads, int dt) {
  DecodeStep *step = new DecodeStep();
  if (!step->Init(max_batch, n_heads, n_kv_heads, static_cast<DataType>(dt))) {
    delete step;
    return nullptr;
  }
  return step;
}

void gpu_decode_step_destroy(void *step) { delete static_cast<DecodeStep *>(step); }

int gpu_decode_step_prepare(void *step, const int32_t *kv_len_host, int batch, int append_new, gpu_stream_t stream) {
  if (!step) return GPU_OPS_E_INVALID;
  return static_cast<DecodeStep *>(step)->Prepare(kv_len_host, batch, append_new != 0, static_cast<cudaStream_t>(stream));
}

int gpu_attention_layer_set_shared_step(void *layer, void *step) {
  if (!layer) return GPU_OPS_E_INVALID;
  as_layer(layer)->SetSharedStep(static_cast<DecodeStep *>(step));
  return GPU_OPS_OK;
}

size_t gpu_kv_cache_layout(gpu_attn_desc *desc, int cache_layout, int n_kv_heads, int max_seq_len, int head_dim) {
  if (!desc || n_kv_heads <= 0 || max_seq_len <= 0 || head_dim <= 0 || (cache_layout != 0 && cache_layout != 1)) return 0;
  return KVCacheLayout(desc, cache_layout == 0 ? CacheLayout::TokenMajor : CacheLayout::HeadMajor, n_kv_heads, max_seq_len,
                       head_dim);
}

int gpu_attention_layer_forward_host(void *layer, void *out_host, const void *qkv_host, int batch, int cur_pos,
                                     int prev_pos, const int32_t *kv_len_host, gpu_stream_t stream) {
  if (!layer || !out_host || !qkv_host || cur_pos < prev_pos || prev_pos < 0) return GPU_OPS_E_INVALID;
  InferenceCtx ctx(cur_pos, prev_pos);
  ctx.gpu_stream = static_cast<cudaStream_t>(stream);
  return as_layer(layer)->ForwardHost(out_host, qkv_host, ctx, batch, kv_len_host);
}

int gpu_attention_layer_set_host_copy_overlap(void *layer, int on) {
  if (!layer) return GPU_OPS_E_INVALID;
  as_layer(layer)->SetHostCopyOverlap(on != 0);
  return GPU_OPS_OK;
}

int gpu_attention_layer_forward_fused(void *layer, void *out, const void *qkv, const void *qkv_bias, int batch,
                                      int cur_pos, int prev_pos, const int32_t *kv_len_host, gpu_stream_t stream) {
  if (!layer || !out || !qkv || cur_pos < prev_pos || prev_pos < 0) return GPU_OPS_E_INVALID;
  InferenceCtx ctx(cur_pos, prev_pos);
  ctx.gpu_stream = static_cast<cudaStream_t>(stream);
  return as_layer(layer)->ForwardFused(out, qkv, qkv_bias, ctx, batch, kv_len_host);
}

int gpu_attention_layer_cache(void *layer, void **k_cache, void **v_cache) {
  if (!layer || !k_cache || !v_cache) return GPU_OPS_E_INVALID;
  *k_cache = as_layer(layer)->k_cache_ptr();
  *v_cache = as_layer(layer)->v_cache_ptr();
  return GPU_OPS_OK;
}

} // extern "C"
