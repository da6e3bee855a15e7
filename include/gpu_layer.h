/*
 * gpu_layer.h -- C ABI of the host layer of libgpu_ops.so: the GPU device
 * abstraction and the attention section of the transformer layers, as opaque
 * handles.  The C++ classes behind it (llm_simple_b200/csrc/host/) mirror the
 * reference's own (cited per function); this header is what a non-C++ host
 * (tests, benchmark, a binding in another language) links against.
 *
 * Status codes are those of gpu_ops.h.
 */
#ifndef LLM_SIMPLE_GPU_LAYER_H_
#define LLM_SIMPLE_GPU_LAYER_H_

#include <stddef.h>
#include <stdint.h>

#include "gpu_ops.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- device memory pool: GPUAllocator, the counterpart of NPUAllocator
 * (src/device.hpp:24-39, src/device_npu.cpp:22-67).  Tensor::MakeGPUTensor
 * (src/device_npu.cpp:70-77 for the NPU) draws from it. ---- */
void *gpu_allocator_allocate(size_t bytes);
void gpu_allocator_deallocate(void *ptr);
/* out[5] = backend bytes, pooled bytes, backend allocations, pool hits, backend frees */
void gpu_allocator_stats(size_t out[5]);
void gpu_allocator_trim(void);
void gpu_allocator_set_limit(size_t bytes);
/* on != 0: serve the pool from host malloc/free instead of cudaMalloc/cudaFree,
 * so that the pool policy can be exercised on a machine without a GPU. */
void gpu_allocator_use_host_backend(int on);

/* RoPE table as ModelBase::InitFreqCIS builds it (src/model_base.cpp:27-66):
 * host_out [max_seq_len][head_dim/2][2] fp32 (cos, sin); dt = 5 rounds every
 * value to bf16.  Host memory in, host memory out. */
void gpu_init_freq_cis(float *host_out, int head_dim, int max_seq_len, float theta, int dt);

/* ---- KV cache layout: the three cache strides of *desc for a per-layer cache
 * of max_seq_len positions per sequence.  cache_layout 0 = token-major
 * [seq][pos][kv_head][D], the reference's (src/llama2_layer_npu.cpp:1148-1149
 * allocates n_kv_heads * D * max_seq_len elements, :830-843 appends at byte
 * offset prev_pos * n_kv_heads * D * 2); 1 = head-major [seq][kv_head][pos][D].
 * Returns the elements one sequence's K (or V) cache occupies, 0 on bad
 * arguments. ---- */
size_t gpu_kv_cache_layout(gpu_attn_desc *desc, int cache_layout, int n_kv_heads, int max_seq_len,
                           int head_dim);

/* ---- attention section of a transformer layer.  kind 0: Llama-2
 * (Llamma2TransformerLayerNPUImpl, src/llama2_layer_npu.cpp:283-374: MHA, fp16);
 * kind 1: Qwen2 (Qwen2TransformerLayerNPUImpl, :780-869: GQA).  The layer owns
 * its KV cache for max_batch sequences of max_seq_len positions (reference:
 * k_cache / v_cache members, src/llama2_layer_npu.hpp:43-95), the RoPE table
 * (unless shared_freq_cis_dev is given) and the decode scratch.  cache_layout
 * 0 = token-major (reference), 1 = head-major.  k_cache_ext / v_cache_ext: use
 * this device memory for the caches instead of allocating (both or neither).
 * Returns NULL on failure. ---- */
void *gpu_attention_layer_create(int kind, int n_heads, int n_kv_heads, int head_dim, int max_seq_len,
                                 int max_batch, int dt, float rope_theta, int rope_is_neox_style,
                                 int cache_layout, const float *shared_freq_cis_dev, void *k_cache_ext,
                                 void *v_cache_ext);
void gpu_attention_layer_destroy(void *layer);

/* Forward of the attention section with the reference's InferenceCtx meaning
 * (src/model_base.hpp:40-48): cur_size = cur_pos - prev_pos new tokens per
 * sequence, all sequences at prev_pos.  q [batch][cur_size][n_heads*D], k / v
 * [batch][cur_size][n_kv_heads*D] raw projections, out [batch][cur_size][n_heads*D]
 * (device).  cur_size == 1 runs the fused decode step, otherwise fused RoPE +
 * append followed by causal attention. */
int gpu_attention_layer_forward(void *layer, void *out, const void *q, const void *k, const void *v,
                                int batch, int cur_pos, int prev_pos, gpu_stream_t stream);

/* One decode step with a cache length per sequence (host array). */
int gpu_attention_layer_decode_ragged(void *layer, void *out, const void *q, const void *k,
                                      const void *v, const int32_t *kv_len_host, int batch,
                                      gpu_stream_t stream);

/* Cache lengths that a model uploads once per step for all its layers: device
 * int32 [batch], max(kv_len) + 1, and sum(kv_len + 1) (scheduling hint, 0 =
 * unknown).  While set, decode calls use it. */
int gpu_attention_layer_set_shared_lens(void *layer, const int32_t *kv_len_dev, int max_kv_len,
                                        long total_kv_len);

/* State that a model prepares once per decode step for all its layers: the work
 * partition of the step (gpu_attn_decode_plan) for the sequences' cache lengths
 * -- which the host knows, as the reference's generation loop knows cur_pos /
 * prev_pos (src/model_base.hpp:40-48) -- with its device copy and the scratch of
 * the planned decode kernel.  prepare() enqueues the upload on `stream` without
 * waiting for it; the layers' calls of the step follow on the same stream.
 * While a step is set on a layer, its decode calls run
 * gpu_attn_decode_planned_layer on it and ignore their own length arguments.
 * Call with the device current that will run the layers. */
void *gpu_decode_step_create(int max_batch, int n_heads, int n_kv_heads, int dt);
void gpu_decode_step_destroy(void *step);
int gpu_decode_step_prepare(void *step, const int32_t *kv_len_host, int batch, int append_new,
                            gpu_stream_t stream);
int gpu_attention_layer_set_shared_step(void *layer, void *step /* NULL unsets */);

/* The same forward with HOST buffers: qkv_host [batch][cur_size][(n_heads +
 * 2 n_kv_heads)*D] (q, k, v columns of one packed projection row; pinned memory
 * for asynchronous copies), out_host [batch][cur_size][n_heads*D].  The kernels
 * and the copy of the output are enqueued on `stream`; synchronise it before
 * reading out_host.  The copy of the input runs on a stream the layer owns and
 * `stream` waits for it, so that it overlaps the work `stream` still holds (the
 * previous layer's kernels): qkv_host must hold its data when the call is made
 * and keep it until `stream` has passed the call.  In a one-token step whose
 * out_host is pinned memory the kernels store the output rows into out_host
 * themselves and no copy follows them. */
int gpu_attention_layer_forward_host(void *layer, void *out_host, const void *qkv_host, int batch,
                                     int cur_pos, int prev_pos, const int32_t *kv_len_host,
                                     gpu_stream_t stream);

/* on = 0: gpu_attention_layer_forward_host copies its input on `stream` itself,
 * behind the stream's earlier work (for a qkv_host that is filled by that work),
 * and always copies its output from a device buffer.  on = 1 (the default): as
 * described above.  A stream under capture always takes the input copy on itself. */
int gpu_attention_layer_set_host_copy_overlap(void *layer, int on);

/* Device-buffer entry fed from a fused projection output: qkv [batch][cur_size]
 * [(n_heads + 2 n_kv_heads)*D] on the device (the tensor npu_split_qkv_layer,
 * prebuild/npu_ops.h:27-30, would split), qkv_bias one such row or NULL (the
 * Qwen2 q/k/v biases, src/llama2_layer_npu.cpp:1020-1055), out [batch][cur_size]
 * [n_heads*D] on the device.  kv_len_host as for gpu_attention_layer_forward_host. */
int gpu_attention_layer_forward_fused(void *layer, void *out, const void *qkv, const void *qkv_bias,
                                      int batch, int cur_pos, int prev_pos,
                                      const int32_t *kv_len_host, gpu_stream_t stream);

/* Device addresses of the layer's K and V caches. */
int gpu_attention_layer_cache(void *layer, void **k_cache, void **v_cache);

#ifdef __cplusplus
}
#endif
#endif /* LLM_SIMPLE_GPU_LAYER_H_ */
