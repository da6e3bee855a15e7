// The attention section of the transformer layers on the GPU backend.
//
// Mirrors what Llamma2TransformerLayerNPUImpl / Qwen2TransformerLayerNPUImpl
// (src/llama2_layer_npu.hpp:43-95) hold and do between the Q/K/V projections and
// o_proj (src/llama2_layer_npu.cpp:283-374, :780-869): members k_cache / v_cache,
// the RoPE table, and a Forward that rotates, appends and attends.  Everything
// else of those layers (norms, GEMMs, MLP) is outside this library.
//
// Added relative to the reference, which is batch 1: a batch dimension
// (independent sequences with their own cache rows) and ragged decode lengths.
#pragma once

#include <cuda_runtime.h>

#include <memory>
#include <vector>

#include "device.hpp"
#include "gpu_ops.h"

// Same fields as the reference's InferenceCtx (src/model_base.hpp:40-48); the
// stream is a CUDA stream.
class InferenceCtx {
public:
  InferenceCtx(size_t cur_pos, size_t prev_pos) : cur_pos(int(cur_pos)), prev_pos(int(prev_pos)) {
    cur_size = this->cur_pos - this->prev_pos; // src/model_base.cpp:22-25
  }
  int cur_pos;
  int prev_pos;
  int cur_size;
  cudaStream_t gpu_stream{nullptr};
};

// Host builder of the RoPE table, ModelBase::InitFreqCIS (src/model_base.cpp:27-66):
// freq[i] = 1 / pow(theta, 2i / D) in double rounded to float, angle = float(pos) * freq[i]
// in fp32, (cos, sin) interleaved; for DT_BFLOAT16 every value is rounded to bf16
// (ties to even, src/util.cpp:33-72) and stored back as fp32.
// out: [max_seq_len][head_dim/2][2].
void InitFreqCIS(float *out, int head_dim, int max_seq_len, float theta, DataType dt);

enum class CacheLayout { TokenMajor = 0, HeadMajor = 1 };

// The three cache strides of gpu_attn_desc for a per-layer KV cache of `max_seq_len` positions per
// sequence: token-major [seq][pos][kv_head][D] is the reference's layout
// (src/llama2_layer_npu.cpp:1148-1149: kvH * D * max_seq_len elements, appended at byte offset
// prev_pos * kvH * D * 2, :830-843), head-major [seq][kv_head][pos][D] keeps one head's positions
// contiguous.  Returns the elements one sequence occupies.
size_t KVCacheLayout(gpu_attn_desc *desc, CacheLayout layout, int n_kv_heads, int max_seq_len, int head_dim);

// What a model prepares once per decode step for all its layers: the work partition of the step
// (gpu_attn_decode_plan) for the sequences' cache lengths, which the host knows as the reference's
// generation loop knows cur_pos / prev_pos (src/model_base.hpp:40-48), its device copy and the
// scratch of the planned decode kernel.  Prepare() never waits for the stream: the plan is built
// in one of two pinned buffers used by alternate steps (an event tells when a buffer's upload has
// been read) and the device copy is overwritten in stream order, behind the previous step's kernels.
class DecodeStep {
public:
  ~DecodeStep();
  bool Init(int max_batch, int n_heads, int n_kv_heads, DataType dt);
  // kv_len_host: tokens already cached per sequence.  Enqueues the upload on `stream`; the layers'
  // calls of this step must follow on the same stream.
  int Prepare(const int32_t *kv_len_host, int batch, bool append_new, cudaStream_t stream);
  bool ready() const { return cur_ >= 0; }
  int batch() const { return batch_; }
  const void *plan_host() const { return cur_ >= 0 ? pinned_[cur_] : nullptr; }
  const void *plan_dev() const { return plan_dev_ ? plan_dev_->data_ptr : nullptr; }
  void *workspace() const { return workspace_ ? workspace_->data_ptr : nullptr; }
  size_t workspace_bytes() const { return workspace_bytes_; }

private:
  gpu_attn_desc desc_{};
  size_t plan_bytes_{0}, workspace_bytes_{0};
  void *pinned_[2] = {nullptr, nullptr};
  cudaEvent_t uploaded_[2] = {nullptr, nullptr};
  bool in_flight_[2] = {false, false};
  int cur_{-1}, batch_{0};
  std::shared_ptr<Tensor> plan_dev_, workspace_;
};

struct AttentionConfig {
  int n_heads{0};
  int n_kv_heads{0};
  int head_dim{128};
  int max_seq_len{2048};
  int max_batch{1};
  DataType data_type{DT_FLOAT16};
  float rope_theta{10000.0f};
  bool rope_is_neox_style{false};
  CacheLayout cache_layout{CacheLayout::HeadMajor};
};

class AttentionLayerGPUImpl {
public:
  virtual ~AttentionLayerGPUImpl();

  // Allocates the caches ([max_batch] x layout of [max_seq_len][n_kv_heads][D]),
  // the decode scratch and the RoPE table (or adopts `shared_freq_cis`, a device
  // table built once per model as the reference does).  External cache memory
  // may be adopted instead of allocated (both or neither).
  virtual bool Init(const AttentionConfig &cfg, const float *shared_freq_cis = nullptr, void *k_cache_ext = nullptr,
                    void *v_cache_ext = nullptr);
  virtual void UnInit();

  // Attention section for `batch` sequences that all sit at ctx.prev_pos and
  // receive ctx.cur_size new tokens: q [batch][cur_size][n_heads*D],
  // k, v [batch][cur_size][n_kv_heads*D] raw projections (device).  Returns the
  // [batch][cur_size][n_heads*D] tensor that feeds o_proj.
  std::shared_ptr<Tensor> Forward(std::shared_ptr<Tensor> q, std::shared_ptr<Tensor> k, std::shared_ptr<Tensor> v,
                                  InferenceCtx &ctx, int batch = 1);

  // Same on raw device pointers, output preallocated by the caller.
  int ForwardRaw(void *out, const void *q, const void *k, const void *v, InferenceCtx &ctx, int batch);

  // One decode step with per-sequence cache lengths (host array, `batch` entries).
  int DecodeRagged(void *out, const void *q, const void *k, const void *v, const int32_t *kv_len_host, int batch,
                   cudaStream_t stream);

  // Device entry fed from a fused projection output: qkv [batch][cur_size][(n_heads +
  // 2 n_kv_heads)*D] (the tensor npu_split_qkv_layer would split), bias one such row or
  // NULL (the q/k/v biases of the Qwen2 projections, src/llama2_layer_npu.cpp:1020-1055,
  // when the projection itself does not add them).  Split, bias, RoPE and append happen
  // in one pass over the row; the one-token step adds the bias in a small pass of its
  // own and leaves the rest to the decode kernel.  kv_len_host as in ForwardHost.
  int ForwardFused(void *out, const void *qkv, const void *bias, InferenceCtx &ctx, int batch,
                   const int32_t *kv_len_host);

  // Host-buffer entry: q/k/v packed as [batch][cur_size][(n_heads + 2 n_kv_heads)*D]
  // in (pinned) host memory, output to host memory.  The kernels and the copy of the
  // output are enqueued on the stream.  The copy of the input runs on a stream of the
  // layer's own and the caller's stream waits for it, so it overlaps whatever the
  // caller's stream is still busy with (the previous layer's kernels): qkv_host must
  // hold its data when the call is made and keep it until the stream has passed the
  // call.  In a one-token step with out_host in pinned memory the kernels store the
  // output rows into out_host themselves (no copy behind them).  SetHostCopyOverlap(false)
  // puts both copies on the caller's stream, in its order; a stream that is being captured
  // keeps the input copy on itself.  kv_len_host == NULL: uniform ctx.prev_pos.
  int ForwardHost(void *out_host, const void *qkv_host, InferenceCtx &ctx, int batch, const int32_t *kv_len_host);
  void SetHostCopyOverlap(bool on) { overlap_host_copies_ = on; }

  // Per-step state shared by all layers of a model: the device array of cache
  // lengths (tokens already cached per sequence) and its maximum + 1.  While
  // set, decode calls use it instead of uploading their own copy (one upload per
  // step by the model instead of one per layer).  NULL unsets.
  // total_kv_len: sum over the batch of kv_len + 1 (scheduling hint; 0 = unknown).
  void SetSharedLens(const int32_t *kv_len_dev, int max_kv_len, long total_kv_len = 0) {
    shared_lens_ = kv_len_dev;
    shared_max_len_ = max_kv_len;
    shared_total_ = total_kv_len;
  }
  // The step state the model prepared for all its layers (DecodeStep::Prepare): while set, decode
  // calls run the planned kernel on it and ignore their own length arguments.  NULL unsets.
  void SetSharedStep(const DecodeStep *step) { shared_step_ = step; }

  const AttentionConfig &config() const { return cfg_; }
  void *k_cache_ptr() const { return k_cache_raw_; }
  void *v_cache_ptr() const { return v_cache_raw_; }

  std::shared_ptr<Tensor> k_cache; // owned caches (empty when external memory was adopted)
  std::shared_ptr<Tensor> v_cache;

protected:
  gpu_attn_desc MakeDesc(int batch, int m, long q_tok, long q_seq, long kv_tok, long kv_seq) const;
  // One decode step for q / k / v addressed by `d`: on the shared step state, on the shared device
  // lengths, or on a plan built here from kv_len_host (NULL: every sequence holds uniform_len tokens).
  int DecodeStepCall(gpu_attn_desc &d, void *out, const void *q, const void *k, const void *v,
                     const int32_t *kv_len_host, int uniform_len, int batch, cudaStream_t stream);

  AttentionConfig cfg_;
  void *k_cache_raw_{nullptr};
  void *v_cache_raw_{nullptr};
  std::shared_ptr<Tensor> freq_cis_owned_;
  const float *freq_cis_{nullptr};
  std::shared_ptr<Tensor> workspace_;
  size_t workspace_bytes_{0};
  std::unique_ptr<DecodeStep> own_step_; // for calls that come with host lengths and no shared step
  std::shared_ptr<Tensor> staging_in_, staging_out_; // device side of ForwardHost
  size_t staging_in_bytes_{0}, staging_out_bytes_{0};
  // ForwardHost's input copies: the layer's own stream, "input is on the device" and "the kernels
  // have read the staging buffer" events
  cudaStream_t copy_stream_{nullptr};
  cudaEvent_t in_ready_{nullptr}, in_free_{nullptr};
  bool in_free_recorded_{false};
  bool overlap_host_copies_{true};
  const int32_t *shared_lens_{nullptr};
  int shared_max_len_{0};
  long shared_total_{0};
  const DecodeStep *shared_step_{nullptr};
};

// Llama-2 flavour: MHA, fp16 (the reference forces DT_FLOAT16 for llama2,
// src/llama2_main.cpp:172), RoPE pairing from the flag.
class Llamma2AttentionGPUImpl : public AttentionLayerGPUImpl {
public:
  bool Init(const AttentionConfig &cfg, const float *shared_freq_cis = nullptr, void *k_cache_ext = nullptr,
            void *v_cache_ext = nullptr) override;
};

// Qwen2 flavour: GQA, bf16 or fp16.
class Qwen2AttentionGPUImpl : public AttentionLayerGPUImpl {
public:
  bool Init(const AttentionConfig &cfg, const float *shared_freq_cis = nullptr, void *k_cache_ext = nullptr,
            void *v_cache_ext = nullptr) override;
};
