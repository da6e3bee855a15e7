#include "attention_layer_gpu.hpp"

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>

// ---- RoPE table (src/model_base.cpp:27-66, src/util.cpp:33-72) -------------------
static uint16_t fp32_to_bfloat16_rne(uint32_t bits) {
  const uint32_t sign = (bits >> 31) & 1u, exponent = (bits >> 23) & 0xffu;
  const uint32_t sig = (bits & 0x007fffffu) | 0x00800000u;
  uint32_t hi = (sig >> 16) & 0xffu;
  const uint32_t lo = sig & 0xffffu;
  if (lo > 0x8000u || (lo == 0x8000u && (hi & 1u))) hi += 1;
  uint32_t e = exponent;
  if (hi > 0xffu) {
    e += 1;
    hi = 0x80u;
  }
  if (e > 0xffu) e = 0xffu;
  return static_cast<uint16_t>((sign << 15) | (e << 7) | (hi & 0x7fu));
}

void InitFreqCIS(float *out, int head_dim, int max_seq_len, float theta, DataType dt) {
  const int freq_len = head_dim / 2;
  std::vector<float> freq(freq_len);
  for (int i = 0; i < freq_len; ++i)
    freq[i] = 1.0f / (std::pow(theta, static_cast<double>(i * 2) / static_cast<double>(head_dim)));
  for (int pos = 0; pos < max_seq_len; ++pos) {
    const float t = static_cast<float>(pos);
    for (int j = 0; j < freq_len; ++j) {
      const float angle = t * freq[j];
      float c = std::cos(angle), s = std::sin(angle);
      if (dt == DT_BFLOAT16) {
        uint32_t u;
        std::memcpy(&u, &c, 4);
        u = static_cast<uint32_t>(fp32_to_bfloat16_rne(u)) << 16;
        std::memcpy(&c, &u, 4);
        std::memcpy(&u, &s, 4);
        u = static_cast<uint32_t>(fp32_to_bfloat16_rne(u)) << 16;
        std::memcpy(&s, &u, 4);
      }
      out[(static_cast<size_t>(pos) * freq_len + j) * 2] = c;
      out[(static_cast<size_t>(pos) * freq_len + j) * 2 + 1] = s;
    }
  }
}

// ---- cache layout and per-step state ------------------------------------------------
size_t KVCacheLayout(gpu_attn_desc *desc, CacheLayout layout, int n_kv_heads, int max_seq_len, int head_dim) {
  const long D = head_dim;
  desc->cache_seq_stride = static_cast<long>(n_kv_heads) * max_seq_len * D;
  if (layout == CacheLayout::HeadMajor) {
    desc->cache_head_stride = static_cast<long>(max_seq_len) * D;
    desc->cache_pos_stride = D;
  } else {
    desc->cache_head_stride = D;
    desc->cache_pos_stride = n_kv_heads * D;
  }
  return static_cast<size_t>(desc->cache_seq_stride);
}

DecodeStep::~DecodeStep() {
  for (int i = 0; i < 2; ++i) {
    if (uploaded_[i]) cudaEventDestroy(uploaded_[i]);
    if (pinned_[i]) cudaFreeHost(pinned_[i]);
  }
}

bool DecodeStep::Init(int max_batch, int n_heads, int n_kv_heads, DataType dt) {
  if (pinned_[0] || max_batch <= 0 || n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return false;
  desc_ = gpu_attn_desc{};
  desc_.dtype = static_cast<int32_t>(dt);
  desc_.batch = max_batch;
  desc_.n_heads = n_heads;
  desc_.n_kv_heads = n_kv_heads;
  desc_.head_dim = 128;
  plan_bytes_ = gpu_attn_decode_plan_bytes(&desc_, 0);
  if (!plan_bytes_) return false;
  // scratch for the most pieces a plan can have: one per cache plus one per cut
  const size_t max_slots = static_cast<size_t>(max_batch) * n_kv_heads + 1024;
  workspace_bytes_ = max_slots * static_cast<size_t>(n_heads / n_kv_heads) * 129 * sizeof(float);
  for (int i = 0; i < 2; ++i) {
    if (cudaHostAlloc(&pinned_[i], plan_bytes_, cudaHostAllocDefault) != cudaSuccess) return false;
    if (cudaEventCreateWithFlags(&uploaded_[i], cudaEventDisableTiming) != cudaSuccess) return false;
  }
  plan_dev_ = Tensor::MakeGPUTensor(plan_bytes_, DT_UINT8);
  workspace_ = Tensor::MakeGPUTensor(workspace_bytes_, DT_UINT8);
  return plan_dev_->data_ptr && workspace_->data_ptr;
}

int DecodeStep::Prepare(const int32_t *kv_len_host, int batch, bool append_new, cudaStream_t stream) {
  if (!pinned_[0] || !kv_len_host || batch <= 0 || batch > desc_.batch) return GPU_OPS_E_INVALID;
  const int slot = cur_ < 0 ? 0 : 1 - cur_;
  // the buffer last served the step before the previous one: its upload has long been read
  if (in_flight_[slot] && cudaEventSynchronize(uploaded_[slot]) != cudaSuccess) return GPU_OPS_E_CUDA;
  gpu_attn_desc d = desc_;
  d.batch = batch;
  if (int rc = gpu_attn_decode_plan(&d, kv_len_host, append_new ? 1 : 0, 0, pinned_[slot], plan_bytes_)) return rc;
  const size_t used = gpu_attn_decode_plan_size(pinned_[slot]);
  if (gpu_attn_decode_plan_workspace_bytes(pinned_[slot]) > workspace_bytes_) return GPU_OPS_E_WORKSPACE;
  if (cudaMemcpyAsync(plan_dev_->data_ptr, pinned_[slot], used, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
      cudaEventRecord(uploaded_[slot], stream) != cudaSuccess)
    return GPU_OPS_E_CUDA;
  in_flight_[slot] = true;
  cur_ = slot;
  batch_ = batch;
  return GPU_OPS_OK;
}

// ---- layer -----------------------------------------------------------------------
AttentionLayerGPUImpl::~AttentionLayerGPUImpl() { UnInit(); }

void AttentionLayerGPUImpl::UnInit() {
  k_cache.reset();
  v_cache.reset();
  freq_cis_owned_.reset();
  workspace_.reset();
  staging_in_.reset();
  staging_out_.reset();
  staging_in_bytes_ = staging_out_bytes_ = 0;
  if (in_ready_) cudaEventDestroy(in_ready_);
  if (in_free_) cudaEventDestroy(in_free_);
  if (copy_stream_) cudaStreamDestroy(copy_stream_); // returns at once; the stream goes when its work is done
  in_ready_ = in_free_ = nullptr;
  copy_stream_ = nullptr;
  in_free_recorded_ = false;
  own_step_.reset();
  k_cache_raw_ = v_cache_raw_ = nullptr;
  freq_cis_ = nullptr;
  shared_lens_ = nullptr;
  shared_step_ = nullptr;
}

bool AttentionLayerGPUImpl::Init(const AttentionConfig &cfg, const float *shared_freq_cis, void *k_cache_ext,
                                 void *v_cache_ext) {
  UnInit();
  if (cfg.n_heads <= 0 || cfg.n_kv_heads <= 0 || cfg.n_heads % cfg.n_kv_heads || cfg.head_dim != 128 ||
      cfg.max_seq_len <= 0 || cfg.max_batch <= 0 || (cfg.data_type != DT_FLOAT16 && cfg.data_type != DT_BFLOAT16) ||
      (k_cache_ext == nullptr) != (v_cache_ext == nullptr)) {
    std::fprintf(stderr, "AttentionLayerGPUImpl::Init: invalid configuration\n");
    return false;
  }
  cfg_ = cfg;
  // cache: reference allocates kvH * D * max_seq_len 16-bit elements per layer
  // (src/llama2_layer_npu.cpp:726-727, :1148-1149); here once per sequence of the batch
  const size_t cache_elems = static_cast<size_t>(cfg.max_batch) * cfg.n_kv_heads * cfg.max_seq_len * cfg.head_dim;
  if (k_cache_ext) {
    k_cache_raw_ = k_cache_ext;
    v_cache_raw_ = v_cache_ext;
  } else {
    k_cache = Tensor::MakeGPUTensor(cache_elems, cfg.data_type);
    v_cache = Tensor::MakeGPUTensor(cache_elems, cfg.data_type);
    if (!k_cache->data_ptr || !v_cache->data_ptr) return false;
    k_cache_raw_ = k_cache->data_ptr;
    v_cache_raw_ = v_cache->data_ptr;
  }
  if (shared_freq_cis) {
    freq_cis_ = shared_freq_cis;
  } else {
    const size_t n = static_cast<size_t>(cfg.max_seq_len) * cfg.head_dim;
    auto host = Tensor::MakeCPUTensor(n, DT_FLOAT32);
    InitFreqCIS(static_cast<float *>(host->data_ptr), cfg.head_dim, cfg.max_seq_len, cfg.rope_theta, cfg.data_type);
    freq_cis_owned_ = host->to(DEV_GPU);
    if (!freq_cis_owned_ || !freq_cis_owned_->data_ptr) return false;
    freq_cis_ = static_cast<const float *>(freq_cis_owned_->data_ptr);
  }
  gpu_attn_desc d = MakeDesc(cfg.max_batch, 1, 0, 0, 0, 0);
  workspace_bytes_ = gpu_attn_decode_workspace_bytes(&d, cfg.max_seq_len);
  workspace_ = Tensor::MakeGPUTensor(workspace_bytes_ > 0 ? workspace_bytes_ : 16, DT_UINT8);
  return workspace_->data_ptr != nullptr;
}

gpu_attn_desc AttentionLayerGPUImpl::MakeDesc(int batch, int m, long q_tok, long q_seq, long kv_tok, long kv_seq) const {
  gpu_attn_desc d{};
  const long D = cfg_.head_dim;
  d.dtype = static_cast<int32_t>(cfg_.data_type);
  d.batch = batch;
  d.n_heads = cfg_.n_heads;
  d.n_kv_heads = cfg_.n_kv_heads;
  d.head_dim = cfg_.head_dim;
  d.is_neox_style = cfg_.rope_is_neox_style ? 1 : 0;
  d.q_tok_stride = q_tok ? q_tok : cfg_.n_heads * D;
  d.q_seq_stride = q_seq ? q_seq : m * d.q_tok_stride;
  d.kv_in_tok_stride = kv_tok ? kv_tok : cfg_.n_kv_heads * D;
  d.kv_in_seq_stride = kv_seq ? kv_seq : m * d.kv_in_tok_stride;
  d.out_tok_stride = cfg_.n_heads * D;
  d.out_seq_stride = m * d.out_tok_stride;
  KVCacheLayout(&d, cfg_.cache_layout, cfg_.n_kv_heads, cfg_.max_seq_len, cfg_.head_dim);
  return d;
}

int AttentionLayerGPUImpl::DecodeStepCall(gpu_attn_desc &d, void *out, const void *q, const void *k, const void *v,
                                          const int32_t *kv_len_host, int uniform_len, int batch, cudaStream_t stream) {
  const DecodeStep *step = shared_step_;
  if (!step && shared_lens_) {
    d.total_kv_len = shared_total_;
    return gpu_attn_decode_layer(&d, out, nullptr, nullptr, q, k, v, k_cache_raw_, v_cache_raw_, freq_cis_, shared_lens_,
                                 nullptr, 1, shared_max_len_, workspace_->data_ptr, workspace_bytes_, stream);
  }
  if (!step) {
    // no state shared by the model: cut the work for this call
    std::vector<int32_t> uniform;
    if (!kv_len_host) {
      uniform.assign(batch, uniform_len);
      kv_len_host = uniform.data();
    }
    for (int b = 0; b < batch; ++b)
      if (kv_len_host[b] < 0 || kv_len_host[b] + 1 > cfg_.max_seq_len) return GPU_OPS_E_INVALID;
    if (!own_step_) {
      own_step_.reset(new DecodeStep());
      if (!own_step_->Init(cfg_.max_batch, cfg_.n_heads, cfg_.n_kv_heads, cfg_.data_type)) {
        own_step_.reset();
        return GPU_OPS_E_CUDA;
      }
    }
    if (int rc = own_step_->Prepare(kv_len_host, batch, true, stream)) return rc;
    step = own_step_.get();
  }
  if (!step->ready() || step->batch() != batch) return GPU_OPS_E_INVALID;
  return gpu_attn_decode_planned_layer(&d, nullptr, step->plan_host(), step->plan_dev(), out, nullptr, nullptr, q, k, v,
                                       k_cache_raw_, v_cache_raw_, freq_cis_, nullptr, step->workspace(),
                                       step->workspace_bytes(), stream);
}

int AttentionLayerGPUImpl::ForwardRaw(void *out, const void *q, const void *k, const void *v, InferenceCtx &ctx,
                                      int batch) {
  if (batch <= 0 || batch > cfg_.max_batch || ctx.cur_size <= 0 || ctx.prev_pos < 0 || ctx.cur_pos > cfg_.max_seq_len)
    return GPU_OPS_E_INVALID;
  cudaStream_t s = ctx.gpu_stream;
  if (ctx.cur_size == 1) {
    // decode: every sequence sits at prev_pos
    std::vector<int32_t> lens(batch, ctx.prev_pos);
    return DecodeRagged(out, q, k, v, lens.data(), batch, s);
  }
  gpu_attn_desc d = MakeDesc(batch, ctx.cur_size, 0, 0, 0, 0);
  // rotate Q in a pooled temporary (the reference's q_emb), K/V straight into the cache
  auto q_emb = Tensor::MakeGPUTensor(static_cast<size_t>(batch) * ctx.cur_size * cfg_.n_heads * cfg_.head_dim,
                                     cfg_.data_type);
  if (!q_emb->data_ptr) return GPU_OPS_E_CUDA;
  int rc = gpu_rope_kv_append_layer(&d, q_emb->data_ptr, k_cache_raw_, v_cache_raw_, q, k, v, freq_cis_, nullptr,
                                    ctx.prev_pos, ctx.cur_size, s);
  if (rc) return rc;
  rc = gpu_attn_prefill_layer(&d, out, q_emb->data_ptr, k_cache_raw_, v_cache_raw_, ctx.cur_size, ctx.prev_pos, s);
  // q_emb returns to the pool when it goes out of scope; the pool is not
  // stream-aware, and later users of the block are ordered after this kernel
  // because the layer issues everything on the same stream.
  return rc;
}

int AttentionLayerGPUImpl::DecodeRagged(void *out, const void *q, const void *k, const void *v,
                                        const int32_t *kv_len_host, int batch, cudaStream_t stream) {
  if (batch <= 0 || batch > cfg_.max_batch) return GPU_OPS_E_INVALID;
  if (!kv_len_host && !shared_step_ && !shared_lens_) return GPU_OPS_E_INVALID;
  gpu_attn_desc d = MakeDesc(batch, 1, 0, 0, 0, 0);
  return DecodeStepCall(d, out, q, k, v, kv_len_host, 0, batch, stream);
}

std::shared_ptr<Tensor> AttentionLayerGPUImpl::Forward(std::shared_ptr<Tensor> q, std::shared_ptr<Tensor> k,
                                                       std::shared_ptr<Tensor> v, InferenceCtx &ctx, int batch) {
  auto out = Tensor::MakeGPUTensor(static_cast<size_t>(batch) * ctx.cur_size * cfg_.n_heads * cfg_.head_dim,
                                   cfg_.data_type);
  if (!out->data_ptr) return nullptr;
  if (ForwardRaw(out->data_ptr, q->data_ptr, k->data_ptr, v->data_ptr, ctx, batch) != GPU_OPS_OK) return nullptr;
  return out;
}

int AttentionLayerGPUImpl::ForwardFused(void *out, const void *qkv, const void *bias, InferenceCtx &ctx, int batch,
                                        const int32_t *kv_len_host) {
  if (batch <= 0 || batch > cfg_.max_batch || ctx.cur_size <= 0 || ctx.prev_pos < 0 || ctx.cur_pos > cfg_.max_seq_len)
    return GPU_OPS_E_INVALID;
  const long D = cfg_.head_dim;
  const long row = (cfg_.n_heads + 2L * cfg_.n_kv_heads) * D;
  cudaStream_t s = ctx.gpu_stream;
  if (ctx.cur_size > 1) {
    gpu_attn_desc d = MakeDesc(batch, ctx.cur_size, 0, 0, 0, 0);
    auto q_emb = Tensor::MakeGPUTensor(static_cast<size_t>(batch) * ctx.cur_size * cfg_.n_heads * D, cfg_.data_type);
    if (!q_emb->data_ptr) return GPU_OPS_E_CUDA;
    int rc = gpu_qkv_rope_kv_append_layer(&d, q_emb->data_ptr, k_cache_raw_, v_cache_raw_, qkv, ctx.cur_size * row, row,
                                          bias, freq_cis_, nullptr, ctx.prev_pos, ctx.cur_size, s);
    if (rc) return rc;
    return gpu_attn_prefill_layer(&d, out, q_emb->data_ptr, k_cache_raw_, v_cache_raw_, ctx.cur_size, ctx.prev_pos, s);
  }
  // one token per sequence: the decode kernel reads q, k, v as columns of the packed row
  std::shared_ptr<Tensor> biased;
  const char *base = static_cast<const char *>(qkv);
  if (bias) {
    biased = Tensor::MakeGPUTensor(static_cast<size_t>(batch) * row, cfg_.data_type);
    if (!biased->data_ptr) return GPU_OPS_E_CUDA;
    int rc = gpu_bias_add_layer(biased->data_ptr, qkv, bias, batch, static_cast<int>(row), row,
                                static_cast<int>(cfg_.data_type), s);
    if (rc) return rc;
    base = static_cast<const char *>(biased->data_ptr);
  }
  const void *q = base, *k = base + cfg_.n_heads * D * 2, *v = base + (cfg_.n_heads + cfg_.n_kv_heads) * D * 2;
  gpu_attn_desc d = MakeDesc(batch, 1, row, row, row, row);
  return DecodeStepCall(d, out, q, k, v, kv_len_host, ctx.prev_pos, batch, s);
}

int AttentionLayerGPUImpl::ForwardHost(void *out_host, const void *qkv_host, InferenceCtx &ctx, int batch,
                                       const int32_t *kv_len_host) {
  if (batch <= 0 || batch > cfg_.max_batch || ctx.cur_size <= 0 || ctx.prev_pos < 0 || ctx.cur_pos > cfg_.max_seq_len)
    return GPU_OPS_E_INVALID;
  const long D = cfg_.head_dim;
  const long row = (cfg_.n_heads + 2L * cfg_.n_kv_heads) * D;
  const size_t in_bytes = static_cast<size_t>(batch) * ctx.cur_size * row * 2;
  const size_t out_bytes = static_cast<size_t>(batch) * ctx.cur_size * cfg_.n_heads * D * 2;
  if (in_bytes > staging_in_bytes_) {
    staging_in_bytes_ = 0;
    staging_in_ = Tensor::MakeGPUTensor(in_bytes, DT_UINT8);
    if (!staging_in_ || !staging_in_->data_ptr) return GPU_OPS_E_CUDA;
    staging_in_bytes_ = in_bytes;
  }
  if (out_bytes > staging_out_bytes_) {
    staging_out_bytes_ = 0;
    staging_out_ = Tensor::MakeGPUTensor(out_bytes, DT_UINT8);
    if (!staging_out_ || !staging_out_->data_ptr) return GPU_OPS_E_CUDA;
    staging_out_bytes_ = out_bytes;
  }
  cudaStream_t s = ctx.gpu_stream;
  // The input goes up on the layer's own stream, so that it does not queue behind the kernels the
  // caller's stream still holds; a stream under capture keeps everything in its own order.
  bool overlap = overlap_host_copies_, capturing_stream = false;
  if (overlap) {
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone)
      overlap = false, capturing_stream = true;
  }
  if (overlap && !copy_stream_) {
    if (cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&in_ready_, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&in_free_, cudaEventDisableTiming) != cudaSuccess)
      return GPU_OPS_E_CUDA;
  }
  if (overlap) {
    // not before the previous call's kernels have read (prefill: rotated in place) the buffer
    if (in_free_recorded_ && cudaStreamWaitEvent(copy_stream_, in_free_, 0) != cudaSuccess) return GPU_OPS_E_CUDA;
    if (cudaMemcpyAsync(staging_in_->data_ptr, qkv_host, in_bytes, cudaMemcpyHostToDevice, copy_stream_) != cudaSuccess ||
        cudaEventRecord(in_ready_, copy_stream_) != cudaSuccess || cudaStreamWaitEvent(s, in_ready_, 0) != cudaSuccess)
      return GPU_OPS_E_CUDA;
  } else {
    if (cudaMemcpyAsync(staging_in_->data_ptr, qkv_host, in_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess)
      return GPU_OPS_E_CUDA;
  }
  const char *base = static_cast<const char *>(staging_in_->data_ptr);
  const void *q = base, *k = base + cfg_.n_heads * D * 2, *v = base + (cfg_.n_heads + cfg_.n_kv_heads) * D * 2;
  int rc;
  // A one-token step writes a few hundred KB of output rows: when out_host is pinned memory the kernels
  // store them there themselves (the device address of the same bytes) and no copy is queued behind them.
  void *out_dev = staging_out_->data_ptr;
  if (ctx.cur_size == 1 && overlap_host_copies_) {
    // asked on every call: the buffer behind an address may have been freed and replaced since the last one
    cudaPointerAttributes at{};
    if (cudaPointerGetAttributes(&at, out_host) == cudaSuccess && at.type == cudaMemoryTypeHost && at.devicePointer &&
        reinterpret_cast<uintptr_t>(at.devicePointer) % 16 == 0)
      out_dev = at.devicePointer;
    else
      cudaGetLastError(); // an address the runtime does not know leaves an error behind
  }
  const bool direct_out = out_dev != staging_out_->data_ptr;
  if (ctx.cur_size == 1) {
    // q, k, v are columns of one packed row: strides say so
    gpu_attn_desc d = MakeDesc(batch, 1, row, row, row, row);
    rc = DecodeStepCall(d, out_dev, q, k, v, kv_len_host, ctx.prev_pos, batch, s);
  } else {
    gpu_attn_desc d = MakeDesc(batch, ctx.cur_size, row, ctx.cur_size * row, row, ctx.cur_size * row);
    // rotate Q in place inside the staging buffer
    rc = gpu_rope_kv_append_layer(&d, const_cast<void *>(q), k_cache_raw_, v_cache_raw_, q, k, v, freq_cis_, nullptr,
                                  ctx.prev_pos, ctx.cur_size, s);
    if (!rc)
      rc = gpu_attn_prefill_layer(&d, staging_out_->data_ptr, q, k_cache_raw_, v_cache_raw_, ctx.cur_size,
                                  ctx.prev_pos, s);
  }
  if (overlap_host_copies_) {
    // whichever way this call's input came, the next overlapped copy must wait for these kernels
    if (!in_free_ && cudaEventCreateWithFlags(&in_free_, cudaEventDisableTiming) != cudaSuccess) return GPU_OPS_E_CUDA;
    if (!capturing_stream) {
      if (cudaEventRecord(in_free_, s) != cudaSuccess) return GPU_OPS_E_CUDA;
      in_free_recorded_ = true;
    }
  }
  if (rc) return rc;
  if (!direct_out &&
      cudaMemcpyAsync(out_host, staging_out_->data_ptr, out_bytes, cudaMemcpyDeviceToHost, s) != cudaSuccess)
    return GPU_OPS_E_CUDA;
  return GPU_OPS_OK;
}

bool Llamma2AttentionGPUImpl::Init(const AttentionConfig &cfg, const float *shared_freq_cis, void *k_cache_ext,
                                   void *v_cache_ext) {
  AttentionConfig c = cfg;
  c.n_kv_heads = c.n_heads;     // MHA: the cache holds n_heads * head_dim per position
  c.data_type = DT_FLOAT16;     // src/llama2_main.cpp:172
  return AttentionLayerGPUImpl::Init(c, shared_freq_cis, k_cache_ext, v_cache_ext);
}

bool Qwen2AttentionGPUImpl::Init(const AttentionConfig &cfg, const float *shared_freq_cis, void *k_cache_ext,
                                 void *v_cache_ext) {
  return AttentionLayerGPUImpl::Init(cfg, shared_freq_cis, k_cache_ext, v_cache_ext);
}
