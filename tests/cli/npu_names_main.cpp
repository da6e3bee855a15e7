// The attention section of a transformer layer written with the reference's
// operator names, compiled against include/npu_ops_compat.hpp: RoPE of the new
// rows, two device-to-device copies into token-major caches at prev_pos, then
// the attention operator over the first cur_pos rows of the caches -- the call
// sequence of src/llama2_layer_npu.cpp:283-374 (--arch llama2: npu_rope_layer,
// npu_flash_attn_opt_prefill_layer) and :780-869 (--arch qwen2:
// npu_rope_single_layer twice, npu_flash_attn_gqa_layer).  One prefill of
// --prompt tokens, then --steps decode steps; every output is compared with
// the CPU checker fed with the same rows.  Also exercises npu_split_qkv_layer
// (the inputs arrive as one fused q|k|v row) and npu_flash_attn_layer (cross-
// check of the first llama2 call).
#include "gpu_op_test_util.h"
#include "npu_ops_compat.hpp"

namespace {
struct InferenceCtx { // src/model_base.hpp:40-48, the fields the attention section reads
  aclrtStream npu_stream;
  int cur_pos, cur_size, prev_pos;
};
int g_handler_calls = 0;
void counting_handler(const char *op, int status, const char *message) {
  ++g_handler_calls;
  std::printf("handler: %s status %d: %s\n", op, status, message);
}
} // namespace

int main(int argc, char **argv) {
  Flags f(argc, argv);
  const bool qwen = f.get("arch", "qwen2") == "qwen2";
  const int head_dim = 128, prompt = f.get_int("prompt", 200), steps = f.get_int("steps", 5);
  const int n_kv_heads = f.get_int("kv_head_num", qwen ? 2 : 8);
  const int n_heads = qwen ? n_kv_heads * f.get_int("group_size", 6) : n_kv_heads;
  const DataType dtype = f.get("dtype", qwen ? "bfloat16" : "float16") == "bfloat16" ? DT_BFLOAT16 : DT_FLOAT16;
  const bool neox = f.get_bool("is_neox", qwen);
  const int max_seq_len = prompt + steps, hidden_dim = n_heads * head_dim, kv_dim = n_kv_heads * head_dim;
  const int total = prompt + steps, row = hidden_dim + 2 * kv_dim;
  std::printf("attention section with the reference's names: %s heads %d/%d prompt %d steps %d dtype %s neox %d\n",
              qwen ? "qwen2" : "llama2", n_heads, n_kv_heads, prompt, steps,
              dtype == DT_BFLOAT16 ? "bfloat16" : "float16", int(neox));

  std::vector<float> table(static_cast<size_t>(max_seq_len) * head_dim);
  cpu_init_freq_cis(table.data(), head_dim, max_seq_len, qwen ? 1e6f : 1e4f, dtype);
  std::vector<uint16_t> qkv; // [total][q | k | v], what a fused projection would produce
  make_random_bits(qkv, static_cast<size_t>(total) * row, dtype, static_cast<uint32_t>(f.get_int("seed", 11)));

  CHECK_CUDA(cudaSetDevice(0));
  InferenceCtx ctx{};
  CHECK_CUDA(cudaStreamCreate(&ctx.npu_stream));
  auto to_dev = [&](const void *src, size_t elems, DataType dt) {
    auto h = Tensor::MakeCPUTensor(elems, dt);
    std::memcpy(h->data_ptr, src, SizeOfTensor(elems, dt));
    return h->to(DEV_GPU);
  };
  auto freq_cis = to_dev(table.data(), table.size(), DT_FLOAT32);
  auto qkv_dev = to_dev(qkv.data(), qkv.size(), dtype);
  auto k_cache = Tensor::MakeGPUTensor(static_cast<size_t>(max_seq_len) * kv_dim, dtype);
  auto v_cache = Tensor::MakeGPUTensor(static_cast<size_t>(max_seq_len) * kv_dim, dtype);
  CHECK_CUDA(cudaMemset(k_cache->data_ptr, 0xff, SizeOfTensor(static_cast<size_t>(max_seq_len) * kv_dim, dtype))); // NaN
  CHECK_CUDA(cudaMemset(v_cache->data_ptr, 0xff, SizeOfTensor(static_cast<size_t>(max_seq_len) * kv_dim, dtype)));

  // checker state: rotated K rows and raw V rows of everything fed so far
  std::vector<uint16_t> k_all(static_cast<size_t>(total) * kv_dim), v_all(k_all.size());
  bool ok = true;
  double worst = 0;

  for (int call = 0; call <= steps; ++call) {
    ctx.prev_pos = call == 0 ? 0 : prompt + call - 1;
    ctx.cur_size = call == 0 ? prompt : 1;
    ctx.cur_pos = ctx.prev_pos + ctx.cur_size;
    const size_t n_q = static_cast<size_t>(ctx.cur_size) * hidden_dim, n_kv = static_cast<size_t>(ctx.cur_size) * kv_dim;
    auto q = Tensor::MakeGPUTensor(n_q, dtype), k = Tensor::MakeGPUTensor(n_kv, dtype), v = Tensor::MakeGPUTensor(n_kv, dtype);
    auto q_emb = Tensor::MakeGPUTensor(n_q, dtype), k_emb = Tensor::MakeGPUTensor(n_kv, dtype);
    auto out = Tensor::MakeGPUTensor(n_q, dtype);
    void *rows = static_cast<uint16_t *>(qkv_dev->data_ptr) + static_cast<size_t>(ctx.prev_pos) * row;
    npu_split_qkv_layer(q->data_ptr, k->data_ptr, v->data_ptr, rows, ctx.cur_size, hidden_dim, kv_dim, kv_dim, dtype,
                        ctx.npu_stream);
    if (qwen) {
      npu_rope_single_layer(q_emb->data_ptr, freq_cis->data_ptr, q->data_ptr, ctx.prev_pos, ctx.cur_size, n_heads,
                            hidden_dim, neox, dtype, ctx.npu_stream);
      npu_rope_single_layer(k_emb->data_ptr, freq_cis->data_ptr, k->data_ptr, ctx.prev_pos, ctx.cur_size, n_kv_heads,
                            kv_dim, neox, dtype, ctx.npu_stream);
    } else {
      npu_rope_layer(q_emb->data_ptr, k_emb->data_ptr, freq_cis->data_ptr, q->data_ptr, k->data_ptr, ctx.prev_pos,
                     ctx.cur_size, n_heads, hidden_dim, neox, dtype, ctx.npu_stream);
    }
    const size_t copy_size = SizeOfTensor(n_kv, dtype), copy_offset = SizeOfTensor(static_cast<size_t>(ctx.prev_pos) * kv_dim, dtype);
    CHECK_CUDA(cudaMemcpyAsync(static_cast<uint8_t *>(k_cache->data_ptr) + copy_offset, k_emb->data_ptr, copy_size,
                               cudaMemcpyDeviceToDevice, ctx.npu_stream));
    CHECK_CUDA(cudaMemcpyAsync(static_cast<uint8_t *>(v_cache->data_ptr) + copy_offset, v->data_ptr, copy_size,
                               cudaMemcpyDeviceToDevice, ctx.npu_stream));
    if (qwen)
      npu_flash_attn_gqa_layer(out->data_ptr, q_emb->data_ptr, k_cache->data_ptr, v_cache->data_ptr, ctx.cur_size,
                               ctx.cur_pos, ctx.prev_pos, n_heads / n_kv_heads, n_kv_heads, head_dim, dtype,
                               ctx.npu_stream);
    else
      npu_flash_attn_opt_prefill_layer(out->data_ptr, q_emb->data_ptr, k_cache->data_ptr, v_cache->data_ptr,
                                       ctx.cur_size, ctx.cur_pos, ctx.prev_pos, n_heads, head_dim, dtype,
                                       ctx.npu_stream);
    CHECK_CUDA(cudaStreamSynchronize(ctx.npu_stream));
    auto out_cpu = out->to(DEV_CPU);

    // the checker on the same rows
    std::vector<uint16_t> q_in(n_q), k_in(n_kv), q_r(n_q), k_r(n_kv);
    for (int t = 0; t < ctx.cur_size; ++t) {
      const uint16_t *src = qkv.data() + static_cast<size_t>(ctx.prev_pos + t) * row;
      std::memcpy(q_in.data() + static_cast<size_t>(t) * hidden_dim, src, hidden_dim * 2);
      std::memcpy(k_in.data() + static_cast<size_t>(t) * kv_dim, src + hidden_dim, kv_dim * 2);
      std::memcpy(v_all.data() + static_cast<size_t>(ctx.prev_pos + t) * kv_dim, src + hidden_dim + kv_dim, kv_dim * 2);
    }
    cpu_rope_single_layer(q_r.data(), table.data(), q_in.data(), ctx.prev_pos, ctx.cur_size, n_heads, hidden_dim, neox, dtype);
    cpu_rope_single_layer(k_r.data(), table.data(), k_in.data(), ctx.prev_pos, ctx.cur_size, n_kv_heads, kv_dim, neox, dtype);
    std::memcpy(k_all.data() + static_cast<size_t>(ctx.prev_pos) * kv_dim, k_r.data(), n_kv * 2);
    std::vector<float> golden(n_q), got(n_q);
    if (cpu_flash_attn_gqa_layer(nullptr, golden.data(), q_r.data(), k_all.data(), v_all.data(), ctx.cur_size, ctx.cur_pos,
                                 ctx.prev_pos, n_heads / n_kv_heads, n_kv_heads, head_dim, dtype, ORACLE_MODE_GOLDEN,
                                 cpu_oracle_max_threads()))
      return 2;
    std::vector<uint16_t> gr(n_q);
    cpu_f32_to_dt(gr.data(), golden.data(), n_q, dtype);
    cpu_dt_to_f32(golden.data(), gr.data(), n_q, dtype);
    cpu_dt_to_f32(got.data(), static_cast<uint16_t *>(out_cpu->data_ptr), n_q, dtype);
    Report r = compare(got, golden, dtype);
    char what[64];
    std::snprintf(what, sizeof what, "call %d (m=%d n=%d offset=%d)", call, ctx.cur_size, ctx.cur_pos, ctx.prev_pos);
    print_report(what, r);
    if (r.above) std::printf("  elements above 1e-2: %zu (beyond one ulp of the dtype: %zu)\n", r.above, r.beyond);
    ok = ok && r.within_bound();
    worst = std::fmax(worst, r.max_abs);

    if (call == 0 && !qwen) { // the plain MHA operator gives the same bits as the prefill-optimised name
      auto out2 = Tensor::MakeGPUTensor(n_q, dtype);
      npu_flash_attn_layer(out2->data_ptr, q_emb->data_ptr, k_cache->data_ptr, v_cache->data_ptr, ctx.cur_size,
                           ctx.cur_pos, ctx.prev_pos, n_heads, head_dim, dtype, ctx.npu_stream);
      CHECK_CUDA(cudaStreamSynchronize(ctx.npu_stream));
      auto out2_cpu = out2->to(DEV_CPU);
      const bool same = std::memcmp(out2_cpu->data_ptr, out_cpu->data_ptr, SizeOfTensor(n_q, dtype)) == 0;
      std::printf("npu_flash_attn_layer == npu_flash_attn_opt_prefill_layer: %s\n", same ? "yes" : "no");
      ok = ok && same;
    }
  }
  // the caches hold the checker's rotated K and the raw V, bit for bit
  auto kc_cpu = k_cache->to(DEV_CPU), vc_cpu = v_cache->to(DEV_CPU);
  const bool cache_same = std::memcmp(kc_cpu->data_ptr, k_all.data(), k_all.size() * 2) == 0 &&
                          std::memcmp(vc_cpu->data_ptr, v_all.data(), v_all.size() * 2) == 0;
  std::printf("caches bit-identical to the checker: %s\n", cache_same ? "yes" : "no");
  ok = ok && cache_same;

  // a rejected call reaches the installed handler instead of returning silently
  npu_ops_compat_set_error_handler(counting_handler);
  npu_flash_attn_layer(nullptr, nullptr, nullptr, nullptr, 1, 1, 0, n_heads, 64 /* unsupported head_dim */, dtype,
                       ctx.npu_stream);
  npu_ops_compat_set_error_handler(nullptr);
  std::printf("error handler calls: %d\n", g_handler_calls);
  ok = ok && g_handler_calls == 1;

  std::printf("worst max_abs %.3e\n", worst);
  std::printf(ok ? "test success\n" : "test failed\n");
  CHECK_CUDA(cudaStreamDestroy(ctx.npu_stream));
  return ok ? 0 : 1;
}
