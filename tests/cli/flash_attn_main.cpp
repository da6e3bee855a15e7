// Attention operator test program.  Same flags as the reference's
// tests/flash_attn_main.cpp:14-23 (--m --n --offset --head_num --head_dim),
// plus --dtype, --group_size, --kv_head_num, --seed, --mode strict|golden.
// Runs gpu_flash_attn_layer / gpu_flash_attn_gqa_layer on seeded N(0,1) inputs
// and compares with the CPU checker, as tests/flash_attn_test.cpp:67-236 compares
// the NPU operator with its Eigen golden.
#include "gpu_op_test_util.h"

int main(int argc, char **argv) {
  Flags f(argc, argv);
  if (f.has("help")) {
    std::printf("--m 2048 --n 2048 --offset 0 --head_num 32 --head_dim 128 [--dtype float16|bfloat16] "
                "[--group_size G --kv_head_num K] [--seed S] [--mode golden|strict]\n");
    return 1;
  }
  const int m = f.get_int("m", 2048), n = f.get_int("n", 2048), offset = f.get_int("offset", 0);
  const int head_dim = f.get_int("head_dim", 128);
  const int group = f.get_int("group_size", 1);
  const int kvh = f.get_int("kv_head_num", f.get_int("head_num", 32));
  const int H = group * kvh;
  const int dt = f.get("dtype", "float16") == "bfloat16" ? DT_BFLOAT16 : DT_FLOAT16;
  const int mode = f.get("mode", "golden") == "strict" ? ORACLE_MODE_STRICT : ORACLE_MODE_GOLDEN;
  const uint32_t seed = static_cast<uint32_t>(f.get_int("seed", 20250));
  std::printf("FlashAttentionOpTest::Run {m=%d,n=%d,offset=%d,heads=%d (group %d x kv %d),head_dim=%d,dtype=%s}\n", m,
              n, offset, H, group, kvh, head_dim, dt == DT_BFLOAT16 ? "bfloat16" : "float16");

  std::vector<uint16_t> q, k, v;
  make_random_bits(q, static_cast<size_t>(m) * H * head_dim, dt, seed);
  make_random_bits(k, static_cast<size_t>(n) * kvh * head_dim, dt, seed + 1);
  make_random_bits(v, static_cast<size_t>(n) * kvh * head_dim, dt, seed + 2);

  CHECK_CUDA(cudaSetDevice(0));
  cudaStream_t stream;
  CHECK_CUDA(cudaStreamCreate(&stream));
  const DataType dtype = static_cast<DataType>(dt);
  auto mk = [&](const std::vector<uint16_t> &h) {
    auto host = Tensor::MakeCPUTensor(h.size(), dtype);
    std::memcpy(host->data_ptr, h.data(), h.size() * 2);
    return host->to(DEV_GPU);
  };
  auto dq = mk(q), dk = mk(k), dv = mk(v);
  auto dout = Tensor::MakeGPUTensor(static_cast<size_t>(m) * H * head_dim, dtype);
  CHECK_CUDA(cudaMemset(dout->data_ptr, 0, static_cast<size_t>(m) * H * head_dim * 2));
  int rc = group == 1 ? gpu_flash_attn_layer(dout->data_ptr, dq->data_ptr, dk->data_ptr, dv->data_ptr, m, n, offset,
                                              kvh, head_dim, dt, stream)
                      : gpu_flash_attn_gqa_layer(dout->data_ptr, dq->data_ptr, dk->data_ptr, dv->data_ptr, m, n, offset,
                                                 group, kvh, head_dim, dt, stream);
  if (rc) {
    std::fprintf(stderr, "operator failed: %d %s\n", rc, gpu_ops_last_error_string());
    return 2;
  }
  CHECK_CUDA(cudaStreamSynchronize(stream));
  auto hout = dout->to(DEV_CPU);
  std::vector<float> out(static_cast<size_t>(m) * H * head_dim), golden(out.size());
  cpu_dt_to_f32(out.data(), static_cast<uint16_t *>(hout->data_ptr), out.size(), dt);

  std::vector<uint16_t> g16(out.size());
  rc = cpu_flash_attn_gqa_layer(g16.data(), golden.data(), q.data(), k.data(), v.data(), m, n, offset, group, kvh,
                                head_dim, dt, mode, cpu_oracle_max_threads());
  if (rc) return 2;
  if (mode == ORACLE_MODE_STRICT) cpu_dt_to_f32(golden.data(), g16.data(), golden.size(), dt);
  // compare against the golden rounded to the dtype, as the reference rounds its RoPE golden
  std::vector<uint16_t> gr(golden.size());
  std::vector<float> golden_rounded(golden.size());
  cpu_f32_to_dt(gr.data(), golden.data(), golden.size(), dt);
  cpu_dt_to_f32(golden_rounded.data(), gr.data(), gr.size(), dt);
  Report vs_f32 = compare(out, golden, dt), vs_rounded = compare(out, golden_rounded, dt);
  print_report("vs fp32 golden       ", vs_f32);
  print_report("vs golden in dtype   ", vs_rounded);
  // The bound: mean-abs 1e-3 and every element within max(1e-2, one ulp of the dtype at that
  // magnitude) of the golden rounded to the dtype.  How many elements needed the second term is printed.
  std::printf("elements above 1e-2: %zu of %zu (within one ulp of the dtype: %zu, beyond: %zu)\n", vs_rounded.above,
              out.size(), vs_rounded.above - vs_rounded.beyond, vs_rounded.beyond);
  std::printf("reference all_close(1e-3, 1e-3) on the fp32 golden: %s\n", vs_f32.all_close ? "yes" : "no");
  const bool ok = vs_rounded.within_bound() && vs_f32.mean_abs <= 2e-3;
  std::printf(ok ? "test success\n" : "test failed\n");
  CHECK_CUDA(cudaStreamDestroy(stream));
  return ok ? 0 : 1;
}
