// RoPE operator test program.  Same flags as the reference's
// tests/rope_single_layer_main.cpp:37-46 (--max_seq_length --head_dim --head_num
// --seq_len --is_neox --offset --dtype).  Unlike the reference's test class,
// which never stores its is_neox argument, the flag is honoured here.
// Golden: tests/rope_single_layer_test.cpp:78-97 via the CPU checker; the GPU
// result must be bit-identical.
#include "gpu_op_test_util.h"

int main(int argc, char **argv) {
  Flags f(argc, argv);
  if (f.has("help") || !f.has("dtype")) {
    std::printf("--dtype float16|bfloat16 [--max_seq_length 4096 --head_dim 128 --head_num 32 --seq_len 32 "
                "--is_neox true --offset 0 --seed S]\n");
    return 1;
  }
  const int max_seq = f.get_int("max_seq_length", 4096), head_dim = f.get_int("head_dim", 128);
  const int heads = f.get_int("head_num", 32), seq_len = f.get_int("seq_len", 32), offset = f.get_int("offset", 0);
  const bool neox = f.get_bool("is_neox", true);
  const int dt = f.get("dtype", "float16") == "bfloat16" ? DT_BFLOAT16 : DT_FLOAT16;
  std::printf("RoPESingleOpTest max_seq_len %d head_num %d head_dim %d offset %d seq_len %d is_neox %d\n", max_seq,
              heads, head_dim, offset, seq_len, int(neox));
  if (offset + seq_len > max_seq) {
    std::fprintf(stderr, "offset + seq_len exceeds max_seq_length\n");
    return 2;
  }
  std::vector<float> table(static_cast<size_t>(max_seq) * head_dim);
  cpu_init_freq_cis_test(table.data(), head_dim, max_seq); // the table of the reference's tests (theta 10000, powf)
  std::vector<uint16_t> x;
  make_random_bits(x, static_cast<size_t>(seq_len) * heads * head_dim, dt, static_cast<uint32_t>(f.get_int("seed", 7)));
  std::vector<uint16_t> golden(x.size());
  cpu_rope_single_layer(golden.data(), table.data(), x.data(), offset, seq_len, heads, heads * head_dim, neox, dt);

  CHECK_CUDA(cudaSetDevice(0));
  cudaStream_t stream;
  CHECK_CUDA(cudaStreamCreate(&stream));
  const DataType dtype = static_cast<DataType>(dt);
  auto hx = Tensor::MakeCPUTensor(x.size(), dtype);
  std::memcpy(hx->data_ptr, x.data(), x.size() * 2);
  auto ht = Tensor::MakeCPUTensor(table.size(), DT_FLOAT32);
  std::memcpy(ht->data_ptr, table.data(), table.size() * 4);
  auto dx = hx->to(DEV_GPU), dtab = ht->to(DEV_GPU);
  auto dy = Tensor::MakeGPUTensor(x.size(), dtype);
  int rc = gpu_rope_single_layer(dy->data_ptr, dtab->data_ptr, dx->data_ptr, offset, seq_len, heads, heads * head_dim,
                                 neox, dt, stream);
  if (rc) {
    std::fprintf(stderr, "operator failed: %d %s\n", rc, gpu_ops_last_error_string());
    return 2;
  }
  CHECK_CUDA(cudaStreamSynchronize(stream));
  auto hy = dy->to(DEV_CPU);
  const bool exact = std::memcmp(hy->data_ptr, golden.data(), golden.size() * 2) == 0;
  std::vector<float> a(x.size()), b(x.size());
  cpu_dt_to_f32(a.data(), static_cast<uint16_t *>(hy->data_ptr), a.size(), dt);
  cpu_dt_to_f32(b.data(), golden.data(), b.size(), dt);
  print_report("rope", compare(a, b));
  std::printf("bit-identical: %s\n", exact ? "yes" : "no");
  std::printf(exact ? "test success\n" : "test failed\n");
  CHECK_CUDA(cudaStreamDestroy(stream));
  return exact ? 0 : 1;
}
