// Source-compatible overloads of the reference's attention-path operators.
//
// Include this where the reference includes "npu_ops.h" and the attention
// sections of its transformer layers (src/llama2_layer_npu.cpp:283-374 Llama-2,
// :780-869 Qwen2) compile unchanged against CUDA memory: same function names,
// same argument order, `DataType` for the element type and the stream taken by
// reference, exactly as prebuild/npu_ops.h declares them:
//
//   npu_flash_attn_layer              prebuild/npu_ops.h:6-8
//   npu_flash_attn_gqa_layer          prebuild/npu_ops.h:10-13
//   npu_flash_attn_opt_prefill_layer  prebuild/npu_ops.h:15-18
//   npu_split_qkv_layer               prebuild/npu_ops.h:27-30
//   npu_rope_layer                    prebuild/npu_ops.h:39-42
//   npu_rope_single_layer             prebuild/npu_ops.h:44-47
//
// The reference's operators return void; the C functions of gpu_ops.h return a
// status.  A non-zero status goes to the handler installed with
// npu_ops_compat_set_error_handler(); the default one prints the library's
// message to stderr and aborts: a rejected call leaves its output unwritten, and
// the reference's call sites have no way to learn that from a void function.
//
// Define NPU_OPS_COMPAT_NO_ACL_TYPES before including when the translation unit
// already has its own `aclrtStream` (e.g. a build that keeps the Ascend headers).
#pragma once

#include <cstdio>
#include <cstdlib>

#include <cuda_runtime_api.h>

#include "defs.hpp"
#include "gpu_ops.h"

#ifndef NPU_OPS_COMPAT_NO_ACL_TYPES
using aclrtStream = cudaStream_t; // the reference's stream handle (acl/acl.h), here a CUDA stream
#endif

using npu_ops_compat_error_handler = void (*)(const char *op, int status, const char *message);

inline void npu_ops_compat_default_handler(const char *op, int status, const char *message) {
  std::fprintf(stderr, "%s failed: status %d: %s\n", op, status, message);
  std::abort();
}

inline npu_ops_compat_error_handler &npu_ops_compat_handler_slot() {
  static npu_ops_compat_error_handler h = npu_ops_compat_default_handler;
  return h;
}

// Returns the previous handler.  nullptr restores the default.
inline npu_ops_compat_error_handler npu_ops_compat_set_error_handler(npu_ops_compat_error_handler h) {
  npu_ops_compat_error_handler old = npu_ops_compat_handler_slot();
  npu_ops_compat_handler_slot() = h ? h : npu_ops_compat_default_handler;
  return old;
}

inline void npu_ops_compat_check(const char *op, int status) {
  if (status != 0) npu_ops_compat_handler_slot()(op, status, gpu_ops_last_error_string());
}

inline void npu_flash_attn_layer(void *output_dev, void *q_dev, void *k_dev, void *v_dev, int m, int n, int offset,
                                 int head_num, int head_dim, DataType dt, aclrtStream &stream) {
  npu_ops_compat_check("npu_flash_attn_layer", gpu_flash_attn_layer(output_dev, q_dev, k_dev, v_dev, m, n, offset,
                                                                    head_num, head_dim, static_cast<int>(dt), stream));
}

inline void npu_flash_attn_gqa_layer(void *output_dev, void *q_dev, void *k_dev, void *v_dev, int m, int n,
                                     int offset, int group_size, int kv_head_num, int head_dim, DataType dt,
                                     aclrtStream &stream) {
  npu_ops_compat_check("npu_flash_attn_gqa_layer",
                       gpu_flash_attn_gqa_layer(output_dev, q_dev, k_dev, v_dev, m, n, offset, group_size, kv_head_num,
                                                head_dim, static_cast<int>(dt), stream));
}

inline void npu_flash_attn_opt_prefill_layer(void *output_dev, void *q_dev, void *k_dev, void *v_dev, int m, int n,
                                             int offset, int head_num, int head_dim, DataType dt,
                                             aclrtStream &stream) {
  npu_ops_compat_check("npu_flash_attn_opt_prefill_layer",
                       gpu_flash_attn_opt_prefill_layer(output_dev, q_dev, k_dev, v_dev, m, n, offset, head_num,
                                                        head_dim, static_cast<int>(dt), stream));
}

inline void npu_split_qkv_layer(void *output_q_dev, void *output_k_dev, void *output_v_dev, void *input_qkv,
                                int batch, int q_dim, int k_dim, int v_dim, DataType dt, aclrtStream &stream) {
  npu_ops_compat_check("npu_split_qkv_layer",
                       gpu_split_qkv_layer(output_q_dev, output_k_dev, output_v_dev, input_qkv, batch, q_dim, k_dim,
                                           v_dim, static_cast<int>(dt), stream));
}

inline void npu_rope_layer(void *output_q_dev, void *output_k_dev, void *freqs_cis_dev, void *input_q_dev,
                           void *input_k_dev, int start_pos, int cur_size, int n_heads, int hidden_dim,
                           bool is_neox_style, DataType dt, aclrtStream &stream) {
  npu_ops_compat_check("npu_rope_layer",
                       gpu_rope_layer(output_q_dev, output_k_dev, freqs_cis_dev, input_q_dev, input_k_dev, start_pos,
                                      cur_size, n_heads, hidden_dim, is_neox_style ? 1 : 0, static_cast<int>(dt),
                                      stream));
}

inline void npu_rope_single_layer(void *output_x_dev, void *freqs_cis_dev, void *input_x_dev, int start_pos,
                                  int cur_size, int n_heads, int hidden_dim, bool is_neox_style, DataType dt,
                                  aclrtStream &stream) {
  npu_ops_compat_check("npu_rope_single_layer",
                       gpu_rope_single_layer(output_x_dev, freqs_cis_dev, input_x_dev, start_pos, cur_size, n_heads,
                                             hidden_dim, is_neox_style ? 1 : 0, static_cast<int>(dt), stream));
}
