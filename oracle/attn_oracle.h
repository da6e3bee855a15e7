/*
 * attn_oracle.h -- CPU restatement of llm_simple's attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing shipped by the library links, loads or
 * calls this; it exists so the CUDA kernels can be checked ("call both,
 * compare") and so a CPU baseline can be timed beside them.
 *
 * HOW IT IS PINNED.  The reference stores no golden vectors (its tests draw
 * unseeded random inputs and compute an Eigen golden at run time) and its
 * device library is a closed AArch64/Ascend binary, so the pins are outputs of
 * reference code compiled where it lies (oracle/build_ref.py ->
 * oracle/_ref/libref_pins.so; fixtures tests/golden/ref_pins.npz made by
 * tests/golden/make_ref_pins.py, checked by tests/test_ref_pins.py):
 *   - fp32_to_bfloat16 (src/util.cpp:33-72): identical on all 2^32 patterns;
 *   - the RoPE table of ModelBase::InitFreqCIS (src/model_base.cpp:27-83) and
 *     of the tests' twin (tests/npu_op_test_util.cpp:109-142): bit-identical;
 *   - the RoPE golden loop (tests/rope_single_layer_test.cpp:78-95), the mask
 *     loop (tests/flash_attn_test.cpp:124-132), all_close
 *     (tests/npu_op_test_util.cpp:33-48): bit-identical / same verdicts.
 * NOT pinned by reference code: the two contractions and the softmax of the
 * attention golden (Eigen tensor expressions; Eigen is not installed, so they
 * cannot be compiled here).  Those are pinned by analytic known-answer cases,
 * by an independently written numpy restatement and by PyTorch's CPU
 * scaled_dot_product_attention in fp32 as a second opinion (<= 2e-5).  GQA head
 * mapping, bf16 attention and batch > 1 have no reference test at all.
 *
 * Reference lines each function follows are cited at its definition.
 *
 * dtype codes are the reference's DataType values (prebuild/defs.hpp:8-18):
 * 4 = fp16, 5 = bf16.  All 16-bit tensors are passed as raw uint16_t storage.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORACLE_DT_FLOAT16 = 4, ORACLE_DT_BFLOAT16 = 5 };

/* mode of cpu_attn_*: where intermediate roundings happen */
enum {
  ORACLE_MODE_STRICT = 0, /* src/llama2_layer_cpu.cpp: S, P and O rounded to the 16-bit dtype */
  ORACLE_MODE_GOLDEN = 1  /* tests/flash_attn_test.cpp: fp32 throughout, fp32 output */
};

/* src/model_base.cpp:27-83 (double pow; bf16 variant re-rounded) */
void cpu_init_freq_cis(float *freq_cis, int head_dim, int max_seq_len, float theta, int dt);
/* tests/npu_op_test_util.cpp:109-142 (powf, theta 10000) */
void cpu_init_freq_cis_test(float *freq_cis, int head_dim, int max_seq_len);

/* src/util.cpp:33-72 */
uint16_t cpu_fp32_to_bfloat16(uint32_t fp32_bits);

/* round-to-nearest-even of one raw fp32 pattern to bf16 as the element conversions below do it
 * (NaN stays NaN, which src/util.cpp's routine does not guarantee) */
uint16_t cpu_f32_bits_to_bf16(uint32_t fp32_bits);

/* element conversions used by the tests to prepare/inspect 16-bit buffers */
void cpu_f32_to_dt(uint16_t *dst, const float *src, size_t n, int dt);
void cpu_dt_to_f32(float *dst, const uint16_t *src, size_t n, int dt);

/* tests/rope_single_layer_test.cpp:78-97 */
int cpu_rope_single_layer(uint16_t *out_x, const float *freqs_cis, const uint16_t *in_x,
                          int start_pos, int cur_size, int n_heads, int hidden_dim,
                          int is_neox_style, int dt);
/* tests/npu_operator_test.cpp:1005-1026, src/llama2_layer_cpu.cpp:835-859 */
int cpu_rope_layer(uint16_t *out_q, uint16_t *out_k, const float *freqs_cis,
                   const uint16_t *in_q, const uint16_t *in_k, int start_pos, int cur_size,
                   int n_heads, int hidden_dim, int is_neox_style, int dt);

/* src/llama2_layer_cpu.cpp:141-161, src/llama2_layer_npu.cpp:325-338: token-major append */
int cpu_kv_append(uint16_t *k_cache, uint16_t *v_cache, const uint16_t *k_emb,
                  const uint16_t *v, int prev_pos, int cur_size, int kv_heads, int head_dim);

/*
 * Attention with explicit element strides (covers the reference's token-major
 * cache and the head-major cache).  q: [m][kvH*G][D] with row stride q_row;
 * k/v element (pos, kv_head, d) at pos*pos_stride + kv_head*head_stride + d.
 * out row stride out_row (elements).  STRICT writes out16, GOLDEN writes out32
 * (the other pointer may be NULL).  threads <= 1 runs single-threaded.
 */
int cpu_attn_strided(uint16_t *out16, float *out32, const uint16_t *q, const uint16_t *k,
                     const uint16_t *v, int m, int n, int offset, int group_size,
                     int kv_head_num, int head_dim, int dt, int mode, long q_row,
                     long k_pos_stride, long k_head_stride, long v_pos_stride,
                     long v_head_stride, long out_row, int threads);

/* reference-shaped wrappers (prebuild/npu_ops.h:6-18), token-major k/v */
int cpu_flash_attn_layer(uint16_t *out16, float *out32, const uint16_t *q, const uint16_t *k,
                         const uint16_t *v, int m, int n, int offset, int head_num,
                         int head_dim, int dt, int mode, int threads);
int cpu_flash_attn_gqa_layer(uint16_t *out16, float *out32, const uint16_t *q,
                             const uint16_t *k, const uint16_t *v, int m, int n, int offset,
                             int group_size, int kv_head_num, int head_dim, int dt, int mode,
                             int threads);

/* intermediates, for the known-answer checks of the unfused triple
 * (tests/npu_operator_test.cpp:553-715 S, :93-189 P): one head, fp32. */
int cpu_scores_one_head(float *s_out, float *p_out, const uint16_t *q, const uint16_t *k,
                        int m, int n, int offset, int head_dim, int dt, int mode, long q_row,
                        long k_pos_stride);

/* the reference tests' comparison (tests/npu_op_test_util.cpp:33-48); returns 1 if close */
int cpu_all_close(const float *out, const float *golden, size_t n, float abs_err, float rel_err);

int cpu_oracle_max_threads(void);

#ifdef __cplusplus
}
#endif
