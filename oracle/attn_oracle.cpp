/*
 * attn_oracle.cpp -- CPU restatement of llm_simple's attention hot path.
 *
 * TEST INFRASTRUCTURE ONLY (checker and timed CPU baseline); the shipped
 * library never calls it.  What pins it to reference code: see attn_oracle.h.
 *
 * The reference's CPU layer (src/llama2_layer_cpu.cpp) materialises, per call,
 * the full [H, m, n] score tensor three times (fp32, fp16, softmax fp16) and
 * contracts head by head with Eigen on one thread.  This file keeps the same
 * algorithm and rounding points but walks one (head, row) at a time so that
 * memory stays bounded; the result of each element depends only on its own row,
 * so this changes nothing numerically.  Contractions here sum in vector lanes
 * (as Eigen's do); summation order is the only freedom taken.
 *
 * Two deliberate deviations from src/llama2_layer_cpu.cpp, both following the
 * reference's own test goldens instead:
 *   - the RoPE table row is (start_pos + s) as in
 *     tests/rope_single_layer_test.cpp:81-82; the CPU layer uses row s
 *     (src/llama2_layer_cpu.cpp:838-839), which is only right when prev_pos==0;
 *   - the neox pairing (f, f + D/2) is honoured as in
 *     tests/rope_single_layer_test.cpp:86-91; the CPU layer is interleaved-only.
 * Extensions the reference has no CPU code for: bf16 (same rounding points with
 * bf16), GQA (kv_head = q_head / group_size, the call-site convention of
 * src/llama2_layer_npu.cpp:866-869), and explicit strides.
 */
#include "attn_oracle.h"

#include <cmath>
#include <cstring>
#include <limits>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

inline float half_bits_to_f32(uint16_t h) {
  _Float16 x;
  std::memcpy(&x, &h, 2);
  return static_cast<float>(x);
}
inline uint16_t f32_to_half_bits(float f) {
  _Float16 x = static_cast<_Float16>(f); /* round-to-nearest-even, overflow -> inf */
  uint16_t h;
  std::memcpy(&h, &x, 2);
  return h;
}
inline float bf16_bits_to_f32(uint16_t b) {
  uint32_t u = static_cast<uint32_t>(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
/* round-to-nearest-even on the raw bits; inf/nan pass through */
inline uint16_t f32_to_bf16_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) {
    uint16_t hi = static_cast<uint16_t>(u >> 16);
    if (u & 0x007fffffu) hi |= 0x0040; /* keep NaN a NaN */
    return hi;
  }
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return static_cast<uint16_t>(u >> 16);
}

inline float to_f32(uint16_t x, int dt) {
  return dt == ORACLE_DT_BFLOAT16 ? bf16_bits_to_f32(x) : half_bits_to_f32(x);
}
inline uint16_t from_f32(float f, int dt) {
  return dt == ORACLE_DT_BFLOAT16 ? f32_to_bf16_bits(f) : f32_to_half_bits(f);
}
inline float round_dt(float f, int dt) { return to_f32(from_f32(f, dt), dt); }

bool dt_ok(int dt) { return dt == ORACLE_DT_FLOAT16 || dt == ORACLE_DT_BFLOAT16; }

/* tests/rope_single_layer_test.cpp:78-97 -- one tensor, fp32 rotate, round to dtype */
void rope_rows(uint16_t *out, const float *freqs_cis, const uint16_t *in, int start_pos,
               int cur_size, int n_heads, int hidden_dim, bool neox, int dt) {
  const int head_dim = hidden_dim / n_heads;
  const int freq_len = head_dim / 2;
  for (int s = 0; s < cur_size; ++s) {
    const float *row = freqs_cis + static_cast<size_t>(s + start_pos) * freq_len * 2;
    for (int h = 0; h < n_heads; ++h) {
      const size_t base = static_cast<size_t>(s) * hidden_dim + static_cast<size_t>(h) * head_dim;
      for (int f = 0; f < freq_len; ++f) {
        const float fc = row[2 * f];
        const float fd = row[2 * f + 1];
        const int ia = neox ? f : 2 * f;
        const int ib = neox ? freq_len + f : 2 * f + 1;
        const float a = to_f32(in[base + ia], dt);
        const float b = to_f32(in[base + ib], dt);
        /* (a + ib)(c + id) = (ac - bd) + i(ad + bc) */
        out[base + ia] = from_f32(a * fc - b * fd, dt);
        out[base + ib] = from_f32(a * fd + b * fc, dt);
      }
    }
  }
}

/*
 * One query row of one head.  Follows, in order:
 *   scores  src/llama2_layer_cpu.cpp:186-219  /  tests/flash_attn_test.cpp:124-145
 *   softmax src/llama2_layer_cpu.cpp:647-677  /  tests/flash_attn_test.cpp:156-170
 *   P.V     src/llama2_layer_cpu.cpp:272-296  /  tests/flash_attn_test.cpp:173-192
 * kf / vf are the head's K and V widened to fp32, [n][D] dense.
 * s_buf / p_buf: scratch of n floats.  o_acc: D floats (result, before rounding).
 */
void attn_row(float *o_acc, float *s_buf, float *p_buf, const float *qf, const float *kf,
              const float *vf, int row, int n, int offset, int D, float scale, int dt,
              int mode) {
  const float neg_inf = -std::numeric_limits<float>::infinity();
  for (int c = 0; c < n; ++c) {
    const float *kr = kf + static_cast<size_t>(c) * D;
    float acc = 0.f;
#pragma omp simd reduction(+ : acc)
    for (int d = 0; d < D; ++d) acc += qf[d] * kr[d];
    /* mask is added before the scale in both reference sources */
    const float mask = (c > row + offset) ? neg_inf : 0.f;
    float s = (acc + mask) * scale;
    if (mode == ORACLE_MODE_STRICT) s = round_dt(s, dt); /* llama2_layer_cpu.cpp:218-219 */
    s_buf[c] = s;
  }
  float mx = neg_inf;
  for (int c = 0; c < n; ++c) mx = s_buf[c] > mx ? s_buf[c] : mx;
  float sum = 0.f;
  for (int c = 0; c < n; ++c) {
    p_buf[c] = std::exp(s_buf[c] - mx);
    sum += p_buf[c];
  }
  for (int c = 0; c < n; ++c) {
    float p = p_buf[c] / sum;
    if (mode == ORACLE_MODE_STRICT) p = round_dt(p, dt); /* llama2_layer_cpu.cpp:675 */
    p_buf[c] = p;
  }
  for (int d = 0; d < D; ++d) o_acc[d] = 0.f;
  for (int c = 0; c < n; ++c) {
    const float p = p_buf[c];
    if (p == 0.f) continue; /* masked columns contribute exactly zero */
    const float *vr = vf + static_cast<size_t>(c) * D;
#pragma omp simd
    for (int d = 0; d < D; ++d) o_acc[d] += p * vr[d];
  }
}

} /* namespace */

extern "C" {

uint16_t cpu_fp32_to_bfloat16(uint32_t fp32_bits) {
  /* src/util.cpp:33-72: round the 24-bit significand to 8 bits, ties to even,
   * carry into the exponent, saturate the exponent field at 0xFF. */
  const uint32_t sign = (fp32_bits >> 31) & 1u;
  const uint32_t exponent = (fp32_bits >> 23) & 0xffu;
  const uint32_t sig24 = (fp32_bits & 0x007fffffu) | 0x00800000u;
  uint32_t hi = (sig24 >> 16) & 0xffu;
  const uint32_t lo = sig24 & 0xffffu;
  if (lo > 0x8000u || (lo == 0x8000u && (hi & 1u))) hi += 1;
  uint32_t e = exponent;
  if (hi > 0xffu) {
    e += 1;
    hi = 0x80u;
  }
  if (e > 0xffu) e = 0xffu;
  return static_cast<uint16_t>((sign << 15) | (e << 7) | (hi & 0x7fu));
}

void cpu_init_freq_cis(float *freq_cis, int head_dim, int max_seq_len, float theta, int dt) {
  /* src/model_base.cpp:27-57 */
  const int freq_len = head_dim / 2;
  std::vector<float> freq(freq_len);
  for (int i = 0; i < freq_len; ++i) {
    freq[i] = 1.0f / (std::pow(theta, static_cast<double>(i * 2) / static_cast<double>(head_dim)));
  }
  for (int p = 0; p < max_seq_len; ++p) {
    const float t = static_cast<float>(p);
    for (int j = 0; j < freq_len; ++j) {
      const float angle = t * freq[j]; /* fp32 product, as stored in freq_outer */
      const size_t i = static_cast<size_t>(p) * freq_len + j;
      freq_cis[2 * i] = std::cos(angle);
      freq_cis[2 * i + 1] = std::sin(angle);
    }
  }
  if (dt == ORACLE_DT_BFLOAT16) {
    /* src/model_base.cpp:59-66 */
    const size_t total = static_cast<size_t>(freq_len) * max_seq_len * 2;
    for (size_t i = 0; i < total; ++i) {
      uint32_t u;
      std::memcpy(&u, &freq_cis[i], 4);
      u = static_cast<uint32_t>(cpu_fp32_to_bfloat16(u)) << 16;
      std::memcpy(&freq_cis[i], &u, 4);
    }
  }
}

void cpu_init_freq_cis_test(float *freq_cis, int head_dim, int max_seq_len) {
  /* tests/npu_op_test_util.cpp:109-142 */
  const float theta = 10000.0f;
  const int freq_len = head_dim / 2;
  std::vector<float> freq(freq_len);
  for (int i = 0; i < freq_len; ++i) {
    freq[i] = 1.0f / (powf(theta, static_cast<float>(i * 2) / static_cast<float>(head_dim)));
  }
  for (int p = 0; p < max_seq_len; ++p) {
    const float t = static_cast<float>(p);
    for (int j = 0; j < freq_len; ++j) {
      const float angle = t * freq[j];
      const size_t i = static_cast<size_t>(p) * freq_len + j;
      freq_cis[2 * i] = std::cos(angle);
      freq_cis[2 * i + 1] = std::sin(angle);
    }
  }
}

/* the tensor rounding above on one raw fp32 pattern (for exhaustive comparison with util.cpp's routine) */
uint16_t cpu_f32_bits_to_bf16(uint32_t fp32_bits) {
  float f;
  std::memcpy(&f, &fp32_bits, 4);
  return f32_to_bf16_bits(f);
}

void cpu_f32_to_dt(uint16_t *dst, const float *src, size_t n, int dt) {
  for (size_t i = 0; i < n; ++i) dst[i] = from_f32(src[i], dt);
}
void cpu_dt_to_f32(float *dst, const uint16_t *src, size_t n, int dt) {
  for (size_t i = 0; i < n; ++i) dst[i] = to_f32(src[i], dt);
}

int cpu_rope_single_layer(uint16_t *out_x, const float *freqs_cis, const uint16_t *in_x,
                          int start_pos, int cur_size, int n_heads, int hidden_dim,
                          int is_neox_style, int dt) {
  if (!dt_ok(dt) || n_heads <= 0 || hidden_dim % n_heads || (hidden_dim / n_heads) % 2) return -1;
  rope_rows(out_x, freqs_cis, in_x, start_pos, cur_size, n_heads, hidden_dim, is_neox_style != 0, dt);
  return 0;
}

int cpu_rope_layer(uint16_t *out_q, uint16_t *out_k, const float *freqs_cis,
                   const uint16_t *in_q, const uint16_t *in_k, int start_pos, int cur_size,
                   int n_heads, int hidden_dim, int is_neox_style, int dt) {
  if (!dt_ok(dt) || n_heads <= 0 || hidden_dim % n_heads || (hidden_dim / n_heads) % 2) return -1;
  rope_rows(out_q, freqs_cis, in_q, start_pos, cur_size, n_heads, hidden_dim, is_neox_style != 0, dt);
  rope_rows(out_k, freqs_cis, in_k, start_pos, cur_size, n_heads, hidden_dim, is_neox_style != 0, dt);
  return 0;
}

int cpu_kv_append(uint16_t *k_cache, uint16_t *v_cache, const uint16_t *k_emb,
                  const uint16_t *v, int prev_pos, int cur_size, int kv_heads, int head_dim) {
  /* byte offset prev_pos * kv_heads * head_dim * 2, byte count cur_size * ... * 2 */
  const size_t row = static_cast<size_t>(kv_heads) * head_dim;
  std::memcpy(k_cache + prev_pos * row, k_emb, cur_size * row * sizeof(uint16_t));
  std::memcpy(v_cache + prev_pos * row, v, cur_size * row * sizeof(uint16_t));
  return 0;
}

int cpu_attn_strided(uint16_t *out16, float *out32, const uint16_t *q, const uint16_t *k,
                     const uint16_t *v, int m, int n, int offset, int group_size,
                     int kv_head_num, int head_dim, int dt, int mode, long q_row,
                     long k_pos_stride, long k_head_stride, long v_pos_stride,
                     long v_head_stride, long out_row, int threads) {
  if (!dt_ok(dt) || m <= 0 || n <= 0 || group_size <= 0 || kv_head_num <= 0 || head_dim <= 0) return -1;
  if (mode == ORACLE_MODE_STRICT && !out16) return -1;
  if (mode == ORACLE_MODE_GOLDEN && !out32) return -1;
  const int D = head_dim;
  const float scale = 1 / sqrtf(static_cast<float>(head_dim));
  const int n_heads = group_size * kv_head_num;
  int nthr = threads > 1 ? threads : 1;
  (void)nthr;
#pragma omp parallel num_threads(nthr)
  {
    std::vector<float> kf(static_cast<size_t>(n) * D), vf(static_cast<size_t>(n) * D);
    std::vector<float> s_buf(n), p_buf(n), qf(D), o(D);
#pragma omp for schedule(dynamic, 1)
    for (int kvh = 0; kvh < kv_head_num; ++kvh) {
      for (int c = 0; c < n; ++c) {
        const uint16_t *kr = k + c * k_pos_stride + kvh * k_head_stride;
        const uint16_t *vr = v + c * v_pos_stride + kvh * v_head_stride;
        for (int d = 0; d < D; ++d) {
          kf[static_cast<size_t>(c) * D + d] = to_f32(kr[d], dt);
          vf[static_cast<size_t>(c) * D + d] = to_f32(vr[d], dt);
        }
      }
      for (int g = 0; g < group_size; ++g) {
        const int h = kvh * group_size + g;
        for (int r = 0; r < m; ++r) {
          const uint16_t *qr = q + r * q_row + static_cast<long>(h) * D;
          for (int d = 0; d < D; ++d) qf[d] = to_f32(qr[d], dt);
          attn_row(o.data(), s_buf.data(), p_buf.data(), qf.data(), kf.data(), vf.data(), r, n,
                   offset, D, scale, dt, mode);
          /* [H][m][D] -> [m][H*D] (llama2_layer_cpu.cpp:294-296, flash_attn_test.cpp:190-192) */
          if (mode == ORACLE_MODE_STRICT) {
            uint16_t *orow = out16 + r * out_row + static_cast<long>(h) * D;
            for (int d = 0; d < D; ++d) orow[d] = from_f32(o[d], dt);
          } else {
            float *orow = out32 + r * out_row + static_cast<long>(h) * D;
            for (int d = 0; d < D; ++d) orow[d] = o[d];
          }
        }
      }
    }
  }
  (void)n_heads;
  return 0;
}

int cpu_flash_attn_gqa_layer(uint16_t *out16, float *out32, const uint16_t *q,
                             const uint16_t *k, const uint16_t *v, int m, int n, int offset,
                             int group_size, int kv_head_num, int head_dim, int dt, int mode,
                             int threads) {
  const long kv_row = static_cast<long>(kv_head_num) * head_dim;
  const long q_row = static_cast<long>(kv_head_num) * group_size * head_dim;
  return cpu_attn_strided(out16, out32, q, k, v, m, n, offset, group_size, kv_head_num, head_dim,
                          dt, mode, q_row, kv_row, head_dim, kv_row, head_dim, q_row, threads);
}

int cpu_flash_attn_layer(uint16_t *out16, float *out32, const uint16_t *q, const uint16_t *k,
                         const uint16_t *v, int m, int n, int offset, int head_num,
                         int head_dim, int dt, int mode, int threads) {
  return cpu_flash_attn_gqa_layer(out16, out32, q, k, v, m, n, offset, 1, head_num, head_dim, dt,
                                  mode, threads);
}

int cpu_scores_one_head(float *s_out, float *p_out, const uint16_t *q, const uint16_t *k,
                        int m, int n, int offset, int head_dim, int dt, int mode, long q_row,
                        long k_pos_stride) {
  if (!dt_ok(dt)) return -1;
  const int D = head_dim;
  const float scale = 1 / sqrtf(static_cast<float>(head_dim));
  std::vector<float> kf(static_cast<size_t>(n) * D), vf(static_cast<size_t>(n) * D, 0.f), qf(D), o(D);
  for (int c = 0; c < n; ++c)
    for (int d = 0; d < D; ++d) kf[static_cast<size_t>(c) * D + d] = to_f32(k[c * k_pos_stride + d], dt);
  for (int r = 0; r < m; ++r) {
    for (int d = 0; d < D; ++d) qf[d] = to_f32(q[r * q_row + d], dt);
    /* attn_row leaves the scaled scores in s_buf and the probabilities in p_buf */
    attn_row(o.data(), s_out + static_cast<size_t>(r) * n, p_out + static_cast<size_t>(r) * n,
             qf.data(), kf.data(), vf.data(), r, n, offset, D, scale, dt, mode);
  }
  return 0;
}

int cpu_all_close(const float *out, const float *golden, size_t n, float abs_err, float rel_err) {
  /* tests/npu_op_test_util.cpp:33-48: fails only when BOTH bounds are exceeded */
  for (size_t i = 0; i < n; ++i) {
    const float a = out[i], b = golden[i];
    const float abs_diff = std::fabs(a - b);
    const float max_abs = std::fabs(a) > std::fabs(b) ? std::fabs(a) : std::fabs(b);
    if (abs_diff > abs_err && (abs_diff / max_abs) > rel_err) return 0;
    if (std::isnan(a) != std::isnan(b)) return 0;
  }
  return 1;
}

int cpu_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

} /* extern "C" */
