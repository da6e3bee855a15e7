// C entry points over the pieces of the reference that oracle/build_ref.py compiles from the
// reference tree: the functions of src/util.cpp and tests/npu_op_test_util.cpp as they are, and
// three code blocks that build_ref.py extracts into oracle/_ref/*.inc at build time, placed here
// inside the declarations they need.  Test infrastructure only.
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <limits>

#include <spdlog/spdlog.h>

#include "defs.hpp" // the reference's prebuild/defs.hpp: DataType, DeviceType

// ---- compiled unmodified from the reference tree (src/util.cpp, tests/npu_op_test_util.cpp)
uint16_t fp32_to_bfloat16(uint32_t fp32_bits);
bool all_close(float *output_buffer, float *golden_buffer, size_t size, float abs_err, float relative_err);
void InitFreqCIS(float *freq_cis, int head_dim, int max_seq_len);

// ---- ModelBase::InitFreqCIS (src/model_base.cpp:27-83): the members the function touches, and
//      the Ascend calls of its device branch (not taken: device_type is DEV_CPU here)
#define CHECK_ACL(x) ((void)0)
#define ACL_MEM_MALLOC_HUGE_FIRST 0
#define ACL_MEMCPY_HOST_TO_DEVICE 0
struct ModelConfig {
  int max_seq_len;
  DeviceType device_type;
};
class ModelBase {
public:
  bool InitFreqCIS(const float theta, const DataType dt);
  int hidden_dim, n_heads;
  ModelConfig config;
  float *freq_cis;
};
#include "init_freq_cis.inc"

extern "C" {

uint16_t ref_fp32_to_bfloat16(uint32_t bits) { return fp32_to_bfloat16(bits); }

// Number of 32-bit patterns in [lo, hi) on which `other` differs from the reference's routine;
// *first receives the first such pattern.
uint64_t ref_bf16_sweep(uint16_t (*other)(uint32_t), uint64_t lo, uint64_t hi, uint32_t *first) {
  uint64_t bad = 0, first_bad = UINT64_MAX;
#pragma omp parallel for reduction(+ : bad) reduction(min : first_bad) schedule(static)
  for (uint64_t u = lo; u < hi; ++u) {
    const uint32_t x = static_cast<uint32_t>(u);
    if (fp32_to_bfloat16(x) != other(x)) {
      ++bad;
      if (u < first_bad) first_bad = u;
    }
  }
  if (first && bad) *first = static_cast<uint32_t>(first_bad);
  return bad;
}

int ref_all_close(const float *out, const float *golden, size_t n, float abs_err, float rel_err) {
  // the reference's routine prints the first mismatch to stdout; its verdict is what is wanted
  return all_close(const_cast<float *>(out), const_cast<float *>(golden), n, abs_err, rel_err) ? 1 : 0;
}

void ref_test_init_freq_cis(float *freq_cis, int head_dim, int max_seq_len) { InitFreqCIS(freq_cis, head_dim, max_seq_len); }

// out: [max_seq_len][head_dim/2][2]
int ref_model_init_freq_cis(float *out, int head_dim, int max_seq_len, float theta, int dt) {
  ModelBase m;
  m.n_heads = 1;
  m.hidden_dim = head_dim;
  m.config.max_seq_len = max_seq_len;
  m.config.device_type = DEV_CPU;
  m.freq_cis = nullptr;
  if (!m.InitFreqCIS(theta, static_cast<DataType>(dt))) return -1;
  std::memcpy(out, m.freq_cis, sizeof(float) * static_cast<size_t>(max_seq_len) * head_dim);
  delete[] m.freq_cis;
  return 0;
}

// The golden loop of RoPESingleOpTest::Run (tests/rope_single_layer_test.cpp:78-95) over fp32
// arrays; the test rounds input and golden to the 16-bit type around it (:72-73, :97), which the
// caller does.
void ref_rope_golden(float *golden_fp32, const float *host_input, const float *host_freq_cis, int offset, int seq_len,
                     int head_num, int head_dim, int is_neox_flag) {
  const bool is_neox = is_neox_flag != 0;
  int freq_len = head_dim / 2;
  int hidden_dim = head_num * head_dim;
#include "rope_golden_loop.inc"
}

// The mask loop of FlashAttentionOpTest::Run (tests/flash_attn_test.cpp:124-132).
void ref_causal_mask(float *host_mask, int m, int n, int offset) {
#include "mask_loop.inc"
}

} // extern "C"
