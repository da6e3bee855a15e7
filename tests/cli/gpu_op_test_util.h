// Shared pieces of the operator test programs: flag parsing, seeded inputs, the
// reference's comparison rule, and the report.  Counterpart of the reference's
// tests/npu_op_test_util.{h,cpp}; the CPU checker (oracle/attn_oracle.h) plays
// the role of its Eigen golden.
#pragma once

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <random>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "attn_oracle.h"
#include "defs.hpp"
#include "device.hpp"
#include "gpu_ops.h"

#define CHECK_CUDA(x)                                                                                      \
  do {                                                                                                     \
    cudaError_t err__ = (x);                                                                               \
    if (err__ != cudaSuccess) {                                                                            \
      std::fprintf(stderr, "%s:%d cudaError: %s\n", __FILE__, __LINE__, cudaGetErrorString(err__));        \
      std::exit(2);                                                                                        \
    }                                                                                                      \
  } while (0)

// --name value / --name=value flags with defaults
class Flags {
public:
  Flags(int argc, char **argv) {
    for (int i = 1; i < argc; ++i) {
      std::string a = argv[i];
      if (a.rfind("--", 0) != 0) continue;
      a = a.substr(2);
      auto eq = a.find('=');
      if (eq != std::string::npos)
        kv_[a.substr(0, eq)] = a.substr(eq + 1);
      else if (i + 1 < argc && std::string(argv[i + 1]).rfind("--", 0) != 0)
        kv_[a] = argv[++i];
      else
        kv_[a] = "true";
    }
  }
  bool has(const std::string &k) const { return kv_.count(k) != 0; }
  int get_int(const std::string &k, int dflt) const { return has(k) ? std::atoi(kv_.at(k).c_str()) : dflt; }
  std::string get(const std::string &k, const std::string &dflt) const { return has(k) ? kv_.at(k) : dflt; }
  bool get_bool(const std::string &k, bool dflt) const {
    if (!has(k)) return dflt;
    const std::string &v = kv_.at(k);
    return v == "1" || v == "true" || v == "True";
  }

private:
  std::map<std::string, std::string> kv_;
};

// seeded N(0,1), rounded to the 16-bit dtype (the reference draws unseeded uniform(-1,1),
// tests/npu_op_test_util.cpp:3-11)
inline void make_random_bits(std::vector<uint16_t> &dst, size_t n, int dt, uint32_t seed) {
  std::mt19937 gen(seed);
  std::normal_distribution<float> dis(0.f, 1.f);
  std::vector<float> f(n);
  for (size_t i = 0; i < n; ++i) f[i] = dis(gen);
  dst.resize(n);
  cpu_f32_to_dt(dst.data(), f.data(), n, dt);
}

struct Report {
  double max_abs = 0, mean_abs = 0;
  size_t worst = 0;
  bool all_close = false; // the reference tests' verdict (1e-3 abs or 1e-3 rel)
  bool within_bar = false; // max-abs <= 1e-2 and mean-abs <= 1e-3
  // elements further than 1e-2 from the golden, and how many of those are also further than one
  // ulp of the 16-bit type at the golden's magnitude (bf16 values of magnitude >= 2 lie 1.6e-2
  // apart, so a correctly rounded result of a differently ordered sum can land on the neighbour)
  size_t above = 0, beyond = 0;
  bool within_bound() const { return mean_abs <= 1e-3 && beyond == 0; }
};

inline Report compare(const std::vector<float> &out, const std::vector<float> &golden, int dt = DT_FLOAT16) {
  Report r;
  double sum = 0;
  const int mant = dt == DT_BFLOAT16 ? 7 : 10;
  for (size_t i = 0; i < out.size(); ++i) {
    const double d = std::fabs(static_cast<double>(out[i]) - golden[i]);
    sum += d;
    if (d > 1e-2) {
      ++r.above;
      const double mag = std::fmax(std::fabs(static_cast<double>(golden[i])), std::ldexp(1.0, -14));
      if (!(d <= std::ldexp(1.0, static_cast<int>(std::floor(std::log2(mag))) - mant))) ++r.beyond;
    }
    if (d > r.max_abs) {
      r.max_abs = d;
      r.worst = i;
    }
  }
  r.mean_abs = out.empty() ? 0 : sum / out.size();
  r.all_close = cpu_all_close(out.data(), golden.data(), out.size(), 1e-3f, 1e-3f) != 0;
  r.within_bar = r.max_abs <= 1e-2 && r.mean_abs <= 1e-3;
  return r;
}

inline void print_report(const char *what, const Report &r) {
  std::printf("%s: max_abs %.3e mean_abs %.3e worst_index %zu all_close(1e-3) %s within(1e-2,1e-3) %s\n", what,
              r.max_abs, r.mean_abs, r.worst, r.all_close ? "yes" : "no", r.within_bar ? "yes" : "no");
}
