// RoPE + KV-cache append in one elementwise pass.
//
// One launch rotates Q, rotates K straight into the cache and copies V into the
// cache (reference: npu_rope_layer / npu_rope_single_layer followed by two
// device-to-device copies, src/llama2_layer_npu.cpp:206-208, :325-338,
// :790-798, :830-843).  The same kernel serves the reference-shaped RoPE
// operators by pointing the destinations at plain tensors, the split of a fused
// q|k|v projection row (npu_split_qkv_layer, prebuild/npu_ops.h:27-30) by pointing
// the three sources into that row, and the projection bias of the Qwen2 layers
// (src/llama2_layer_npu.cpp:1020-1055) by an optional per-head bias row.
//
// HBM-bound: every input element is read once and every output element written
// once with 16-byte accesses; the fp32 table row (512 B per position) is shared
// by all heads of a token and stays in L1/L2.
#include "kernels.h"
#include "common.cuh"

namespace b200attn {

#ifndef ROPE_MIN_CTAS
#define ROPE_MIN_CTAS 5
#endif

// x + bias on one 16-byte chunk: fp32 sum of the two 16-bit values, rounded to the
// element type (the rounding point of a projection whose epilogue adds the bias).
template <typename T> __device__ __forceinline__ void add_bias_chunk(uint4 &u, const uint4 &bv) {
  uint32_t *w = reinterpret_cast<uint32_t *>(&u);
  const uint32_t *bw = reinterpret_cast<const uint32_t *>(&bv);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float2 x = Elem<T>::unpack(w[e]);
    const float2 y = Elem<T>::unpack(bw[e]);
    w[e] = Elem<T>::pack(__fadd_rn(x.x, y.x), __fadd_rn(x.y, y.y));
  }
}

// Eight threads work on one (token, head) row of 128 elements; thread i owns
// the pairs f = 8i .. 8i+7, which live in chunks (2i, 2i+1) for the interleaved
// pairing and in chunks (i, i+8) for the neox pairing.  A group of eight threads
// stays with one token and walks that token's head rows `lanes` apart (`lanes`
// groups share a token, 32 / lanes tokens share a CTA), so the thread's 64 bytes of
// the table row, the token's cache position and its page are fetched once per
// token instead of once per head row.
template <typename T>
__global__ void __launch_bounds__(256, ROPE_MIN_CTAS) rope_append_kernel(RopeParams p, int lanes_log2) {
  const int i = threadIdx.x & 7;
  const int grp = threadIdx.x >> 3;
  const int lanes = 1 << lanes_log2;
  const int first_slot = grp & (lanes - 1);
  const int toks_per_cta = 32 >> lanes_log2;
  const bool any_rotate = (p.s[0].heads && p.s[0].rotate) || (p.s[1].heads && p.s[1].rotate) ||
                          (p.s[2].heads && p.s[2].rotate);
  const int h0 = p.s[0].heads, h01 = h0 + p.s[1].heads;
  for (int b = blockIdx.y; b < p.batch; b += gridDim.y) {
    const int start = p.start_pos_dev ? p.start_pos_dev[b] : p.start_pos;
    for (int t = blockIdx.x * toks_per_cta + (grp >> lanes_log2); t < p.m; t += gridDim.x * toks_per_cta) {
      const int pos = start + t;
      float4 tab[4];
      if (any_rotate) {
        const float4 *row = reinterpret_cast<const float4 *>(p.freqs_cis + static_cast<long>(pos) * kHeadDim + 16 * i);
#pragma unroll
        for (int e = 0; e < 4; ++e) tab[e] = __ldg(row + e);
      }
      long paged_base = -1;
      if (p.pg.table) {
        const long page = p.pg.table[static_cast<long>(b) * p.pg.table_stride + (pos >> p.pg.page_shift)];
        paged_base = page * p.pg.page_stride;
      }
      for (int slot_all = first_slot + lanes * blockIdx.z; slot_all < p.slots; slot_all += lanes * gridDim.z) {
        const int which = (slot_all >= h0) + (slot_all >= h01);
        const int slot = slot_all - (which == 0 ? 0 : which == 1 ? h0 : h01);
        const RopeStream &st = p.s[which];
        const T *src = static_cast<const T *>(st.src) + b * st.src_seq + t * st.src_tok + slot * kHeadDim;
        T *dst;
        if (st.dst_at_pos && paged_base >= 0)
          dst = static_cast<T *>(st.dst) + paged_base + (pos & ((1 << p.pg.page_shift) - 1)) * st.dst_tok +
                slot * st.dst_head;
        else
          dst = static_cast<T *>(st.dst) + b * st.dst_seq + (st.dst_at_pos ? pos : t) * st.dst_tok + slot * st.dst_head;
        const int c0 = (st.rotate && !p.is_neox) ? 2 * i : i;
        const int c1 = (st.rotate && !p.is_neox) ? 2 * i + 1 : i + 8;
        // the tensors stream through once: keep them from evicting the table and bias rows in L1
        uint4 u0 = __ldcs(reinterpret_cast<const uint4 *>(src + c0 * 8));
        uint4 u1 = __ldcs(reinterpret_cast<const uint4 *>(src + c1 * 8));
        if (st.bias) {
          const T *bias = static_cast<const T *>(st.bias) + slot * kHeadDim;
          add_bias_chunk<T>(u0, __ldg(reinterpret_cast<const uint4 *>(bias + c0 * 8)));
          add_bias_chunk<T>(u1, __ldg(reinterpret_cast<const uint4 *>(bias + c1 * 8)));
        }
        if (st.rotate) rope_chunk_pair<T>(u0, u1, tab, p.is_neox != 0);
        *reinterpret_cast<uint4 *>(dst + c0 * 8) = u0;
        *reinterpret_cast<uint4 *>(dst + c1 * 8) = u1;
      }
    }
  }
}

cudaError_t launch_rope_append(const RopeParams &p, bool bf16, cudaStream_t stream) {
  if (static_cast<long>(p.batch) * p.m * p.slots == 0) return cudaSuccess;
  // Eight row groups per token amortise the table row over slots / 8 head rows; with few tokens
  // (a decode step, a short prompt) more groups share a token, and at 32 groups per token the
  // head rows are spread over CTAs as well, so that the launch still fills the GPU.
#ifndef ROPE_LANES0
#define ROPE_LANES0 3
#endif
  int lanes_log2 = ROPE_LANES0;
  while (lanes_log2 < 5 && static_cast<long>(p.batch) * ((p.m + (32 >> lanes_log2) - 1) / (32 >> lanes_log2)) < 148L * 8)
    ++lanes_log2;
  while (lanes_log2 > 0 && (1 << (lanes_log2 - 1)) >= p.slots) --lanes_log2;
  const int toks_per_cta = 32 >> lanes_log2;
  const unsigned gx = static_cast<unsigned>((p.m + toks_per_cta - 1) / toks_per_cta);
  const unsigned gy = static_cast<unsigned>(p.batch < 65535 ? p.batch : 65535);
  unsigned gz = 1;
  if (lanes_log2 == 5 && static_cast<long>(gx) * gy < 148L * 8) gz = static_cast<unsigned>((p.slots + 31) / 32);
  dim3 grid(gx, gy, gz);
  if (bf16)
    rope_append_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p, lanes_log2);
  else
    rope_append_kernel<__half><<<grid, 256, 0, stream>>>(p, lanes_log2);
  return cudaGetLastError();
}

} // namespace b200attn
