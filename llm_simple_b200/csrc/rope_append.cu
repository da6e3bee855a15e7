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
// pairing and in chunks (i, i+8) for the neox pairing.
template <typename T>
__global__ void __launch_bounds__(256) rope_append_kernel(RopeParams p) {
  const long total = static_cast<long>(p.batch) * p.m * p.slots * 8;
  for (long idx = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long>(gridDim.x) * blockDim.x) {
    const int i = static_cast<int>(idx & 7);
    long rest = idx >> 3;
    int slot = static_cast<int>(rest % p.slots);
    rest /= p.slots;
    const int t = static_cast<int>(rest % p.m);
    const int b = static_cast<int>(rest / p.m);

    int which = 0;
    if (slot >= p.s[0].heads) {
      slot -= p.s[0].heads;
      which = 1;
      if (slot >= p.s[1].heads) {
        slot -= p.s[1].heads;
        which = 2;
      }
    }
    const RopeStream &st = p.s[which];
    const int start = p.start_pos_dev ? p.start_pos_dev[b] : p.start_pos;
    const T *src = static_cast<const T *>(st.src) + b * st.src_seq + t * st.src_tok + slot * kHeadDim;
    T *dst;
    if (st.dst_at_pos && p.pg.table) {
      const int pos = start + t;
      const long page = p.pg.table[static_cast<long>(b) * p.pg.table_stride + (pos >> p.pg.page_shift)];
      dst = static_cast<T *>(st.dst) + page * p.pg.page_stride + (pos & ((1 << p.pg.page_shift) - 1)) * st.dst_tok +
            slot * st.dst_head;
    } else {
      dst = static_cast<T *>(st.dst) + b * st.dst_seq + (t + (st.dst_at_pos ? start : 0)) * st.dst_tok +
            slot * st.dst_head;
    }
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
    if (st.rotate) {
      const float4 *tab = reinterpret_cast<const float4 *>(p.freqs_cis + (static_cast<long>(start) + t) * kHeadDim + 16 * i);
      rope_chunk_pair<T>(u0, u1, tab, p.is_neox != 0);
    }
    *reinterpret_cast<uint4 *>(dst + c0 * 8) = u0;
    *reinterpret_cast<uint4 *>(dst + c1 * 8) = u1;
  }
}

cudaError_t launch_rope_append(const RopeParams &p, bool bf16, cudaStream_t stream) {
  const long total = static_cast<long>(p.batch) * p.m * p.slots * 8;
  if (total == 0) return cudaSuccess;
  long blocks = (total + 255) / 256;
  const long cap = 148L * 8 * 16; // grid-stride beyond this
  if (blocks > cap) blocks = cap;
  if (bf16)
    rope_append_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  else
    rope_append_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(p);
  return cudaGetLastError();
}

} // namespace b200attn
