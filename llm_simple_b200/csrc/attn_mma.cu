// Attention kernels on the warp-level tensor path (mma.sync m16n8k16):
//
//   attn_decode_kernel   grouped-query decode / small-m attention over the KV
//                        cache, split along the cache, with the new token's
//                        RoPE + append fused in (HBM-bound: every K/V byte is
//                        fetched once with 16-byte cp.async into a 3-stage ring)
//   attn_merge_kernel    log-sum-exp merge of split (or cross-device) partials
//   attn_prefill_mma_kernel  causal attention for any (m, n, offset); the
//                        general path and the cross-check of the tcgen05 kernel
//
// Reference semantics: tests/flash_attn_test.cpp:106-192 (mask col > row+offset,
// scale 1/sqrt(D), row softmax, O = P.V, output [m][H*D]); GQA head mapping
// q_head / group (src/llama2_layer_npu.cpp:866-869).
#include "kernels.h"
#include "common.cuh"

#include <limits.h>

#include <mutex>
#include <utility>
#include <vector>

namespace b200attn {

namespace {

constexpr int kDecodeThreads = 128;
constexpr int kDecodeStages = 3;
constexpr int kTileN = 64;                          // key positions per pipeline stage
constexpr int kTileBytes = kTileN * kRowBytes;      // 16 KB
constexpr int kRedStride = 136;                     // floats per row of the cross-warp reduction buffer
constexpr int kDecodeQBytes = 16 * kRowBytes;       // 4 KB
constexpr int kDecodeSmem = kDecodeQBytes + 2 * kRowBytes + kDecodeStages * 2 * kTileBytes;

} // namespace

// grid: (max_splits, n_kv_heads, batch); block: 128 threads = 4 warps.
// Each warp takes 16 of the 64 key positions of a stage against all 16
// (padded) query rows of the KV head, and keeps its own online-softmax state;
// the four states are merged through shared memory at the end.
template <typename T>
__global__ void __launch_bounds__(kDecodeThreads, 2) attn_decode_kernel(DecodeParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char *q_s = smem;
  T *knew_s = reinterpret_cast<T *>(smem + kDecodeQBytes);
  T *vnew_s = knew_s + kHeadDim;
  unsigned char *stage_s = smem + kDecodeQBytes + 2 * kRowBytes;

  // Launched with programmatic stream serialisation: this grid may be scheduled while
  // the previous kernel of the stream is still draining.  Let the next one in as early
  // as possible, and touch no memory before the previous grid has completed and flushed.
  // With early_kv the caller guarantees that the length array and the cached rows below
  // kv_len are older than the two kernels that precede this one on the stream (consecutive
  // calls work on different layers' caches), so the first K/V tiles are requested before the
  // wait and the start-up latency of this kernel overlaps the tail of the previous ones.
  cudaTriggerProgrammaticLaunchCompletion();
  if (!p.early_kv) cudaGridDependencySynchronize();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.g.group;
  const int H = p.g.n_heads;

  const int len_old = p.kv_len_dev ? p.kv_len_dev[b] : p.kv_len;
  const int total = len_old + (p.append ? 1 : 0);
  const int nsplit = max(1, (total + p.chunk - 1) / p.chunk);
  // the grid was sized from the host's bound of the lengths: a longer sequence cannot be covered
  // (its last positions, the new token among them, would be dropped) -- tell the host
  if (split == 0 && nsplit > static_cast<int>(gridDim.x) && tid == 0 && p.error_flag)
    *reinterpret_cast<volatile int *>(p.error_flag) = kStatusLengthBeyondBound;
  if (split >= nsplit) return;
  const int pos0 = split * p.chunk;
  const int pos_end = min(total, pos0 + p.chunk);
  const int load_end = min(pos_end, len_old); // positions that exist in global memory
  const int rows = p.m * G;
  const bool has_new = p.append && pos_end == total;

  // flat cache: the sequence's block; paged cache: the pool, pages looked up per tile
  const bool paged = p.pg.table != nullptr;
  const int32_t *ptab = paged ? p.pg.table + static_cast<long>(b) * p.pg.table_stride : nullptr;
  const long seq_off = paged ? 0 : b * p.g.c_seq;
  const T *kbase = static_cast<const T *>(p.k_cache) + seq_off + kvh * p.g.c_head;
  const T *vbase = static_cast<const T *>(p.v_cache) + seq_off + kvh * p.g.c_head;
  // element offset of cache position pos (which must exist) from kbase / vbase
  auto pos_off = [&](int pos) -> long {
    if (!paged) return static_cast<long>(pos) * p.g.c_pos;
    return static_cast<long>(ptab[pos >> p.pg.page_shift]) * p.pg.page_stride +
           static_cast<long>(pos & ((1 << p.pg.page_shift) - 1)) * p.g.c_pos;
  };

  const int ntiles = (pos_end - pos0 + kTileN - 1) / kTileN;
  auto load_tile = [&](int t) {
    const int tpos = pos0 + t * kTileN;
    const uint32_t ks = smem_u32(stage_s + (t % kDecodeStages) * 2 * kTileBytes);
    const uint32_t vs = ks + kTileBytes;
    // a tile of 64 positions starts at a multiple of 64 and so lies inside one page
    const long tile_off = tpos < load_end ? pos_off(tpos) : 0;
#pragma unroll
    for (int it = 0; it < kTileN * 16 / kDecodeThreads; ++it) {
      const int cidx = tid + it * kDecodeThreads;
      const int row = cidx >> 4, chunk = cidx & 15;
      const int pos = tpos + row;
      const bool valid = pos < load_end;
      const long off = valid ? tile_off + row * p.g.c_pos + chunk * 8 : 0;
      cp_async16(ks + swz_off(row, chunk), kbase + off, valid ? 16 : 0);
      cp_async16(vs + swz_off(row, chunk), vbase + off, valid ? 16 : 0);
    }
  };

  // start the pipeline before the (latency-bound) prologue work
#pragma unroll
  for (int s = 0; s < kDecodeStages - 1; ++s) {
    if (s < ntiles) load_tile(s);
    cp_async_commit();
  }

  if (p.early_kv) cudaGridDependencySynchronize();

  // ---- query rows -> shared memory (rotated here when the caller passes raw q)
  const int rope_row = (p.rope_pos_dev ? p.rope_pos_dev[b] : len_old);
  for (int idx = tid; idx < 16 * 8; idx += kDecodeThreads) {
    const int rho = idx >> 3, i = idx & 7;
    uint4 u0 = make_uint4(0, 0, 0, 0), u1 = u0;
    const bool inter = p.rotate_q && !p.is_neox;
    const int c0 = inter ? 2 * i : i, c1 = inter ? 2 * i + 1 : i + 8;
    if (rho < rows) {
      const int r = rho / G, g = rho - r * G;
      const T *src = static_cast<const T *>(p.q) + b * p.g.q_seq + r * p.g.q_tok + (kvh * G + g) * kHeadDim;
      u0 = *reinterpret_cast<const uint4 *>(src + c0 * 8);
      u1 = *reinterpret_cast<const uint4 *>(src + c1 * 8);
      if (p.rotate_q) {
        const float4 *tab =
            reinterpret_cast<const float4 *>(p.freqs_cis + (static_cast<long>(rope_row) + r) * kHeadDim + 16 * i);
        rope_chunk_pair<T>(u0, u1, tab, p.is_neox != 0);
      }
    }
    *reinterpret_cast<uint4 *>(q_s + swz_off(rho, c0)) = u0;
    *reinterpret_cast<uint4 *>(q_s + swz_off(rho, c1)) = u1;
  }
  // ---- the new token: rotate K, keep K/V in shared memory for this CTA and
  //      write them to the cache for later steps
  if (has_new && tid < 16) {
    const int i = tid & 7;
    const bool is_k = tid < 8;
    const bool inter = is_k && !p.is_neox;
    const int c0 = inter ? 2 * i : i, c1 = inter ? 2 * i + 1 : i + 8;
    const T *src = static_cast<const T *>(is_k ? p.k_new : p.v_new) + b * p.kv_in_seq + kvh * kHeadDim;
    uint4 u0 = *reinterpret_cast<const uint4 *>(src + c0 * 8);
    uint4 u1 = *reinterpret_cast<const uint4 *>(src + c1 * 8);
    if (is_k) {
      const float4 *tab = reinterpret_cast<const float4 *>(p.freqs_cis + static_cast<long>(rope_row) * kHeadDim + 16 * i);
      rope_chunk_pair<T>(u0, u1, tab, p.is_neox != 0);
    }
    T *sdst = is_k ? knew_s : vnew_s;
    *reinterpret_cast<uint4 *>(sdst + c0 * 8) = u0;
    *reinterpret_cast<uint4 *>(sdst + c1 * 8) = u1;
    T *gdst = static_cast<T *>(is_k ? p.k_cache : p.v_cache) + seq_off + kvh * p.g.c_head + pos_off(len_old);
    *reinterpret_cast<uint4 *>(gdst + c0 * 8) = u0;
    *reinterpret_cast<uint4 *>(gdst + c1 * 8) = u1;
  }
  __syncthreads();

  uint32_t qa[8][4];
  load_q_frags(qa, smem_u32(q_s), 0, lane);

  // causal limits of this thread's two rows (positions >= limit are masked)
  int lim0 = INT_MAX, lim1 = INT_MAX;
  if (p.offset >= 0) {
    lim0 = p.offset + (lane >> 2) / G + 1;
    lim1 = p.offset + ((lane >> 2) + 8) / G + 1;
  }

  WarpAcc acc;
  acc.init();
  const int new_tile = has_new ? (len_old - pos0) / kTileN : -1;

  for (int t = 0; t < ntiles; ++t) {
    cp_async_wait<kDecodeStages - 2>();
    __syncthreads();
    // refill the stage consumed in the previous iteration
    if (t + kDecodeStages - 1 < ntiles) load_tile(t + kDecodeStages - 1);
    cp_async_commit();

    unsigned char *st = stage_s + (t % kDecodeStages) * 2 * kTileBytes;
    if (t == new_tile) {
      // the new token is not read back from global memory: patch its row in
      const int row = (len_old - pos0) - t * kTileN;
      if (tid < 32) {
        const int chunk = tid & 15;
        const T *src = (tid < 16) ? knew_s : vnew_s;
        unsigned char *dst = st + (tid < 16 ? 0 : kTileBytes) + swz_off(row, chunk);
        *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(src + chunk * 8);
      }
      __syncthreads();
    }
    const int col0 = pos0 + t * kTileN + warp * 16;
    if (col0 < pos_end) {
      warp_tile<T, 2>(acc, qa, smem_u32(st), smem_u32(st + kTileBytes), warp * 16, col0, pos_end, lim0, lim1,
                      p.scale_log2, lane);
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the four warps' states
  float *red_o = reinterpret_cast<float *>(stage_s);              // [4][16][kRedStride]
  float *red_ml = red_o + 4 * 16 * kRedStride;                    // [4][16][2]
  float sum0 = acc.sum[0], sum1 = acc.sum[1];
  sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
  sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
  sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
  sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
  {
    const int g0 = lane >> 2, cq = 2 * (lane & 3);
    float *r0 = red_o + (warp * 16 + g0) * kRedStride + cq;
    float *r1 = r0 + 8 * kRedStride;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      *reinterpret_cast<float2 *>(r0 + nt * 8) = make_float2(acc.o[nt][0], acc.o[nt][1]);
      *reinterpret_cast<float2 *>(r1 + nt * 8) = make_float2(acc.o[nt][2], acc.o[nt][3]);
    }
    if ((lane & 3) == 0) {
      red_ml[(warp * 16 + g0) * 2 + 0] = acc.mx[0];
      red_ml[(warp * 16 + g0) * 2 + 1] = sum0;
      red_ml[(warp * 16 + g0 + 8) * 2 + 0] = acc.mx[1];
      red_ml[(warp * 16 + g0 + 8) * 2 + 1] = sum1;
    }
  }
  __syncthreads();

  const int d = tid; // 128 threads, one per output column
  for (int rho = 0; rho < rows; ++rho) {
    float mw[4], M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      mw[w] = red_ml[(w * 16 + rho) * 2];
      M = fmaxf(M, mw[w]);
    }
    float L = 0.f, o = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = exp2f(mw[w] - M);
        L += f * red_ml[(w * 16 + rho) * 2 + 1];
        o += f * red_o[(w * 16 + rho) * kRedStride + d];
      }
    }
    const float res = (L > 0.f) ? o / L : 0.f;
    const int r = rho / G, g = rho - r * G;
    const int h = kvh * G + g;
    const long row_id = (static_cast<long>(b) * p.m + r) * H + h;
    if (p.max_splits > 1) {
      p.ws_o[(row_id * p.max_splits + split) * kHeadDim + d] = res;
      if (d == 0) p.ws_lse[row_id * p.max_splits + split] = (L > 0.f) ? M + log2f(L) : -INFINITY;
    } else if (p.o_partial) {
      p.o_partial[row_id * kHeadDim + d] = res;
      if (d == 0) p.lse_partial[row_id] = (L > 0.f) ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
    } else {
      static_cast<T *>(p.out)[b * p.g.out_seq + r * p.g.out_tok + h * kHeadDim + d] = Elem<T>::from_f32(res);
    }
  }
}

// grid: rows; block: 128 threads (one per output column)
template <typename T> __global__ void __launch_bounds__(128) attn_merge_kernel(MergeParams p) {
  cudaTriggerProgrammaticLaunchCompletion();
  cudaGridDependencySynchronize(); // the partials come from the previous kernel of the stream
  const int row = blockIdx.x, d = threadIdx.x;
  const int b = row / p.rows_per_seq;
  int n_parts = p.n_parts;
  if (n_parts <= 0) {
    const int total = (p.kv_len_dev ? p.kv_len_dev[b] : p.kv_len) + p.append;
    n_parts = max(1, (total + p.chunk - 1) / p.chunk);
  }
  n_parts = min(n_parts, p.max_parts); // never read beyond the row's slots, whatever the length says
  const float to_log2 = p.lse_is_log2 ? 1.f : kLog2e;
  float M = -INFINITY;
  // part i of this row: (lse index, o index / 128)
  auto lse_at = [&](int i) -> float {
    return p.part_major ? p.parts_lse[static_cast<long>(i) * p.part_stride_lse + row]
                        : p.parts_lse[static_cast<long>(row) * p.max_parts + i];
  };
  auto o_at = [&](int i) -> float {
    return p.part_major ? p.parts_o[static_cast<long>(i) * p.part_stride_o + static_cast<long>(row) * kHeadDim + d]
                        : p.parts_o[(static_cast<long>(row) * p.max_parts + i) * kHeadDim + d];
  };
  for (int i = 0; i < n_parts; ++i) M = fmaxf(M, lse_at(i) * to_log2);
  float W = 0.f, o = 0.f;
  if (M != -INFINITY) {
    for (int i = 0; i < n_parts; ++i) {
      const float w = exp2f(lse_at(i) * to_log2 - M);
      W += w;
      o += w * o_at(i);
    }
  }
  const float res = (W > 0.f) ? o / W : 0.f;
  if (p.o_partial) {
    p.o_partial[static_cast<long>(row) * kHeadDim + d] = res;
    if (d == 0) p.lse_partial[row] = (W > 0.f) ? (M + log2f(W)) * 0.6931471805599453f : -INFINITY;
  } else {
    const int rem = row - b * p.rows_per_seq;
    const int r = rem / p.n_heads, h = rem - r * p.n_heads;
    static_cast<T *>(p.out)[b * p.out_seq + r * p.out_tok + h * kHeadDim + d] = Elem<T>::from_f32(res);
  }
}

// ---------------------------------------------------------------------------
// General causal attention.  grid: (q tiles of 64 rows, heads, batch), the
// longest (last) q tile first; block: 4 warps x 16 rows; K/V in 64-position
// tiles, double-buffered with cp.async.
// ---------------------------------------------------------------------------
namespace {
constexpr int kPfRows = 64;
constexpr int kPfSmem = kPfRows * kRowBytes + 2 * 2 * kTileBytes; // 80 KB
} // namespace

template <typename T>
__global__ void __launch_bounds__(128, 2) attn_prefill_mma_kernel(PrefillParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char *q_s = smem;
  unsigned char *stage_s = smem + kPfRows * kRowBytes;

  const int qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kvh = h / p.g.group;
  const int row0 = qt * kPfRows;
  const int row_end = min(p.m, row0 + kPfRows);
  const int kv_end = min(p.n, p.offset + row_end); // last row sees positions < offset + row_end
  const int ntiles = (kv_end + kTileN - 1) / kTileN;

  const T *qbase = static_cast<const T *>(p.q) + b * p.g.q_seq + h * kHeadDim;
  // flat cache: the sequence's block; paged cache: the pool, one page lookup per tile of 64
  const bool paged = p.pg.table != nullptr;
  const int32_t *ptab = paged ? p.pg.table + static_cast<long>(b) * p.pg.table_stride : nullptr;
  const long seq_off = paged ? 0 : b * p.g.c_seq;
  const T *kbase = static_cast<const T *>(p.k_cache) + seq_off + kvh * p.g.c_head;
  const T *vbase = static_cast<const T *>(p.v_cache) + seq_off + kvh * p.g.c_head;

  auto load_tile = [&](int t) {
    const int tpos = t * kTileN;
    const uint32_t ks = smem_u32(stage_s + (t & 1) * 2 * kTileBytes);
    const uint32_t vs = ks + kTileBytes;
    long tile_off = static_cast<long>(tpos) * p.g.c_pos;
    if (paged && tpos < kv_end)
      tile_off = static_cast<long>(ptab[tpos >> p.pg.page_shift]) * p.pg.page_stride +
                 static_cast<long>(tpos & ((1 << p.pg.page_shift) - 1)) * p.g.c_pos;
#pragma unroll
    for (int it = 0; it < kTileN * 16 / 128; ++it) {
      const int cidx = tid + it * 128;
      const int row = cidx >> 4, chunk = cidx & 15;
      const int pos = tpos + row;
      const bool valid = pos < kv_end;
      const long off = valid ? tile_off + row * p.g.c_pos + chunk * 8 : 0;
      cp_async16(ks + swz_off(row, chunk), kbase + off, valid ? 16 : 0);
      cp_async16(vs + swz_off(row, chunk), vbase + off, valid ? 16 : 0);
    }
  };
  {
    const uint32_t qs = smem_u32(q_s);
#pragma unroll
    for (int it = 0; it < kPfRows * 16 / 128; ++it) {
      const int cidx = tid + it * 128;
      const int row = cidx >> 4, chunk = cidx & 15;
      const bool valid = row0 + row < p.m;
      const long off = valid ? (row0 + row) * p.g.q_tok + chunk * 8 : 0;
      cp_async16(qs + swz_off(row, chunk), qbase + off, valid ? 16 : 0);
    }
  }
  if (ntiles > 0) load_tile(0);
  cp_async_commit();

  uint32_t qa[8][4];
  WarpAcc acc;
  acc.init();
  const int r0 = row0 + warp * 16 + (lane >> 2);
  const int lim0 = p.offset + r0 + 1, lim1 = p.offset + r0 + 8 + 1;

  for (int t = 0; t < ntiles; ++t) {
    if (t + 1 < ntiles) load_tile(t + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (t == 0) load_q_frags(qa, smem_u32(q_s), warp * 16, lane);
    unsigned char *st = stage_s + (t & 1) * 2 * kTileBytes;
    // skip tiles entirely above this warp's rows
    if (t * kTileN < p.offset + row0 + warp * 16 + 16) {
      warp_tile<T, 8>(acc, qa, smem_u32(st), smem_u32(st + kTileBytes), 0, t * kTileN, kv_end, lim0, lim1,
                      p.scale_log2, lane);
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  float sum0 = acc.sum[0], sum1 = acc.sum[1];
  sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
  sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
  sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
  sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
  const float inv0 = sum0 > 0.f ? 1.f / sum0 : 0.f, inv1 = sum1 > 0.f ? 1.f / sum1 : 0.f;
  T *obase = static_cast<T *>(p.out) + b * p.g.out_seq + h * kHeadDim + 2 * (lane & 3);
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) {
    if (r0 < p.m)
      *reinterpret_cast<uint32_t *>(obase + r0 * p.g.out_tok + nt * 8) =
          Elem<T>::pack(acc.o[nt][0] * inv0, acc.o[nt][1] * inv0);
    if (r0 + 8 < p.m)
      *reinterpret_cast<uint32_t *>(obase + (r0 + 8) * p.g.out_tok + nt * 8) =
          Elem<T>::pack(acc.o[nt][2] * inv1, acc.o[nt][3] * inv1);
  }
}

// ---------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------
// The shared-memory opt-in is a property of (function, device): set it on the first launch of a
// function on a device.  (Keyed on the function's address: the two instantiations of a kernel
// template have the same pointer type.)
template <typename K> static cudaError_t set_smem(K kernel, int bytes) {
  static std::mutex mu;
  static std::vector<std::pair<const void *, int>> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const std::pair<const void *, int> key(reinterpret_cast<const void *>(kernel), dev);
  std::lock_guard<std::mutex> lk(mu);
  for (const auto &d : done)
    if (d == key) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done.push_back(key);
  return e;
}

// Launch with programmatic stream serialisation (programmatic dependent launch): the
// grid's CTAs may be placed on SMs as the previous kernel's CTAs retire, instead of
// after its last one has gone; the kernels order themselves with
// cudaGridDependencySynchronize().  Hides the launch and scheduling latency between
// the decode kernel, its merge and the next layer's decode kernel.
template <typename P>
static cudaError_t launch_pdl(void (*kernel)(P), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, const P &p) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

cudaError_t launch_attn_decode(const DecodeParams &p, bool bf16, cudaStream_t stream, int *launches) {
  static_assert(4 * 16 * kRedStride * 4 + 4 * 16 * 2 * 4 <= kDecodeStages * 2 * kTileBytes, "reduction buffer");
  cudaError_t e;
  dim3 grid(p.max_splits, p.g.n_kv_heads, p.g.batch);
  if (bf16) {
    if ((e = set_smem(attn_decode_kernel<__nv_bfloat16>, kDecodeSmem)) != cudaSuccess) return e;
    e = launch_pdl(attn_decode_kernel<__nv_bfloat16>, grid, dim3(kDecodeThreads), kDecodeSmem, stream, p);
  } else {
    if ((e = set_smem(attn_decode_kernel<__half>, kDecodeSmem)) != cudaSuccess) return e;
    e = launch_pdl(attn_decode_kernel<__half>, grid, dim3(kDecodeThreads), kDecodeSmem, stream, p);
  }
  if (e != cudaSuccess) return e;
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  *launches = 1;
  if (p.max_splits > 1 && !p.no_merge) {
    MergeParams mp{};
    mp.out = p.out;
    mp.o_partial = p.o_partial;
    mp.lse_partial = p.lse_partial;
    mp.parts_o = p.ws_o;
    mp.parts_lse = p.ws_lse;
    mp.part_major = 0;
    mp.lse_is_log2 = 1;
    mp.rows = p.g.batch * p.m * p.g.n_heads;
    mp.max_parts = p.max_splits;
    mp.n_parts = 0;
    mp.kv_len_dev = p.kv_len_dev;
    mp.kv_len = p.kv_len;
    mp.append = p.append ? 1 : 0;
    mp.chunk = p.chunk;
    mp.rows_per_seq = p.m * p.g.n_heads;
    mp.n_heads = p.g.n_heads;
    mp.m = p.m;
    mp.out_seq = p.g.out_seq;
    mp.out_tok = p.g.out_tok;
    if ((e = launch_attn_merge(mp, bf16, stream)) != cudaSuccess) return e;
    *launches = 2;
  }
  return cudaSuccess;
}

cudaError_t launch_attn_merge(const MergeParams &p, bool bf16, cudaStream_t stream) {
  if (p.rows <= 0) return cudaSuccess;
  cudaError_t e = bf16 ? launch_pdl(attn_merge_kernel<__nv_bfloat16>, dim3(p.rows), dim3(128), 0, stream, p)
                       : launch_pdl(attn_merge_kernel<__half>, dim3(p.rows), dim3(128), 0, stream, p);
  if (e != cudaSuccess) return e;
  return cudaGetLastError();
}

cudaError_t launch_attn_prefill_mma(const PrefillParams &p, bool bf16, cudaStream_t stream) {
  cudaError_t e;
  dim3 grid((p.m + kPfRows - 1) / kPfRows, p.g.n_heads, p.g.batch);
  if (bf16) {
    if ((e = set_smem(attn_prefill_mma_kernel<__nv_bfloat16>, kPfSmem)) != cudaSuccess) return e;
    attn_prefill_mma_kernel<__nv_bfloat16><<<grid, 128, kPfSmem, stream>>>(p);
  } else {
    if ((e = set_smem(attn_prefill_mma_kernel<__half>, kPfSmem)) != cudaSuccess) return e;
    attn_prefill_mma_kernel<__half><<<grid, 128, kPfSmem, stream>>>(p);
  }
  return cudaGetLastError();
}

} // namespace b200attn
