// Cross-device merge of split-KV decode partials over NVLink peer memory.
//
// When a very long cache is sharded by position over the GPUs of a node, every
// rank ends its decode step with a normalised partial output and its
// log-sum-exp per query head (20 KB for 40 heads), and every rank needs all of
// them.  Instead of a collective library call between two kernels, ONE kernel per
// rank does the exchange and the merge:
//   push blocks  (one per peer and four query rows) copy this rank's partial into
//                its slot of the peer's exchange buffer with plain stores over
//                NVLink, fence at system scope and release the rows' flags there;
//   merge blocks (one per query row) wait until every peer's flag in the LOCAL
//                buffer shows this step, then merge the slots from local memory
//                (same arithmetic and order as attn_merge_kernel, so the result
//                is bit-identical to the collective-based path).
// Peer buffers are ordinary device allocations opened through CUDA IPC; no
// multimem, no TMA.  The two kinds of block never wait on each other, and a
// waiting block only waits for kernels on OTHER GPUs.  Every wait is bounded
// (about a second): on expiry the block records an error code in the host-mapped
// status word and finishes.
//
// Buffer of one rank (floats / words), two halves used alternately by
// consecutive steps so that a fast peer cannot overwrite a slot that is still
// being merged:  half h: slots [world][rows*129] fp32, then flags [world][rows] u32.
// There is no counterpart in the reference, which is single-device.
#include "kernels.h"
#include "common.cuh"

namespace b200attn {

namespace {

constexpr int kPushRows = 4; // rows of 128 floats one push block of 128 threads moves with one float4 each

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

} // namespace

// Flags: one word per (source rank, query row) in each buffer half, so that a row can be pushed
// and merged as soon as it exists.
//
// grid, partial already merged on this rank (ws_o == nullptr): (world - 1) x ceil(rows / 4) push
// blocks, then `rows` merge blocks.  grid, partial still split (ws_o != nullptr): `rows` blocks; each merges
// its row's splits, pushes the row to every peer itself and then waits for the peers' rows.
// block: 128 threads.
template <typename T> __global__ void __launch_bounds__(128) attn_xchg_merge_kernel(XchgParams p) {
  const int tid = threadIdx.x;
  const long n = static_cast<long>(p.rows) * (kHeadDim + 1);
  const bool fused = p.ws_o != nullptr;
  const int row_groups = (p.rows + kPushRows - 1) / kPushRows;
  const int n_push = fused ? 0 : (p.world - 1) * row_groups;
  if (static_cast<int>(blockIdx.x) < n_push) {
    // ---- push: kPushRows rows of this rank's slot -> the same rows in one peer's buffer, one 16-byte
    // load and store per thread (a single round trip to local memory), then those rows' flags
    const int pi = static_cast<int>(blockIdx.x) / row_groups, rg = static_cast<int>(blockIdx.x) % row_groups;
    const int peer = pi < p.rank ? pi : pi + 1;
    const int r0 = rg * kPushRows, nr = min(kPushRows, p.rows - r0);
    const float *src = p.slots + static_cast<long>(p.rank) * n;
    float *dst = p.peer_slot[peer];
    if (tid < nr * (kHeadDim / 4)) {
      const long i = static_cast<long>(r0) * kHeadDim + 4 * tid;
      if ((n & 3) == 0) {           // the ranks' slots lie n floats apart: 16-byte aligned when that is a multiple of 4
        *reinterpret_cast<float4 *>(dst + i) = __ldcg(reinterpret_cast<const float4 *>(src + i));
      } else {
        const float a = __ldcg(src + i), b = __ldcg(src + i + 1), c = __ldcg(src + i + 2), e = __ldcg(src + i + 3);
        dst[i] = a, dst[i + 1] = b, dst[i + 2] = c, dst[i + 3] = e;
      }
    }
    if (tid < nr) {
      const long i = static_cast<long>(p.rows) * kHeadDim + r0 + tid;
      dst[i] = __ldcg(src + i);
    }
    __threadfence_system();
    __syncthreads();
    if (tid < nr) st_release_sys(p.peer_flag[peer] + r0 + tid, p.epoch);
    return;
  }
  const int row = blockIdx.x - n_push, d = tid;
  if (fused) {
    // ---- this rank's splits of the row -> one partial (the arithmetic of attn_merge_kernel)
    const int b = row / p.rows_per_seq;
    const int total = p.kv_len_dev[b] + p.append;
    const int n_parts = min(max(1, (total + p.chunk - 1) / p.chunk), p.max_splits); // never beyond the row's slots
    float M = -INFINITY;
    for (int i = 0; i < n_parts; ++i) M = fmaxf(M, p.ws_lse[static_cast<long>(row) * p.max_splits + i]);
    float W = 0.f, o = 0.f;
    if (M != -INFINITY) {
      for (int i = 0; i < n_parts; ++i) {
        const float w = exp2f(p.ws_lse[static_cast<long>(row) * p.max_splits + i] - M);
        W += w;
        o += w * p.ws_o[(static_cast<long>(row) * p.max_splits + i) * kHeadDim + d];
      }
    }
    const float res = (W > 0.f) ? o / W : 0.f;
    const float lse = (W > 0.f) ? (M + log2f(W)) * 0.6931471805599453f : -INFINITY;
    const long o_idx = static_cast<long>(row) * kHeadDim + d, l_idx = static_cast<long>(p.rows) * kHeadDim + row;
    float *mine = const_cast<float *>(p.slots) + static_cast<long>(p.rank) * n;
    mine[o_idx] = res;
    if (d == 0) mine[l_idx] = lse;
    for (int r = 0; r < p.world; ++r) {
      if (r == p.rank) continue;
      p.peer_slot[r][o_idx] = res;
      if (d == 0) p.peer_slot[r][l_idx] = lse;
    }
    __threadfence_system();
    __syncthreads();
    if (tid < p.world && tid != p.rank) st_release_sys(p.peer_flag[tid] + row, p.epoch);
  }
  // ---- wait for every peer's partial of this row and step, then combine
  __shared__ int s_ok;
  if (tid == 0) {
    int ok = 1;
    const long long t0 = clock64();
    for (int r = 0; r < p.world && ok; ++r) {
      if (r == p.rank) continue;
      while (ld_acquire_sys(p.flags + static_cast<long>(r) * p.rows + row) != p.epoch) {
        if (clock64() - t0 > 2000000000LL) {
          *reinterpret_cast<volatile int *>(p.error_flag) = 20 + r; // gave up waiting for rank r
          ok = 0;
          break;
        }
        __nanosleep(64);
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return; // the output row stays unwritten; the host sees the status word
  // the slots were written by other GPUs (and, fused, just now by this block): read them around L1
  auto lse_at = [&](int i) { return __ldcg(p.slots + i * n + static_cast<long>(p.rows) * kHeadDim + row); };
  auto o_at = [&](int i) { return __ldcg(p.slots + i * n + static_cast<long>(row) * kHeadDim + d); };
  float M = -INFINITY;
  for (int i = 0; i < p.world; ++i) M = fmaxf(M, lse_at(i) * kLog2e);
  float W = 0.f, o = 0.f;
  if (M != -INFINITY) {
    for (int i = 0; i < p.world; ++i) {
      const float w = exp2f(lse_at(i) * kLog2e - M);
      W += w;
      o += w * o_at(i);
    }
  }
  const float res = (W > 0.f) ? o / W : 0.f;
  static_cast<T *>(p.out)[static_cast<long>(row) * kHeadDim + d] = Elem<T>::from_f32(res);
}

cudaError_t launch_attn_xchg_merge(const XchgParams &p, bool bf16, cudaStream_t stream) {
  const int row_groups = (p.rows + kPushRows - 1) / kPushRows;
  const unsigned blocks = static_cast<unsigned>((p.ws_o ? 0 : (p.world - 1) * row_groups) + p.rows);
  if (bf16)
    attn_xchg_merge_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(p);
  else
    attn_xchg_merge_kernel<__half><<<blocks, 128, 0, stream>>>(p);
  return cudaGetLastError();
}

} // namespace b200attn
