// Planned grouped-query decode over the KV cache: persistent CTAs fed by TMA.
//
// The fused decode step (RoPE of the new token's Q/K, KV append, attention over
// the cache) for a batch of sequences of different lengths, with the work cut on
// the host (kernels.h: PlanHeader / PlanItem; decode_plan.cpp).  Every (sequence,
// KV head) cache is a run of 64-position tiles; the runs are laid end to end and
// every CTA owns one contiguous, equally expensive share of that line.  A CTA
// walks through its few pieces in a row and its load ring never drains between
// them.
//
// 192 threads per CTA in three roles:
//   warps 0-3  consumers: the arithmetic of attn_decode_kernel (attn_mma.cu) --
//              ldmatrix + mma.sync m16n8k16 with fp32 accumulation, online softmax
//              in the log2 domain, each warp 16 of a tile's 64 positions against
//              the (up to 16) query rows of the KV head; at the end of a piece the
//              four warps' states are combined through the ring stage just emptied
//   warp 4     one lane: TMA producer.  Per tile two boxes of K and two of V
//              ([64 positions][64 elements], 128-byte swizzle) into a 3-stage ring
//              of 32 KB stages behind full/empty mbarriers; the ragged last tile
//              of a cache is fetched in boxes of 16 positions so that at most 15
//              rows beyond the sequence are read.  No multicast.
//   warp 5     stages the next piece's query rows (rotated) and, for the piece
//              that ends a cache, the new token: K rotated, K/V written to the
//              cache and kept in shared memory, from where the consumers patch
//              it into the tile (it is never read back from HBM)
// A piece that is a whole cache writes the result.  The pieces of a cache that
// was cut leave a normalised partial + log-sum-exp each in a scratch slot, and
// attn_plan_merge_kernel, launched behind this kernel as a programmatic
// dependent, merges them with one warp per piece, so that all partials of a
// cache are fetched in a single round trip however many pieces it has.
//
// HBM-bound: every K/V byte is read once; algorithmic bytes per sequence
// 2*kvH*L*256 + 2*H*256 + 4*kvH*256 (L includes the new token).
// Reference semantics: tests/flash_attn_test.cpp:106-192 with m = 1; GQA head
// mapping q_head / group (src/llama2_layer_npu.cpp:866-869); the RoPE + append it
// fuses: src/llama2_layer_npu.cpp:790-798, :830-843.
//
// Every mbarrier wait is bounded (about a second); on expiry the waiter records a
// code in the host-visible status word and the CTA runs to its end.
#include "kernels.h"
#include "common.cuh"
#include "tma.cuh"

#include <limits.h>

namespace b200attn {

namespace dtma {

using namespace tma;

constexpr int kConsumerWarps = 4;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 64;   // + TMA warp + staging warp
constexpr int kStages = 3;
constexpr int kTileN = 64;                        // positions per stage
constexpr uint32_t kHalfBytes = kTileN * 128;     // [64][64 elements] half tile
constexpr uint32_t kTensorTile = 2 * kHalfBytes;  // K or V tile, 16 KB
constexpr uint32_t kStageBytes = 2 * kTensorTile; // K + V

constexpr uint32_t kOffStages = 0;
constexpr uint32_t kOffQ = kOffStages + kStages * kStageBytes;       // 16 rows x 256 B
constexpr uint32_t kOffNew = kOffQ + 16 * kRowBytes;                 // [parity][K, V][128]
constexpr uint32_t kOffRedMl = kOffNew + 2 * 2 * kRowBytes;          // [4 warps][16 rows][max, sum]
constexpr uint32_t kOffBar = kOffRedMl + kConsumerWarps * 16 * 2 * 4;
constexpr uint32_t kSmemTotal = kOffBar + 128;
static_assert(kSmemTotal <= 115712, "two CTAs per SM");
// The four warps' accumulators of a piece meet in the ring stage the piece has just emptied:
// [4 warps][16 rows][128] fp32 is exactly one stage.
static_assert(kConsumerWarps * 16 * kHeadDim * 4 == kStageBytes, "combine buffer = one stage");

// barrier slots
enum { BAR_FULL = 0, BAR_EMPTY = kStages, BAR_QREADY = 2 * kStages, BAR_QFREE, BAR_COUNT };
static_assert(BAR_COUNT * 8 + 8 <= 128, "barrier block");

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }

} // namespace dtma

template <typename T>
__global__ void __launch_bounds__(dtma::kThreads, 2)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const __grid_constant__ CUtensorMap map_k16, const __grid_constant__ CUtensorMap map_v16,
                       PlannedDecodeParams p) {
  using namespace dtma;
  // the ring's tiles need 1024-byte alignment (128-byte swizzle): the dynamic shared memory of a
  // kernel without static shared memory starts on such a boundary (checked below)
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t smem_base = smem_u32(smem);
  unsigned char *q_s = smem + kOffQ;
  T *new_s = reinterpret_cast<T *>(smem + kOffNew);
  float *red_ml = reinterpret_cast<float *>(smem + kOffRedMl);
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(smem + kOffBar + BAR_COUNT * 8);
  auto bar = [&](int i) { return smem_base + kOffBar + 8u * i; };

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.g.group, H = p.g.n_heads;

  // Launched with programmatic stream serialisation: let the next kernel of the stream in as
  // early as possible; nothing the preceding kernels may still write or read is touched before
  // cudaGridDependencySynchronize().  The plan is older than that (it is uploaded once per step),
  // and so are, when the caller says so (early_kv), the cache rows below the cached lengths.
  cudaTriggerProgrammaticLaunchCompletion();
  if (!p.early_kv) cudaGridDependencySynchronize();

  const int32_t *cta_begin = reinterpret_cast<const int32_t *>(p.plan + p.off_cta_begin);
  const PlanItem *items = reinterpret_cast<const PlanItem *>(p.plan + p.off_items);
  const int it0 = cta_begin[blockIdx.x], it1 = cta_begin[blockIdx.x + 1];
  auto load_item = [&](int it) -> PlanItem {
    const int4 *src = reinterpret_cast<const int4 *>(items + it);
    const int4 a = __ldg(src), b = __ldg(src + 1);
    PlanItem w;
    w.b = a.x, w.kvh = a.y, w.pos0 = a.z, w.pos_end = a.w;
    w.len_old = b.x, w.slot = b.y, w.has_new = b.z, w.reserved = b.w;
    return w;
  };
  if (tid == 0) {
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(BAR_FULL + s), 1);
      mbar_init(bar(BAR_EMPTY + s), kConsumerWarps);
    }
    mbar_init(bar(BAR_QREADY), 1);
    mbar_init(bar(BAR_QFREE), kConsumerWarps);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if ((smem_base & 1023u) != 0) {
    if (tid == 0) *reinterpret_cast<volatile int *>(p.error_flag) = 30;
    return;
  }
  // query rows beyond the group stay zero for the whole kernel
  for (int i = tid; i < 16 * kRowBytes / 16; i += kThreads) reinterpret_cast<uint4 *>(q_s)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  if (it0 >= it1) return;

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------------ TMA producer
    if (lane != 0) return;
    const bool paged = p.pg.table != nullptr;
    uint32_t g = 0;
    for (int it = it0; it < it1; ++it) {
      const PlanItem w = load_item(it);
      const int load_end = min(w.pos_end, w.len_old);            // positions that exist in global memory
      const int ntiles = (w.pos_end - w.pos0 + kTileN - 1) / kTileN;
      for (int t = 0; t < ntiles; ++t, ++g) {
        const int s = g % kStages;
        if (!mbar_wait(bar(BAR_EMPTY + s), ((g / kStages) & 1) ^ 1, abort_flag, p.error_flag, 31)) return;
        const int tpos = w.pos0 + t * kTileN;
        const int rows = max(0, min(kTileN, load_end - tpos));
        int c1 = tpos, c3 = w.b;
        if (paged && rows > 0) {
          // a tile of 64 positions starts at a multiple of 64 and so lies inside one page
          c3 = p.pg.table[static_cast<long>(w.b) * p.pg.table_stride + (tpos >> p.pg.page_shift)];
          c1 = tpos & ((1 << p.pg.page_shift) - 1);
        }
        const uint32_t full = bar(BAR_FULL + s);
        const uint32_t dk = smem_base + kOffStages + s * kStageBytes, dv = dk + kTensorTile;
        if (rows == kTileN) {
          mbar_expect_tx(full, kStageBytes);
          tma_load_4d(dk, &map_k, full, 0, c1, w.kvh, c3);
          tma_load_4d(dk + kHalfBytes, &map_k, full, 64, c1, w.kvh, c3);
          tma_load_4d(dv, &map_v, full, 0, c1, w.kvh, c3);
          tma_load_4d(dv + kHalfBytes, &map_v, full, 64, c1, w.kvh, c3);
        } else if (rows == 0) {
          mbar_arrive(full); // the tile holds the new token only, which comes from shared memory
        } else {
          // ragged end of the cache: boxes of 16 positions, placed where a full box would put them
          const int nsub = (rows + 15) / 16;
          mbar_expect_tx(full, static_cast<uint32_t>(nsub) * 16 * 128 * 4);
          for (int j = 0; j < nsub; ++j) {
            const uint32_t o = static_cast<uint32_t>(j) * 16 * 128;
            tma_load_4d(dk + o, &map_k16, full, 0, c1 + 16 * j, w.kvh, c3);
            tma_load_4d(dk + kHalfBytes + o, &map_k16, full, 64, c1 + 16 * j, w.kvh, c3);
            tma_load_4d(dv + o, &map_v16, full, 0, c1 + 16 * j, w.kvh, c3);
            tma_load_4d(dv + kHalfBytes + o, &map_v16, full, 64, c1 + 16 * j, w.kvh, c3);
          }
        }
      }
    }
    return;
  }

  if (warp == kConsumerWarps + 1) {
    // ------------------------------------------------------------------ query / new-token staging
    PlanItem w_next = load_item(it0); // the plan and the table positions are older than the preceding kernels
    int rope_next = p.rope_pos_dev ? __ldg(p.rope_pos_dev + w_next.b) : w_next.len_old;
    if (p.early_kv) cudaGridDependencySynchronize(); // q and the new token may come from the preceding kernels
    for (int it = it0; it < it1; ++it) {
      const int i = it - it0;
      const PlanItem w = w_next;
      const int rope_row = rope_next;
      if (it + 1 < it1) {
        w_next = load_item(it + 1);
        rope_next = p.rope_pos_dev ? __ldg(p.rope_pos_dev + w_next.b) : w_next.len_old;
      }
      // the consumers have taken the previous piece's rows into registers
      if (i > 0 && !mbar_wait(bar(BAR_QFREE), (i - 1) & 1, abort_flag, p.error_flag, 32)) return;
      for (int idx = lane; idx < G * 8; idx += 32) {
        const int rho = idx >> 3, j = idx & 7;
        const bool inter = !p.is_neox;
        const int c0 = inter ? 2 * j : j, c1 = inter ? 2 * j + 1 : j + 8;
        const T *src = static_cast<const T *>(p.q) + w.b * p.g.q_seq + (w.kvh * G + rho) * kHeadDim;
        uint4 u0 = *reinterpret_cast<const uint4 *>(src + c0 * 8);
        uint4 u1 = *reinterpret_cast<const uint4 *>(src + c1 * 8);
        const float4 *tab = reinterpret_cast<const float4 *>(p.freqs_cis + static_cast<long>(rope_row) * kHeadDim + 16 * j);
        rope_chunk_pair<T>(u0, u1, tab, p.is_neox != 0);
        *reinterpret_cast<uint4 *>(q_s + swz_off(rho, c0)) = u0;
        *reinterpret_cast<uint4 *>(q_s + swz_off(rho, c1)) = u1;
      }
      if (w.has_new && lane < 16) {
        // the new token: rotate K, keep K/V in shared memory for the consumers and write them
        // to the cache for later steps
        const int j = lane & 7;
        const bool is_k = lane < 8;
        const bool inter = is_k && !p.is_neox;
        const int c0 = inter ? 2 * j : j, c1 = inter ? 2 * j + 1 : j + 8;
        const T *src = static_cast<const T *>(is_k ? p.k_new : p.v_new) + w.b * p.kv_in_seq + w.kvh * kHeadDim;
        uint4 u0 = *reinterpret_cast<const uint4 *>(src + c0 * 8);
        uint4 u1 = *reinterpret_cast<const uint4 *>(src + c1 * 8);
        if (is_k) {
          const float4 *tab = reinterpret_cast<const float4 *>(p.freqs_cis + static_cast<long>(rope_row) * kHeadDim + 16 * j);
          rope_chunk_pair<T>(u0, u1, tab, p.is_neox != 0);
        }
        T *sdst = new_s + ((i & 1) * 2 + (is_k ? 0 : 1)) * kHeadDim;
        *reinterpret_cast<uint4 *>(sdst + c0 * 8) = u0;
        *reinterpret_cast<uint4 *>(sdst + c1 * 8) = u1;
        long off;
        if (p.pg.table) {
          const long page = p.pg.table[static_cast<long>(w.b) * p.pg.table_stride + (w.len_old >> p.pg.page_shift)];
          off = page * p.pg.page_stride + static_cast<long>(w.len_old & ((1 << p.pg.page_shift) - 1)) * p.g.c_pos;
        } else {
          off = w.b * p.g.c_seq + static_cast<long>(w.len_old) * p.g.c_pos;
        }
        T *gdst = static_cast<T *>(is_k ? p.k_cache : p.v_cache) + off + w.kvh * p.g.c_head;
        *reinterpret_cast<uint4 *>(gdst + c0 * 8) = u0;
        *reinterpret_cast<uint4 *>(gdst + c1 * 8) = u1;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_QREADY));
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  PlanItem w_next = load_item(it0); // the plan is older than the preceding kernels: read it before the wait
  // outputs and scratch may still be in use by the preceding kernels of the stream
  if (p.early_kv) cudaGridDependencySynchronize();
  uint32_t g = 0;
  const int g0 = lane >> 2, cq = 2 * (lane & 3);
  const int orow = tid >> 3, ocol = (tid & 7) * 4; // output row / first column of this thread in the combines

  // The four warps' (max, sum) of a piece -> red_ml; then, per thread, the factor that turns its
  // accumulators into its warp's share of the normalised result.
  auto publish_ml = [&](const WarpAcc &acc) {
    float sum0 = acc.sum[0], sum1 = acc.sum[1];
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    if ((lane & 3) == 0) {
      red_ml[(warp * 16 + g0) * 2 + 0] = acc.mx[0];
      red_ml[(warp * 16 + g0) * 2 + 1] = sum0;
      red_ml[(warp * 16 + g0 + 8) * 2 + 0] = acc.mx[1];
      red_ml[(warp * 16 + g0 + 8) * 2 + 1] = sum1;
    }
    consumer_sync();
  };
  // row maximum M and total weight L over the four warps
  auto row_ml = [&](int row, float &M, float &L) {
    float mw[kConsumerWarps];
    M = -INFINITY;
#pragma unroll
    for (int x = 0; x < kConsumerWarps; ++x) {
      mw[x] = red_ml[(x * 16 + row) * 2];
      M = fmaxf(M, mw[x]);
    }
    L = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int x = 0; x < kConsumerWarps; ++x) L += exp2f(mw[x] - M) * red_ml[(x * 16 + row) * 2 + 1];
    }
  };
  auto own_factors = [&](const WarpAcc &acc, float &f0, float &f1) {
    float M0, L0, M1, L1;
    row_ml(g0, M0, L0);
    row_ml(g0 + 8, M1, L1);
    f0 = (L0 > 0.f && acc.mx[0] != -INFINITY) ? exp2f(acc.mx[0] - M0) / L0 : 0.f;
    f1 = (L1 > 0.f && acc.mx[1] != -INFINITY) ? exp2f(acc.mx[1] - M1) / L1 : 0.f;
  };
  auto row_lse2 = [&](int row) -> float {
    float M, L;
    row_ml(row, M, L);
    return (L > 0.f) ? M + log2f(L) : -INFINITY;
  };
  // where a piece's (or a merged run's) result goes: four columns of one row, and the row's log-sum-exp
  auto write4 = [&](const PlanItem &w, int row, int col, const float4 &v) {
    const long row_id = static_cast<long>(w.b) * H + static_cast<long>(w.kvh) * G + row;
    if (w.slot >= 0) {
      *reinterpret_cast<float4 *>(p.ws_o + (static_cast<long>(w.slot) * G + row) * kHeadDim + col) = v;
    } else if (p.o_partial) {
      *reinterpret_cast<float4 *>(p.o_partial + row_id * kHeadDim + col) = v;
    } else {
      uint2 u;
      u.x = Elem<T>::pack(v.x, v.y);
      u.y = Elem<T>::pack(v.z, v.w);
      T *dst = static_cast<T *>(p.out) + w.b * p.g.out_seq + (w.kvh * G + row) * kHeadDim + col;
      *reinterpret_cast<uint2 *>(dst) = u;
    }
  };
  auto write_lse = [&](const PlanItem &w, int row, float lse2) {
    if (w.slot >= 0) p.ws_lse[static_cast<long>(w.slot) * G + row] = lse2;
    else if (p.o_partial)
      p.lse_partial[static_cast<long>(w.b) * H + static_cast<long>(w.kvh) * G + row] = lse2 * 0.6931471805599453f;
  };
  // Combines the four warps' states of a piece through `buf` (one free ring stage): leaves in v[k]
  // this thread's four columns ocol + 32 k of row orow of the normalised result (threads with
  // orow < G), in lse2 the row's log-sum-exp (log2 domain).
  auto combine = [&](const WarpAcc &acc, float *buf, float4 (&v)[4], float &lse2) {
    publish_ml(acc);
    float f0, f1;
    own_factors(acc, f0, f1);
    lse2 = orow < G ? row_lse2(orow) : -INFINITY;
    float *r0 = buf + (warp * 16 + g0) * kHeadDim + cq;
    float *r1 = r0 + 8 * kHeadDim;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      // rotate the column blocks by the row so that the eight rows of a warp hit different banks
      const int c = ((nt + g0) & 15) * 8;
      *reinterpret_cast<float2 *>(r0 + c) = make_float2(acc.o[nt][0] * f0, acc.o[nt][1] * f0);
      *reinterpret_cast<float2 *>(r1 + c) = make_float2(acc.o[nt][2] * f1, acc.o[nt][3] * f1);
    }
    consumer_sync();
    if (orow < G) {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int col = ocol + 32 * k;
        const int c = (((col >> 3) + (orow & 7)) & 15) * 8 + (col & 7); // where combine's writers put this column
        v[k] = *reinterpret_cast<const float4 *>(buf + orow * kHeadDim + c);
#pragma unroll
        for (int x = 1; x < kConsumerWarps; ++x) {
          const float4 u = *reinterpret_cast<const float4 *>(buf + (x * 16 + orow) * kHeadDim + c);
          v[k].x += u.x, v[k].y += u.y, v[k].z += u.z, v[k].w += u.w;
        }
      }
    }
    consumer_sync(); // the buffer may be written again
  };
  WarpAcc acc;
  PlanItem w = w_next;
  for (int it = it0; it < it1; ++it) {
    const int i = it - it0;
    w = w_next;
    if (it + 1 < it1) w_next = load_item(it + 1);
    if (!mbar_wait(bar(BAR_QREADY), i & 1, abort_flag, p.error_flag, 33)) return;
    uint32_t qa[8][4];
    load_q_frags(qa, smem_u32(q_s), 0, lane);
    __syncwarp();
    if (lane == 0) mbar_arrive(bar(BAR_QFREE));

    acc.init();
    const int ntiles = (w.pos_end - w.pos0 + kTileN - 1) / kTileN;
    for (int t = 0; t < ntiles; ++t, ++g) {
      const int s = g % kStages;
      if (!mbar_wait(bar(BAR_FULL + s), (g / kStages) & 1, abort_flag, p.error_flag, 34)) return;
      unsigned char *st = smem + kOffStages + s * kStageBytes;
      const int tpos = w.pos0 + t * kTileN;
      const int valid = min(kTileN, w.pos_end - tpos); // rows of the tile that take part
      const bool fix = valid < kTileN || (w.has_new && t == ntiles - 1);
      if (fix) {
        // last tile of a cache: the new token's row comes from shared memory, and the V rows
        // beyond the sequence (stale or never written) must not meet a zero weight as NaN
        if (w.has_new && tid < 32) {
          const int row = w.len_old - tpos, chunk = tid & 15;
          const T *src = new_s + ((i & 1) * 2 + (tid < 16 ? 0 : 1)) * kHeadDim;
          unsigned char *dst = st + (tid < 16 ? 0 : kTensorTile) + tile_off<kHalfBytes>(row, chunk);
          *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(src + chunk * 8);
        }
        for (int c = tid; c < (kTileN - valid) * 16; c += kConsumerThreads) {
          const int row = valid + (c >> 4), chunk = c & 15;
          *reinterpret_cast<uint4 *>(st + kTensorTile + tile_off<kHalfBytes>(row, chunk)) = make_uint4(0, 0, 0, 0);
        }
        consumer_sync();
      }
      const int col0 = tpos + warp * 16;
      if (col0 < w.pos_end) {
        warp_tile<T, 2, kHalfBytes>(acc, qa, smem_u32(st), smem_u32(st + kTensorTile), warp * 16, col0, w.pos_end,
                                    INT_MAX, INT_MAX, p.scale_log2, lane);
      }
      // the stage of a piece's last tile is kept a moment longer: the warps combine through it
      if (t == ntiles - 1 && it != it1 - 1) break;
      if (fix) fence_proxy_async_smem(); // the stage was written by hand; TMA writes it next
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_EMPTY + s));
    }
    if (it == it1 - 1) break; // the share's last piece: handled below, with the ring drained

    // ---- a piece before the share's last one
    float4 v[4];
    float lse2 = -INFINITY;
    if (ntiles > 0) {
      const int s = g % kStages; // the stage just consumed, not yet handed back
      combine(acc, reinterpret_cast<float *>(smem + kOffStages + s * kStageBytes), v, lse2);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_EMPTY + s));
      ++g;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = make_float4(0.f, 0.f, 0.f, 0.f); // an empty cache: zero result
    }
    if (orow < G) {
#pragma unroll
      for (int k = 0; k < 4; ++k) write4(w, orow, ocol + 32 * k, v[k]);
      if ((tid & 7) == 0) write_lse(w, orow, lse2);
    }
  }

  // ---- the share's last piece: every tile has been consumed and no copy is in flight, so any
  //      stage of the ring serves as the combine buffer
  consumer_sync(); // every warp has left the last tile
  float4 v[4];
  float lse2;
  combine(acc, reinterpret_cast<float *>(smem + kOffStages), v, lse2);
  if (orow < G) {
#pragma unroll
    for (int k = 0; k < 4; ++k) write4(w, orow, ocol + 32 * k, v[k]);
    if ((tid & 7) == 0) write_lse(w, orow, lse2);
  }
}

// Merges the pieces of every (sequence, KV head) cache that the plan cut.
// grid: (groups, query rows of a KV head); block: 32 lanes (four output columns each) x
// min(pieces, kMergeWarps) warps.  Warp i folds pieces i, i + warps, ... (normalised partial +
// log-sum-exp each, in slot order), the warps' results meet in shared memory and warp 0 combines
// them in warp order: a fixed summation order.
namespace dtma {
constexpr int kMergeWarps = 32;
}
template <typename T> __global__ void __launch_bounds__(32 * dtma::kMergeWarps) attn_plan_merge_kernel(PlannedDecodeParams p) {
  __shared__ float4 xo[dtma::kMergeWarps][32];
  __shared__ float2 xml[dtma::kMergeWarps];
  cudaTriggerProgrammaticLaunchCompletion();
  const PlanGroup *groups = reinterpret_cast<const PlanGroup *>(p.plan + p.off_groups);
  const int4 ga = __ldg(reinterpret_cast<const int4 *>(groups + blockIdx.x)); // the plan is older than the partials
  const int first = ga.x, n_parts = min(ga.y, p.n_slots - ga.x); // never beyond the scratch the plan sized
  const int G = p.g.group, r = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = blockDim.x >> 5;
  cudaGridDependencySynchronize(); // the partials come from the previous kernel of the stream
  float M = -INFINITY, W = 0.f;
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int x = warp; x < n_parts; x += n_warps) {
    const long slot_row = static_cast<long>(first + x) * G + r;
    const float l = p.ws_lse[slot_row];
    const float4 v = *reinterpret_cast<const float4 *>(p.ws_o + slot_row * kHeadDim + lane * 4);
    if (l != -INFINITY) {
      const float mn = fmaxf(M, l);
      const float fa = exp2f(M - mn), fb = exp2f(l - mn); // fa = 0 for the first piece
      W = W * fa + fb;
      o.x = o.x * fa + fb * v.x, o.y = o.y * fa + fb * v.y, o.z = o.z * fa + fb * v.z, o.w = o.w * fa + fb * v.w;
      M = mn;
    }
  }
  xo[warp][lane] = o;
  if (lane == 0) xml[warp] = make_float2(M, W);
  __syncthreads();
  if (warp != 0) return;
  float Mx = -INFINITY;
  for (int x = 0; x < n_warps; ++x) Mx = fmaxf(Mx, xml[x].x);
  float Wt = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (Mx != -INFINITY) {
    for (int x = 0; x < n_warps; ++x) {
      const float2 ml = xml[x];
      if (ml.x == -INFINITY) continue;
      const float f = exp2f(ml.x - Mx);
      const float4 u = xo[x][lane];
      Wt += f * ml.y;
      acc.x += f * u.x, acc.y += f * u.y, acc.z += f * u.z, acc.w += f * u.w;
    }
  }
  if (Wt > 0.f) acc.x /= Wt, acc.y /= Wt, acc.z /= Wt, acc.w /= Wt;
  const int b = ga.z, h = ga.w * G + r;
  const long row = static_cast<long>(b) * p.g.n_heads + h;
  if (p.o_partial) {
    *reinterpret_cast<float4 *>(p.o_partial + row * kHeadDim + lane * 4) = acc;
    if (lane == 0) p.lse_partial[row] = (Wt > 0.f) ? (Mx + log2f(Wt)) * 0.6931471805599453f : -INFINITY;
  } else {
    uint2 u;
    u.x = Elem<T>::pack(acc.x, acc.y);
    u.y = Elem<T>::pack(acc.z, acc.w);
    *reinterpret_cast<uint2 *>(static_cast<T *>(p.out) + b * p.g.out_seq + h * kHeadDim + lane * 4) = u;
  }
}

namespace {

template <typename... Args>
cudaError_t launch_pdl(void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
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
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// the shared-memory opt-in is a per-device property of the function: set it once per device
template <typename T> cudaError_t opt_in_smem() {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !attr_set[dev]) {
    e = cudaFuncSetAttribute(attn_decode_tma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, dtma::kSmemTotal);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) attr_set[dev] = true;
  }
  return cudaSuccess;
}

template <typename T>
cudaError_t launch_typed(const PlannedDecodeParams &p, const CUtensorMap &mk, const CUtensorMap &mv,
                         const CUtensorMap &mk16, const CUtensorMap &mv16, cudaStream_t stream, int *launches) {
  cudaError_t e = opt_in_smem<T>();
  if (e != cudaSuccess) return e;
  e = launch_pdl(attn_decode_tma_kernel<T>, dim3(p.n_ctas), dim3(dtma::kThreads), dtma::kSmemTotal, stream, mk,
                 mv, mk16, mv16, p);
  if (e != cudaSuccess) return e;
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  *launches = 1;
  if (p.n_groups > 0) {
    const int warps = p.max_parts < dtma::kMergeWarps ? (p.max_parts > 0 ? p.max_parts : 1) : dtma::kMergeWarps;
    e = launch_pdl(attn_plan_merge_kernel<T>, dim3(p.n_groups, p.g.group), dim3(32 * warps), 0, stream, p);
    if (e != cudaSuccess) return e;
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    *launches = 2;
  }
  return cudaSuccess;
}

} // namespace

// CTAs of attn_decode_tma_kernel that the current device can hold at once; 0 on failure.
int decode_planned_max_ctas() {
  static int cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev]) return cached[dev] > 0 ? cached[dev] : 0;
  int result = -1, per_sm = 0, sms = 0;
  if (opt_in_smem<__nv_bfloat16>() == cudaSuccess &&
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_tma_kernel<__nv_bfloat16>, dtma::kThreads,
                                                    dtma::kSmemTotal) == cudaSuccess &&
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && per_sm > 0 && sms > 0)
    result = per_sm * sms;
  (void)cudaGetLastError();
  cached[dev] = result;
  return result > 0 ? result : 0;
}

cudaError_t launch_attn_decode_planned(const PlannedDecodeParams &p, bool bf16, cudaStream_t stream, int *launches) {
  *launches = 0;
  if (p.n_ctas <= 0) return cudaSuccess;
  const AttnGeom &g = p.g;
  CUtensorMap mk, mv, mk16, mv16;
  // (d, position, kv head, sequence), or (d, position in page, kv head, page) over a pool.  The
  // position extent is the longest sequence of the step: rows beyond it are never fetched.
  bool ok;
  if (p.pg.table) {
    const uint64_t ps = 1ull << p.pg.page_shift, np = static_cast<uint64_t>(p.pg.n_pages);
    ok = make_tensor_map_4d(&mk, bf16, p.k_cache, ps, g.n_kv_heads, np, g.c_pos, g.c_head, p.pg.page_stride, 64, 1) &&
         make_tensor_map_4d(&mv, bf16, p.v_cache, ps, g.n_kv_heads, np, g.c_pos, g.c_head, p.pg.page_stride, 64, 1) &&
         make_tensor_map_4d(&mk16, bf16, p.k_cache, ps, g.n_kv_heads, np, g.c_pos, g.c_head, p.pg.page_stride, 16, 1) &&
         make_tensor_map_4d(&mv16, bf16, p.v_cache, ps, g.n_kv_heads, np, g.c_pos, g.c_head, p.pg.page_stride, 16, 1);
  } else {
    const uint64_t n = static_cast<uint64_t>(p.max_total);
    ok = make_tensor_map_4d(&mk, bf16, p.k_cache, n, g.n_kv_heads, g.batch, g.c_pos, g.c_head, g.c_seq, 64, 1) &&
         make_tensor_map_4d(&mv, bf16, p.v_cache, n, g.n_kv_heads, g.batch, g.c_pos, g.c_head, g.c_seq, 64, 1) &&
         make_tensor_map_4d(&mk16, bf16, p.k_cache, n, g.n_kv_heads, g.batch, g.c_pos, g.c_head, g.c_seq, 16, 1) &&
         make_tensor_map_4d(&mv16, bf16, p.v_cache, n, g.n_kv_heads, g.batch, g.c_pos, g.c_head, g.c_seq, 16, 1);
  }
  if (!ok) return cudaErrorNotSupported;
  return bf16 ? launch_typed<__nv_bfloat16>(p, mk, mv, mk16, mv16, stream, launches)
              : launch_typed<__half>(p, mk, mv, mk16, mv16, stream, launches);
}

} // namespace b200attn
