// Causal prefill attention on the 5th-generation tensor cores (sm_100a):
// tcgen05.mma with accumulators in tensor memory (TMEM), operands staged in
// shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), online softmax
// in registers.
//
// One CTA = 256 query rows (two tiles A and B of 128) of one head of one
// sequence, walking the KV cache in tiles of 128 positions up to the causal
// diagonal.  Twelve warps in three groups of four:
//   warp 0        TMA producer (one elected lane): Q tiles once, then K and V
//                 tiles into two-stage rings; the loads of Q and of the first
//                 K / V tile leave before the set-up barrier of the CTA
//   warp 1        MMA issuer (one elected lane): S_X = Q_X.K^T (operands from
//                 shared memory) into TMEM, then O_X += P_X.V with P_X read from
//                 TMEM and V from shared memory (N-major operand); per KV tile
//                 it issues  P.V(A) Q.K(A,next)  P.V(B) Q.K(B,next), so that the
//                 tensor pipe works for one query tile while the other one's
//                 softmax runs; the first half of each P.V starts as soon as the
//                 first 64 positions of P are published
//   warps 2-3     idle (they only give their registers away)
//   warps 4-7     softmax of tile A, warps 8-11 softmax of tile B: one thread
//                 per query row (TMEM lane): tcgen05.ld of the S row, running
//                 max / sum in the log2 domain, P written back over S as packed
//                 16-bit pairs (tcgen05.st); O is only rescaled when the running
//                 max has grown by more than 2^8 since the last rescale;
//                 epilogue O / l -> swizzled staging tile in shared memory -> one TMA
//                 tensor store per tile (rows beyond m clipped by the tensor map)
// TMEM (512 columns): S_A | S_B | O_A | O_B, 128 fp32 columns each; P_X aliases
// the first 64 columns of S_X.
//
// Reference semantics: tests/flash_attn_test.cpp:106-192 (mask col > row+offset,
// scale 1/sqrt(D) folded into the exponent, O = softmax(S).V, out [m][H*D]).
//
// Every wait on an mbarrier is bounded: after about a second without progress
// the waiter raises an error flag that the host reads, and the CTA runs to its
// normal end (TMEM is freed) instead of spinning.
#include "kernels.h"
#include "common.cuh"
#include "tma.cuh"
#include "tc5.cuh"

#include <cuda.h>
#include <cstring>
#include <mutex>
#include <type_traits>

// K and V a chunk of (sequence, head) pairs may hold in L2 together (see the CTA order at the launch)
#ifndef PREFILL_CHUNK_BYTES
#define PREFILL_CHUNK_BYTES (40L << 20)
#endif

namespace b200attn {

namespace tc5 {

using namespace tma;

constexpr int kBM = 128;            // query rows per tile; two tiles per CTA
constexpr int kBN = 128;            // key positions per tile
constexpr int kThreads = 384;
constexpr int kStages = 2;
constexpr uint32_t kHalfTile = 128 * 128;        // bytes of a [128 rows][64 elem] swizzled half tile
constexpr uint32_t kTileBytes = 2 * kHalfTile;   // [128][128] 16-bit
constexpr uint32_t kSmemQ = 0;                   // Q_A, Q_B
constexpr uint32_t kSmemK = kSmemQ + 2 * kTileBytes;
constexpr uint32_t kSmemV = kSmemK + kStages * kTileBytes;
constexpr uint32_t kSmemStg = kSmemV + kStages * kTileBytes;   // output staging tile, used by tile A, then by tile B
constexpr uint32_t kSmemBar = kSmemStg + kTileBytes;
constexpr uint32_t kSmemTotal = kSmemBar + 256 + 1024; // barriers + slack for 1024-byte alignment
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256;       // S_X at kColS + 128 X, O_X at kColO + 128 X
constexpr float kRescaleThreshold = 8.0f;        // log2 domain

// barrier slots (8 bytes each) inside the barrier block; X = 0 (tile A) or 1 (tile B)
enum { BAR_Q = 0, BAR_KFULL = 1, BAR_KEMPTY = 3, BAR_VFULL = 5, BAR_VEMPTY = 7, BAR_SFULL = 9, BAR_PREADY = 11,
       BAR_ODONE = 13, BAR_PHALF = 15, BAR_QB = 17, BAR_STGWR = 18, BAR_STGFREE = 20, BAR_COUNT = 21 };

struct Params {
  void *out;
  int m, n, offset;
  int group;
  long out_seq, out_tok;
  float scale_log2;
  int *error_flag;
  // paged cache: page id of (sequence b, position pos) = page_table[b * table_stride + (pos >> page_shift)]
  const int32_t *page_table;
  int table_stride, page_shift;
  // CTA order (see the launch): chunk_groups (sequence, head) pairs per chunk, `pad` empty places at
  // the front of the first chunk, n_heads and a multiplier that divides by it
  int chunk_groups, pad, n_heads;
  uint32_t heads_mul;
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_k_tail,
                        const __grid_constant__ CUtensorMap map_v_tail,
                        const __grid_constant__ CUtensorMap map_o,
                        Params p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kSmemBar;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + kSmemBar + BAR_COUNT * 8);
  volatile uint32_t *abort_flag = tmem_slot + 1;
  auto bar = [&](int i) { return bar_base + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  // grid = ((sequence, head) pair within its chunk, row block longest first, chunk): CTAs start in that
  // order, so a chunk's longest row blocks all start before its shorter ones
  const int pair = static_cast<int>(blockIdx.z) * p.chunk_groups + static_cast<int>(blockIdx.x) - p.pad;
  if (pair < 0) return;                        // a padding place of the first chunk
  const int qb = gridDim.y - 1 - blockIdx.y;
  const int b = p.heads_mul ? static_cast<int>(__umulhi(static_cast<uint32_t>(pair), p.heads_mul)) : pair / p.n_heads;
  const int h = pair - b * p.n_heads;
  const int kvh = h / p.group;
  const int row0 = qb * 2 * kBM;                 // first row of tile A; tile B starts kBM later
  const bool has_b = row0 + kBM < p.m;
  // KV tiles each query tile needs (up to its causal diagonal / the end of the cache)
  const int nt_a = (min(p.n, p.offset + min(p.m, row0 + kBM)) + kBN - 1) / kBN;
  const int nt_b = has_b ? (min(p.n, p.offset + min(p.m, row0 + 2 * kBM)) + kBN - 1) / kBN : 0;
  const int nt = max(nt_a, nt_b);
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  constexpr uint32_t idesc_qk = instr_desc(fmt, 0), idesc_pv = instr_desc(fmt, 1);

  // K / V tile j of this CTA's KV head: coordinates (flat or paged) and the map to read it through.
  // Flat cache: (d, position, kv head, sequence); rows at and beyond n are outside the map and read
  // as zero.  Paged cache: (d, position in page, kv head, page); the page that holds position n - 1
  // is read through a second map that ends at that position, so that the unwritten rest of the page
  // reads as zero too.
  auto load_kv_tile = [&](int j, bool is_k) {
    const int s = j % kStages;
    int c1 = j * kBN, c3 = b;
    const CUtensorMap *mp = is_k ? &map_k : &map_v;
    if (p.page_table) {
      const int pi = c1 >> p.page_shift;
      c3 = p.page_table[static_cast<long>(b) * p.table_stride + pi];
      c1 &= (1 << p.page_shift) - 1;
      if (pi == ((p.n - 1) >> p.page_shift)) mp = is_k ? &map_k_tail : &map_v_tail;
    }
    const uint32_t full = bar((is_k ? BAR_KFULL : BAR_VFULL) + s);
    const uint32_t dst = smem_base + (is_k ? kSmemK : kSmemV) + s * kTileBytes;
    mbar_expect_tx(full, kTileBytes);
    tma_load_4d(dst, mp, full, 0, c1, kvh, c3);
    tma_load_4d(dst + kHalfTile, mp, full, 64, c1, kvh, c3);
  };
  auto load_q_tile = [&](int x) {
    const uint32_t qbar = bar(x ? BAR_QB : BAR_Q);
    mbar_expect_tx(qbar, kTileBytes);
    tma_load_4d(smem_base + kSmemQ + x * kTileBytes, &map_q, qbar, 0, h, row0 + x * kBM, b);
    tma_load_4d(smem_base + kSmemQ + x * kTileBytes + kHalfTile, &map_q, qbar, 64, h, row0 + x * kBM, b);
  };
  auto issue_first_loads = [&]() {
    load_q_tile(0);
    if (nt > 0) load_kv_tile(0, true);
    if (nt > 0) load_kv_tile(0, false);
    if (has_b) load_q_tile(1);
  };

  if (threadIdx.x == 0) {
    mbar_init(bar(BAR_Q), 1);
    mbar_init(bar(BAR_QB), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(BAR_KFULL + s), 1);
      mbar_init(bar(BAR_KEMPTY + s), 1);
      mbar_init(bar(BAR_VFULL + s), 1);
      mbar_init(bar(BAR_VEMPTY + s), 1);
      mbar_init(bar(BAR_SFULL + s), 1);
      mbar_init(bar(BAR_PREADY + s), 128);
      mbar_init(bar(BAR_ODONE + s), 1);
      mbar_init(bar(BAR_PHALF + s), 128);
      mbar_init(bar(BAR_STGWR + s), 128);
    }
    mbar_init(bar(BAR_STGFREE), 1);
    *abort_flag = 0;
    fence_barrier_init();
    // The first loads leave before TMEM is allocated and the other warps are released, so
    // that their latency (about 2500 cycles from a cold start) overlaps the set-up: Q_A and
    // the first K tile (what the first MMAs need), then the first V tile, then Q_B.
    issue_first_loads();
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(const_cast<uint32_t *>(tmem_slot))),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < 4) {
    reg_dec<64>();
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------- TMA producer
      for (int j = 1; j < nt; ++j) {   // tile 0 left before the set-up barrier
        const int s = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        if (!mbar_wait(bar(BAR_KEMPTY + s), ph ^ 1, abort_flag, p.error_flag, 1)) break;
        load_kv_tile(j, true);
        if (!mbar_wait(bar(BAR_VEMPTY + s), ph ^ 1, abort_flag, p.error_flag, 2)) break;
        load_kv_tile(j, false);
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------- MMA issuer
      bool ok = mbar_wait(bar(BAR_Q), 0, abort_flag, p.error_flag, 3);
      // Descriptors are built once; per instruction only a constant is added to the
      // start-address field.  The issuing thread's own instruction count per MMA must
      // stay well under the 64 cycles a 128x128x16 MMA takes, or the tensor pipe starves.
      const uint32_t dq0 = smem_desc_lo(smem_base + kSmemQ, 16);
      const uint32_t dk0 = smem_desc_lo(smem_base + kSmemK, 16);
      const uint32_t dv0 = smem_desc_lo(smem_base + kSmemV, kHalfTile);
      constexpr uint32_t kTileStep = kTileBytes >> 4; // one tile further, in descriptor address units
      // S_X = Q_X . K[j]^T ; `last` marks the last reader of K[j], which frees the stage
      auto issue_qk = [&](int x, int j, bool last) -> bool {
        const int s = j % kStages;
        if (!mbar_wait(bar(BAR_KFULL + s), (j / kStages) & 1, abort_flag, p.error_flag, 4)) return false;
        tc_fence_after();
        const uint32_t d = tmem + kColS + 128 * x;
        const uint32_t dq = dq0 + x * kTileStep, dk = dk0 + s * kTileStep;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          constexpr uint32_t kHalfStep = kHalfTile >> 4;
          const uint32_t ko = (k >> 2) * kHalfStep + (k & 3) * 2; // 16 elements = 32 bytes per step
          tc_mma_ss(d, dq + ko, dk + ko, kDescHi, idesc_qk, k > 0);
        }
        if (last) tc_commit(bar(BAR_KEMPTY + s));
        tc_commit(bar(BAR_SFULL + x));
        return true;
      };
      // O_X += P_X . V[j] ; `last` marks the last reader of V[j]
      auto issue_pv = [&](int x, int j, bool last) -> bool {
        const int s = j % kStages;
        // The softmax warps publish the first 64 positions of P before they start on the
        // other 64, so that half of this product overlaps their remaining exponentials.
        if (!mbar_wait(bar(BAR_PHALF + x), j & 1, abort_flag, p.error_flag, 10)) return false;
        if (!mbar_wait(bar(BAR_VFULL + s), (j / kStages) & 1, abort_flag, p.error_flag, 6)) return false;
        tc_fence_after();
        const uint32_t pcol = tmem + kColS + 128 * x, ocol = tmem + kColO + 128 * x;
        const uint32_t dv = dv0 + s * kTileStep;
        const uint32_t acc0 = j > 0 ? 1u : 0u;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // 16 positions per step: 8 TMEM columns of packed P, 16 rows (2048 B) of V
          tc_mma_ts(ocol, pcol + 8 * k, dv + k * (2048 >> 4), kDescHi, idesc_pv, k > 0 ? 1u : acc0);
        }
        if (!mbar_wait(bar(BAR_PREADY + x), j & 1, abort_flag, p.error_flag, 5)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 4; k < 8; ++k) tc_mma_ts(ocol, pcol + 8 * k, dv + k * (2048 >> 4), kDescHi, idesc_pv, 1u);
        if (last) tc_commit(bar(BAR_VEMPTY + s));
        tc_commit(bar(BAR_ODONE + x));
        return true;
      };
      // tile B (when present) reads every KV tile that A reads, and reads it after A
      if (ok && nt_a > 0) ok = issue_qk(0, 0, !has_b);
      if (ok && has_b) {
        ok = mbar_wait(bar(BAR_QB), 0, abort_flag, p.error_flag, 11);
        if (ok) ok = issue_qk(1, 0, true);
      }
      for (int j = 0; ok && j < nt; ++j) {
        if (j < nt_a) {
          ok = issue_pv(0, j, !has_b);
          if (ok && j + 1 < nt_a) ok = issue_qk(0, j + 1, !has_b);
        }
        if (ok && has_b) {
          ok = issue_pv(1, j, true);
          if (ok && j + 1 < nt_b) ok = issue_qk(1, j + 1, true);
        }
      }
    }
  } else {
    reg_inc<216>();
    // ------------------------------------------------------------ softmax + epilogue of tile X
    const int x = (warp >> 2) - 1;               // 0: tile A (warps 4-7), 1: tile B (warps 8-11)
    const int quad = warp & 3;                   // TMEM lane quadrant this warp may touch
    const int trow0 = row0 + x * kBM;
    const int row = trow0 + quad * 32 + lane;    // query token index within the call
    const int ntx = x == 0 ? nt_a : nt_b;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t scol = tmem + lane_addr + kColS + 128 * x;
    const uint32_t ocol = tmem + lane_addr + kColO + 128 * x;
    const int vis_end = min(p.n, p.offset + row + 1); // columns < vis_end are visible to this row
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < ntx; ++j) {
      if (!__all_sync(0xffffffffu, mbar_wait(bar(BAR_SFULL + x), j & 1, abort_flag, p.error_flag, 7))) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t su[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc_ld32(scol + 32 * c, su + 32 * c);
      tc_wait_ld();
      const int col0 = j * kBN;
      // only the last tiles of a row block cross the diagonal or the end of the cache
      if (col0 + kBN > min(p.n, p.offset + trow0 + 1)) {
#pragma unroll
        for (int c = 0; c < 128; ++c)
          if (col0 + c >= vis_end) su[c] = 0xff800000u; // -inf
      }
      // row max with eight independent chains of three-input maxima
      float mxa[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mxa[i] = fmaxf(__uint_as_float(su[i]), __uint_as_float(su[8 + i]));
#pragma unroll
      for (int c = 16; c < 128; c += 16) {
#pragma unroll
        for (int i = 0; i < 8; ++i) mxa[i] = max3(mxa[i], __uint_as_float(su[c + i]), __uint_as_float(su[c + 8 + i]));
      }
      float mx = fmaxf(max3(mxa[0], mxa[1], mxa[2]), fmaxf(max3(mxa[3], mxa[4], mxa[5]), fmaxf(mxa[6], mxa[7])));
      mx *= p.scale_log2;
      // lazy rescale: keep the old reference max unless the new one is much larger
      const bool grow = mx > m_ref + kRescaleThreshold;
      if (__any_sync(0xffffffffu, grow) && j > 0) {
        // O must hold every P.V issued so far before it is rescaled
        if (!__all_sync(0xffffffffu, mbar_wait(bar(BAR_ODONE + x), (j - 1) & 1, abort_flag, p.error_flag, 8))) {
          ok = false;
          break;
        }
        tc_fence_after();
        const float f = grow ? ex2(m_ref - mx) : 1.f;
        l *= f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tc_ld32(ocol + 32 * c, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
          tc_st32(ocol + 32 * c, o);
        }
        tc_wait_st();
      }
      if (grow) m_ref = mx;
      // P = 2^(s*scale - m_ref), packed pairs written back to TMEM half a tile at a time
      uint32_t pk[64];
      uint64_t sums[2] = {0ull, 0ull};            // two fp32x2 accumulators
      const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), neg_m2 = pack2(-m_ref, -m_ref);
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        const uint64_t x2 = fma2(pack2(__uint_as_float(su[2 * c]), __uint_as_float(su[2 * c + 1])), scale2, neg_m2);
        float x0, x1;
        unpack2(x2, x0, x1);
        const float p0 = ex2(x0), p1 = ex2(x1);
        sums[c & 1] = add2(sums[c & 1], pack2(p0, p1));
        pk[c] = Elem<T>::pack(p0, p1);
        if (c == 31) {
          // first 64 positions of P: the MMA warp may start P.V on them
          tc_st32(scol, pk);
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(bar(BAR_PHALF + x));
        }
      }
      {
        float a0, a1, a2, a3;
        unpack2(sums[0], a0, a1);
        unpack2(sums[1], a2, a3);
        l += (a0 + a1) + (a2 + a3);
      }
      tc_st32(scol + 32, pk + 32);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(bar(BAR_PREADY + x));
    }
    if (ok && ntx > 0)
      ok = __all_sync(0xffffffffu, mbar_wait(bar(BAR_ODONE + x), (ntx - 1) & 1, abort_flag, p.error_flag, 9));
    if (ok && ntx > 0) {
      // O / l leaves through a swizzled [128][128] staging tile and one TMA tensor store (two boxes; rows
      // beyond m clipped by the tensor map) instead of 16-byte stores of 32 different rows per warp
      // instruction.  Tile A always finishes first (it has no more KV tiles than tile B); tile B waits until
      // A's store has read the tile.
      tc_fence_after();
      const bool elected = quad == 0 && lane == 0;
      if (x == 1 && !__all_sync(0xffffffffu, mbar_wait(bar(BAR_STGFREE), 0, abort_flag, p.error_flag, 13))) ok = false;
      if (ok) {
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int trow = quad * 32 + lane;
        const uint32_t stg_row = smem_base + kSmemStg + trow * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tc_ld32(ocol + 32 * c, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t w0 = Elem<T>::pack(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
            uint32_t w1 = Elem<T>::pack(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
            uint32_t w2 = Elem<T>::pack(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
            uint32_t w3 = Elem<T>::pack(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
            // element d = 32 c + 8 i: half tile c / 2, 16-byte chunk (c & 1) * 4 + i, swizzled by the row
            const uint32_t chunk = static_cast<uint32_t>((c & 1) * 4 + i) ^ static_cast<uint32_t>(trow & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stg_row + (c >> 1) * kHalfTile + (chunk << 4)),
                         "r"(w0), "r"(w1), "r"(w2), "r"(w3)
                         : "memory");
          }
        }
        fence_proxy_async_smem();   // the tensor store reads what this thread wrote
        mbar_arrive(bar(BAR_STGWR + x));
        if (elected && mbar_wait(bar(BAR_STGWR + x), 0, abort_flag, p.error_flag, 14)) {
          asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(&map_o),
                       "r"(smem_base + kSmemStg), "r"(0), "r"(h), "r"(trow0), "r"(b)
                       : "memory");
          asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(&map_o),
                       "r"(smem_base + kSmemStg + kHalfTile), "r"(64), "r"(h), "r"(trow0), "r"(b)
                       : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          if (x == 0) mbar_arrive(bar(BAR_STGFREE));
          asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---------------------------------------------------------------------------
// host side: tensor maps
// ---------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// device word the kernels raise when a bounded wait gives up; one per device
int *error_word() {
  static std::mutex mu;
  static int *words[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  if (!words[dev]) {
    // mapped pinned host memory: the kernel writes it, the host reads it without a copy
    int *h = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void **>(&h), sizeof(int), cudaHostAllocMapped) != cudaSuccess) return nullptr;
    *h = 0;
    words[dev] = h;
  }
  return words[dev];
}

// 4-D map over (d, dim1, dim2, dim3) with a box of 64 x box1 x box2 x 1 elements
bool make_tensor_map_4d_impl(CUtensorMap *map, bool bf16, const void *base, uint64_t n1, uint64_t n2, uint64_t n3, long s1, long s2,
              long s3, uint32_t box1, uint32_t box2) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  auto fix = [](long s) { return static_cast<cuuint64_t>(s > 0 ? s : 128) * 2; }; // bytes; unit extents may carry stride 0
  cuuint64_t dims[4] = {128, n1, n2, n3};
  cuuint64_t strides[3] = {fix(s1), fix(s2), fix(s3)};
  cuuint32_t box[4] = {64, box1, box2, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < 3; ++i)
    if (strides[i] % 16 || strides[i] >= (1ull << 40)) return false;
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                  const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

} // namespace tc5

bool make_tensor_map_4d(CUtensorMap *map, bool bf16, const void *base, uint64_t n1, uint64_t n2, uint64_t n3, long s1,
                        long s2, long s3, uint32_t box1, uint32_t box2) {
  // the encoding depends on nothing but these arguments: keep the most recent ones per thread
  constexpr int kCached = 32;
  struct Entry {
    TensorMapKey key;
    CUtensorMap map;
    bool used;
  };
  thread_local Entry cache[kCached] = {};
  thread_local int next = 0;
  TensorMapKey key{};
  key.base = base, key.n1 = n1, key.n2 = n2, key.n3 = n3, key.s1 = s1, key.s2 = s2, key.s3 = s3;
  key.box1 = box1, key.box2 = box2, key.bf16 = bf16 ? 1u : 0u;
  for (int i = 0; i < kCached; ++i) {
    if (cache[i].used && memcmp(&cache[i].key, &key, sizeof key) == 0) {
      *map = cache[i].map;
      return true;
    }
  }
  if (!tc5::make_tensor_map_4d_impl(map, bf16, base, n1, n2, n3, s1, s2, s3, box1, box2)) return false;
  cache[next].key = key;
  cache[next].map = *map;
  cache[next].used = true;
  next = (next + 1) % kCached;
  return true;
}

int *kernel_error_word_dev() {
  int *w = tc5::error_word();
  int *dev = nullptr;
  if (!w || cudaHostGetDevicePointer(reinterpret_cast<void **>(&dev), w, 0) != cudaSuccess) return nullptr;
  return dev;
}

void attn_clear_error_status() {
  int *w = tc5::error_word();
  if (w) *reinterpret_cast<volatile int *>(w) = 0;
}

int attn_tc5_error_status() {
  int *w = tc5::error_word();
  return w ? *reinterpret_cast<volatile int *>(w) : 0;
}

cudaError_t launch_attn_prefill_tc5(const PrefillParams &p, bool bf16, cudaStream_t stream) {
  using namespace tc5;
  const AttnGeom &g = p.g;
  CUtensorMap mq, mk, mv, mk_tail, mv_tail;
  // q: (d, head, token, seq); k/v: (d, pos, kv_head, seq), or (d, pos in page, kv_head, page) over a pool
  if (!make_tensor_map_4d(&mq, bf16, p.q, g.n_heads, p.m, g.batch, kHeadDim, g.q_tok, g.q_seq, 1, kBM)) return cudaErrorNotSupported;
  CUtensorMap mo;   // out: (d, head, token, seq), like q
  if (!make_tensor_map_4d(&mo, bf16, p.out, g.n_heads, p.m, g.batch, kHeadDim, g.out_tok, g.out_seq, 1, kBM)) return cudaErrorNotSupported;
  if (p.pg.table) {
    const int page_size = 1 << p.pg.page_shift;
    if (page_size < kBN) return cudaErrorNotSupported; // a K / V tile of 128 positions must lie inside one page
    const uint64_t n_pages = static_cast<uint64_t>(p.pg.n_pages);
    const uint64_t tail = static_cast<uint64_t>((p.n - 1) & (page_size - 1)) + 1;
    if (!make_tensor_map_4d(&mk, bf16, p.k_cache, page_size, g.n_kv_heads, n_pages, g.c_pos, g.c_head, p.pg.page_stride, kBN, 1) ||
        !make_tensor_map_4d(&mv, bf16, p.v_cache, page_size, g.n_kv_heads, n_pages, g.c_pos, g.c_head, p.pg.page_stride, kBN, 1) ||
        !make_tensor_map_4d(&mk_tail, bf16, p.k_cache, tail, g.n_kv_heads, n_pages, g.c_pos, g.c_head, p.pg.page_stride, kBN, 1) ||
        !make_tensor_map_4d(&mv_tail, bf16, p.v_cache, tail, g.n_kv_heads, n_pages, g.c_pos, g.c_head, p.pg.page_stride, kBN, 1))
      return cudaErrorNotSupported;
  } else {
    if (!make_tensor_map_4d(&mk, bf16, p.k_cache, p.n, g.n_kv_heads, g.batch, g.c_pos, g.c_head, g.c_seq, kBN, 1) ||
        !make_tensor_map_4d(&mv, bf16, p.v_cache, p.n, g.n_kv_heads, g.batch, g.c_pos, g.c_head, g.c_seq, kBN, 1))
      return cudaErrorNotSupported;
    mk_tail = mk;
    mv_tail = mv;
  }
  int *err = error_word();
  if (!err) return cudaErrorNotSupported;
  int *err_dev = nullptr;
  if (cudaHostGetDevicePointer(reinterpret_cast<void **>(&err_dev), err, 0) != cudaSuccess) return cudaErrorNotSupported;
  Params kp{};
  kp.out = p.out;
  kp.m = p.m;
  kp.n = p.n;
  kp.offset = p.offset;
  kp.group = g.group;
  kp.out_seq = g.out_seq;
  kp.out_tok = g.out_tok;
  kp.scale_log2 = p.scale_log2;
  kp.error_flag = err_dev;
  kp.page_table = p.pg.table;
  kp.table_stride = p.pg.table_stride;
  kp.page_shift = p.pg.page_shift;
  // CTA order.  The row blocks of a (sequence, head) pair cost 1, 2, ... , nqb units (causal), and the
  // hardware starts CTAs in grid order on whichever SM frees up.  Pairs are taken in chunks whose K and V
  // fit in L2 together; inside a chunk the longest row block of every pair comes first, then the next
  // longest, so that the pairs still find their K/V in L2 and the last CTAs to start are the shortest
  // (the partial chunk, if any, goes first).  With pair after pair in full the last pair's longest block
  // starts near the end and runs alone: at 2 waves of CTAs that is a third of the kernel's time.
  const int nqb = (p.m + 2 * kBM - 1) / (2 * kBM);
  const long pairs = static_cast<long>(g.n_heads) * g.batch;
  const long kv_bytes_per_pair = 2L * p.n * kHeadDim * 2 / g.group;     // K and V, shared by a group's heads
  long chunk = (p.l2_window > 0 ? p.l2_window : PREFILL_CHUNK_BYTES) / (kv_bytes_per_pair > 0 ? kv_bytes_per_pair : 1);
  chunk = chunk < 1 ? 1 : chunk > pairs ? pairs : chunk;
  if ((pairs + chunk - 1) / chunk > 65535) chunk = (pairs + 65534) / 65535;
  const long n_chunks = (pairs + chunk - 1) / chunk;
  if (nqb > 65535 || chunk > 0x7fffffffL) return cudaErrorNotSupported;
  kp.chunk_groups = static_cast<int>(chunk);
  kp.pad = static_cast<int>(n_chunks * chunk - pairs);
  kp.n_heads = g.n_heads;
  // floor(pair / n_heads) = (pair * heads_mul) >> 32, exact while pair < 2^32 / n_heads
  kp.heads_mul = (pairs < (1L << 20) && g.n_heads <= 1024) ? static_cast<uint32_t>((1ULL << 32) / g.n_heads + 1) : 0u;
  if (g.n_heads == 1) kp.heads_mul = 0u;    // 2^32 + 1 does not fit; the plain division serves
  dim3 grid(static_cast<unsigned>(chunk), nqb, static_cast<unsigned>(n_chunks));
  // the shared-memory opt-in is a property of (function, device): set it on the first launch per device
  static bool attr_set[2][64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const bool known = dev >= 0 && dev < 64;
  if (!known || !attr_set[bf16 ? 1 : 0][dev]) {
    e = bf16 ? cudaFuncSetAttribute(attn_prefill_tc5_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal)
             : cudaFuncSetAttribute(attn_prefill_tc5_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
    if (e != cudaSuccess) return e;
    if (known) attr_set[bf16 ? 1 : 0][dev] = true;
  }
  if (bf16)
    attn_prefill_tc5_kernel<__nv_bfloat16><<<grid, kThreads, kSmemTotal, stream>>>(mq, mk, mv, mk_tail, mv_tail, mo, kp);
  else
    attn_prefill_tc5_kernel<__half><<<grid, kThreads, kSmemTotal, stream>>>(mq, mk, mv, mk_tail, mv_tail, mo, kp);
  return cudaGetLastError();
}

} // namespace b200attn
