// Causal prefill attention on the 5th-generation tensor cores (sm_100a),
// persistent form: one CTA per SM walks a queue of work items.
//
// A work item = 256 query rows (two tiles A and B of 128) of one head of one
// sequence; items are numbered so that the eight (or however many) row blocks of
// one (sequence, head) follow each other, longest first, and are handed out in
// that order: CTA c starts with item c and takes its next ones from a counter in
// global memory, so that at any time the CTAs in flight work on neighbouring
// (sequence, head) pairs and share their K / V in L2.
//
// Inside an item the kernel is the non-persistent one (attn_tc5.cu): TMA producer
// lane (warp 0), MMA-issuing lane (warp 1; tcgen05.mma, accumulators in tensor
// memory), two groups of four softmax warps (4-7 tile A, 8-11 tile B) with one
// thread per query row; one lane of warp 3 issues the tensor stores of both
// tiles (warp 2 only gives its registers away).  What the persistent form adds is
// the overlap ACROSS items:
//   * tensor memory, barriers and tensor maps are set up once per CTA;
//   * the producer runs ahead: the next item's Q tiles are loaded as soon as the
//     last Q.K^T of the current item has read the old ones, and K / V tiles of the
//     next item follow the last ones of the current item through the same rings;
//   * the MMA lane issues the next item's first Q_A.K^T and Q_B.K^T right behind
//     the current item's last P.V, so that S_A and S_B are there when the softmax
//     warps come back from their epilogue; per item its loop is the one of the
//     non-persistent kernel (every item starts on an even slot of the K / V ring,
//     an odd tile count is padded with an empty slot, so that tile j of an item
//     always lives in stage j & 1);
//   * the epilogue leaves through shared memory: O / l is written as a swizzled
//     [128][128] 16-bit tile and stored with one TMA tensor store (two boxes),
//     rows beyond m clipped by the tensor map, instead of 16-byte stores of 32
//     different rows per warp instruction.
//
// Status: same bits as the non-persistent kernel on every case tried, but slower
// (cfg3-shaped layer 0.46 against 0.39 ms, long rows 2.69 against 2.21 ms), and
// therefore opt-in.  Time stamps taken inside both kernels show where: the softmax
// warps are as fast here (1690 against 1800 cycles per tile), but the products take
// longer to come back: eight Q.K^T MMAs and their commits occupy the issuing lane
// for 720-760 cycles against 540, so the lane, not the softmax, paces the kernel (a
// pair of tiles every 3900 cycles against 3290).  The cause was not found.  Ruled
// out by variant builds: register budgets, the item ring and counter, the staging
// tile and store lane, the grid shape, the size and layout of shared memory,
// polling style, the structure of the issuing loop (the walk of the non-persistent
// kernel, a whole warp walking it, one flat loop over ring tiles, two issuing
// lanes) and whether tile counts and ring stages are known to be warp-uniform.
// Hot code size matters (two alternating copies of the softmax loop cost the
// non-persistent kernel 9 % on short rows and 2 % on long ones), but not enough.
// The issuing lane has no slack in either kernel: issuing the MMAs of a product
// from a rolled loop (three more instructions per MMA) costs 20-25 %.  Unrolling
// this kernel's tile loop by two, so that every ring stage is a literal as the
// compiler makes it in the non-persistent kernel, gains 3-10 % on long rows and
// loses 5 % on short ones.  The non-persistent kernel also starts its CTAs in an
// order that keeps its tail short (chunks of (sequence, head) pairs, longest row
// blocks first), which this kernel's item numbering does not follow.
//
// The counter: two words {next item, CTAs done} per launch, zero before the
// launch; the last CTA to finish zeroes them again.  The host hands each stream
// its own small set of counter pairs (launches on one stream run one after the
// other), see launch_attn_prefill_tc5p; the 2 KB that hold them are the one
// allocation this library makes inside an operator call (first use per device).
//
// Reference semantics: tests/flash_attn_test.cpp:106-192 (mask col > row+offset,
// scale 1/sqrt(D) folded into the exponent, O = softmax(S).V, out [m][H*D]).
//
// Every wait on an mbarrier is bounded: after about a second without progress the
// waiter raises an error flag that the host reads and every role leaves its loop;
// the CTA runs to its normal end (tensor memory is freed).  No group-wide bar.sync
// is used inside the loops, so a role that gave up cannot strand the others.
#include "kernels.h"
#include "common.cuh"
#include "tma.cuh"
#include "tc5.cuh"

#include <cuda.h>
#include <climits>
#include <mutex>
#include <type_traits>
#include <vector>

namespace b200attn {

namespace tc5p {

using namespace tma;
using namespace tc5;

constexpr int kBM = 128;            // query rows per tile; two tiles per item
constexpr int kBN = 128;            // key positions per tile
constexpr int kThreads = 384;
constexpr int kStages = 2;
constexpr int kItemRing = 4;
constexpr uint32_t kHalfTile = 128 * 128;        // bytes of a [128 rows][64 elem] swizzled half tile
constexpr uint32_t kTileBytes = 2 * kHalfTile;   // [128][128] 16-bit
constexpr uint32_t kSmemQ = 0;                   // Q_A, Q_B
constexpr uint32_t kSmemK = kSmemQ + 2 * kTileBytes;
constexpr uint32_t kSmemV = kSmemK + kStages * kTileBytes;
constexpr uint32_t kSmemStg = kSmemV + kStages * kTileBytes;   // output staging tile, shared by both groups
constexpr uint32_t kSmemBar = kSmemStg + kTileBytes;
constexpr uint32_t kSmemTotal = kSmemBar + 512;
static_assert(kSmemTotal <= 232448, "beyond the 227 KB a CTA can opt in to");
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 256;       // S_X at kColS + 128 X, O_X at kColO + 128 X
constexpr float kRescaleThreshold = 8.0f;        // log2 domain
// Register budgets after setmaxnreg: warps 0-3 give registers away, warps 4-11 take them.  The CTA
// is launched with kRegsLaunch per thread (what __launch_bounds__(384, 1) makes the compiler use);
// setmaxnreg.inc waits until the registers are there, so the two budgets must fit that allocation.
constexpr int kRegsLaunch = 168, kRegsControl = 72, kRegsSoftmax = 216;
static_assert(128 * kRegsControl + 256 * kRegsSoftmax <= kThreads * kRegsLaunch, "setmaxnreg.inc would never return");

// barrier slots (8 bytes each); pairs are indexed by X = 0 (tile A) or 1 (tile B), or by ring stage
enum {
  BAR_QFULL = 0, BAR_QEMPTY = 2, BAR_KFULL = 4, BAR_KEMPTY = 6, BAR_VFULL = 8, BAR_VEMPTY = 10, BAR_SFULL = 12,
  BAR_PHALF = 14, BAR_PREADY = 16, BAR_ODONE = 18, BAR_STGRDY = 20, BAR_STGWR = 22, BAR_STGDONE = 24, BAR_STGFREE = 26,
  BAR_ITEMFULL = 27, BAR_ITEMEMPTY = BAR_ITEMFULL + kItemRing, BAR_COUNT = BAR_ITEMEMPTY + kItemRing
};
static_assert(BAR_COUNT * 8 + 16 * 4 <= 512, "barrier block and the words behind it");

struct Params {
  int m, n, offset;
  int group, n_heads;
  int nqb, n_items;              // row blocks of 256 per (sequence, head); items in all
  float scale_log2;
  int *error_flag;
  unsigned int *ticket;          // {next item beyond the first round, CTAs done}
  // paged cache: page id of (sequence b, position pos) = page_table[b * table_stride + (pos >> page_shift)]
  const int32_t *page_table;
  int table_stride, page_shift;
};

struct Item {
  int b, h, kvh, row0, nt_a, nt_b, nt;
  bool has_b, valid;
};

// A value that is the same in every active lane, handed to the compiler as such: the result of a
// warp-wide reduction lives in a uniform register.  The MMA and TMA instructions take their
// descriptors, addresses and coordinates from uniform registers, and loop counters, ring stages and
// barrier parities stay on the uniform datapath only if what they are derived from is known to be
// uniform -- which the compiler cannot see for a number read from shared memory or produced by an
// integer division.  (It is not enough here: the MMA-issuing lane of this kernel still needs 720-760
// cycles per 8 MMAs where the tensor pipe takes 512; see the status note at the top of the file.)
__device__ __forceinline__ int uniform(int v) { return __reduce_max_sync(__activemask(), v); }
// The same for a warp that runs converged: a broadcast from lane 0, the idiom compilers recognise.
__device__ __forceinline__ int uniform_warp(int v) { return __shfl_sync(0xffffffffu, v, 0); }

template <bool kWholeWarp = false>
__device__ __forceinline__ Item decode_item(const Params &p, int item) {
  auto u = [](int v) { return kWholeWarp ? uniform_warp(v) : uniform(v); };
  Item it;
  it.valid = item < p.n_items;
  const int qi = item % p.nqb, bh = item / p.nqb;
  it.h = u(bh % p.n_heads);
  it.b = u(bh / p.n_heads);
  it.kvh = u(it.h / p.group);
  it.row0 = u((p.nqb - 1 - qi) * 2 * kBM);      // longest row block of a (sequence, head) first
  it.has_b = it.row0 + kBM < p.m;
  // KV tiles each query tile needs (up to its causal diagonal / the end of the cache)
  it.nt_a = (min(p.n, p.offset + min(p.m, it.row0 + kBM)) + kBN - 1) / kBN;
  it.nt_b = it.has_b ? (min(p.n, p.offset + min(p.m, it.row0 + 2 * kBM)) + kBN - 1) / kBN : 0;
  it.nt = max(it.nt_a, it.nt_b);
  return it;
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map), "r"(src),
               "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint4 &v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc5p_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_k_tail,
                         const __grid_constant__ CUtensorMap map_v_tail, const __grid_constant__ CUtensorMap map_o,
                         Params p) {
  const unsigned kFirstItem = blockIdx.x, kGridSize = gridDim.x;
  extern __shared__ __align__(1024) unsigned char smem_gen[];
  const uint32_t smem_base = smem_u32(smem_gen);
  if (smem_base & 1023u) {       // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) *reinterpret_cast<volatile int *>(p.error_flag) = 31;
    return;
  }
  const uint32_t bar_base = smem_base + kSmemBar;
  volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + kSmemBar + BAR_COUNT * 8);
  volatile uint32_t *abort_flag = tmem_slot + 1;
  volatile int *item_ring = reinterpret_cast<volatile int *>(tmem_slot + 2);   // kItemRing entries
  uint32_t *stg_seq = const_cast<uint32_t *>(tmem_slot + 2 + kItemRing);       // users of the staging tile so far
  volatile int *stg_coord = reinterpret_cast<volatile int *>(tmem_slot + 8);   // per group: head, first row, sequence, stop
  auto bar = [&](int i) { return bar_base + 8u * i; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
    prefetch_tensormap(&map_o);
  }
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  constexpr uint32_t idesc_qk = instr_desc(fmt, 0), idesc_pv = instr_desc(fmt, 1);

  // K / V tile j of an item, the g-th tile this CTA streams: coordinates (flat or paged) and the map
  // to read it through.  Flat cache: (d, position, kv head, sequence); rows at and beyond n are
  // outside the map and read as zero.  Paged cache: (d, position in page, kv head, page); the page
  // that holds position n - 1 is read through a second map that ends at that position, so that the
  // unwritten rest of the page reads as zero too.
  auto load_kv_tile = [&](const Item &it, int j, uint32_t g, bool is_k) {
    const int s = g % kStages;
    int c1 = j * kBN, c3 = it.b;
    const CUtensorMap *mp = is_k ? &map_k : &map_v;
    if (p.page_table) {
      const int pi = c1 >> p.page_shift;
      c3 = p.page_table[static_cast<long>(it.b) * p.table_stride + pi];
      c1 &= (1 << p.page_shift) - 1;
      if (pi == ((p.n - 1) >> p.page_shift)) mp = is_k ? &map_k_tail : &map_v_tail;
    }
    const uint32_t full = bar((is_k ? BAR_KFULL : BAR_VFULL) + s);
    const uint32_t dst = smem_base + (is_k ? kSmemK : kSmemV) + s * kTileBytes;
    mbar_expect_tx(full, kTileBytes);
    tma_load_4d(dst, mp, full, 0, c1, it.kvh, c3);
    tma_load_4d(dst + kHalfTile, mp, full, 64, c1, it.kvh, c3);
  };
  auto load_q_tile = [&](const Item &it, int x) {
    const uint32_t qbar = bar(BAR_QFULL + x);
    mbar_expect_tx(qbar, kTileBytes);
    tma_load_4d(smem_base + kSmemQ + x * kTileBytes, &map_q, qbar, 0, it.h, it.row0 + x * kBM, it.b);
    tma_load_4d(smem_base + kSmemQ + x * kTileBytes + kHalfTile, &map_q, qbar, 64, it.h, it.row0 + x * kBM, it.b);
  };

  if (threadIdx.x == 0) {
    for (int x = 0; x < 2; ++x) {
      mbar_init(bar(BAR_QFULL + x), 1);
      mbar_init(bar(BAR_QEMPTY + x), 1);
      mbar_init(bar(BAR_KFULL + x), 1);
      mbar_init(bar(BAR_KEMPTY + x), 1);
      mbar_init(bar(BAR_VFULL + x), 1);
      mbar_init(bar(BAR_VEMPTY + x), 1);
      mbar_init(bar(BAR_SFULL + x), 1);
      mbar_init(bar(BAR_PHALF + x), 128);
      mbar_init(bar(BAR_PREADY + x), 128);
      mbar_init(bar(BAR_ODONE + x), 1);
      mbar_init(bar(BAR_STGRDY + x), 1);
      mbar_init(bar(BAR_STGWR + x), 128);
      mbar_init(bar(BAR_STGDONE + x), 1);
    }
    mbar_init(bar(BAR_STGFREE), 1);
    for (int i = 0; i < kItemRing; ++i) {
      mbar_init(bar(BAR_ITEMFULL + i), 1);
      mbar_init(bar(BAR_ITEMEMPTY + i), 9);     // the MMA lane and one lane of each of the eight softmax warps
    }
    *abort_flag = 0;
    *stg_seq = 0;
    stg_coord[3] = 0;
    stg_coord[7] = 0;
    fence_barrier_init();
    // The first item's first loads leave before tensor memory is allocated and the other warps are
    // released, so that their latency overlaps the set-up: Q_A and the first K tile (what the first
    // MMAs need), then the first V tile, then Q_B.
    const Item first = decode_item(p, kFirstItem);   // the grid never exceeds the item count
    load_q_tile(first, 0);
    load_kv_tile(first, 0, 0, true);
    load_kv_tile(first, 0, 0, false);
    if (first.has_b) load_q_tile(first, 1);
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

  // Entry e >= 1 of this CTA's item sequence, read from the ring the producer fills (entry 0 is
  // blockIdx.x).  One lane per consumer warp calls this; -1 when the wait gave up.
  auto fetch_item = [&](int e) -> int {
    const int slot = (e - 1) % kItemRing;
    if (!mbar_wait(bar(BAR_ITEMFULL + slot), ((e - 1) / kItemRing) & 1, abort_flag, p.error_flag, 12)) return -1;
    const int v = uniform(item_ring[slot]);
    mbar_arrive(bar(BAR_ITEMEMPTY + slot));
    return v;
  };

  if (warp < 4) {
    reg_dec<kRegsControl>();
    if (warp == 0 && lane == 0) {
      // ---------------------------------------------------------- TMA producer + item dispenser
      Item it = decode_item(p, kFirstItem);
      uint32_t g = 0;                 // ring slots used so far; every item starts on an even one (stage 0)
      uint32_t qcnt_a = 1, qcnt_b = it.has_b ? 1u : 0u;   // Q tiles loaded so far
      bool ok = true;
      // K and V of tile j into ring slot `slot`, each as soon as its stage has been released
      auto load_slot = [&](const Item &item, int j, uint32_t slot) -> bool {
        const int s = slot % kStages;
        const uint32_t ph = (slot / kStages) & 1;
        if (!mbar_wait(bar(BAR_KEMPTY + s), ph ^ 1, abort_flag, p.error_flag, 1)) return false;
        load_kv_tile(item, j, slot, true);
        if (!mbar_wait(bar(BAR_VEMPTY + s), ph ^ 1, abort_flag, p.error_flag, 2)) return false;
        load_kv_tile(item, j, slot, false);
        return true;
      };
      for (int e = 1; ok; ++e) {
        // take the next item now; its number is needed only after this item's first loads are on their way
        const int next_item = uniform(static_cast<int>(kGridSize + atomicAdd(p.ticket, 1u)));
        if (e > 1) {               // the first item's first loads left before the set-up barrier
          if (!(ok = mbar_wait(bar(BAR_QEMPTY + 0), (qcnt_a & 1) ^ 1, abort_flag, p.error_flag, 13))) break;
          load_q_tile(it, 0);
          ++qcnt_a;
          if (!(ok = load_slot(it, 0, g))) break;
          if (it.has_b) {
            if (!(ok = mbar_wait(bar(BAR_QEMPTY + 1), (qcnt_b & 1) ^ 1, abort_flag, p.error_flag, 14))) break;
            load_q_tile(it, 1);
            ++qcnt_b;
          }
        }
        // Publish the next item before the rest of this one: the MMA lane reads it at the end of this
        // item, and nothing up to here waited for anything it issues after that.
        {
          const int slot = (e - 1) % kItemRing;   // entries are numbered from 1
          if (!(ok = mbar_wait(bar(BAR_ITEMEMPTY + slot), (((e - 1) / kItemRing) & 1) ^ 1, abort_flag, p.error_flag, 15))) break;
          item_ring[slot] = next_item;
          mbar_arrive(bar(BAR_ITEMFULL + slot));
        }
        for (int j = 1; j < it.nt; ++j) {
          if (!(ok = load_slot(it, j, g + j))) break;
        }
        if (!ok) break;
        g += it.nt;
        if (g & 1) {
          // An odd number of tiles: one empty slot keeps the next item on stage 0, so that the MMA lane's
          // stage index is its loop counter's parity.  The slot is "filled" by a plain arrival.
          const uint32_t ph = (g / kStages) & 1;
          if (!(ok = mbar_wait(bar(BAR_KEMPTY + 1), ph ^ 1, abort_flag, p.error_flag, 1))) break;
          mbar_arrive(bar(BAR_KFULL + 1));
          if (!(ok = mbar_wait(bar(BAR_VEMPTY + 1), ph ^ 1, abort_flag, p.error_flag, 2))) break;
          mbar_arrive(bar(BAR_VFULL + 1));
          ++g;
        }
        it = decode_item(p, next_item);
        if (!it.valid) break;
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------------------------------------------------- MMA issuer
      // Descriptors are built once; per instruction only a constant is added to the
      // start-address field.  The issuing thread's own instruction count per MMA must
      // stay well under the 64 cycles a 128x128x16 MMA takes, or the tensor pipe starves.
      const uint32_t dq0 = smem_desc_lo(smem_base + kSmemQ, 16);
      const uint32_t dk0 = smem_desc_lo(smem_base + kSmemK, 16);
      const uint32_t dv0 = smem_desc_lo(smem_base + kSmemV, kHalfTile);
      constexpr uint32_t kTileStep = kTileBytes >> 4; // one tile further, in descriptor address units
      // Per item the loop below is the one of the non-persistent kernel: tile j of the item lives in ring
      // stage j & 1 (every item starts on an even ring slot), so stages and shared-memory descriptors
      // derive from the loop counter alone; what runs across items -- ring slots used, tiles per query
      // tile, Q tiles consumed -- only enters the barrier parities.
      uint32_t g0 = 0;                 // ring slot of the current item's tile 0 (even)
      uint32_t tiles_a = 0, tiles_b = 0, q_par_a = 0, q_par_b = 0;
      // S_X = Q_X . K[j]^T; `last` marks the last reader of K[j], which frees the stage; last_qk the item's
      // last reader of Q_X, which frees the Q tile for the producer
      auto issue_qk = [&](int x, int j, bool last, bool last_qk) -> bool {
        const int s = j % kStages;
        if (!mbar_wait(bar(BAR_KFULL + s), ((g0 + j) / kStages) & 1, abort_flag, p.error_flag, 4)) return false;
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
        if (last_qk) tc_commit(bar(BAR_QEMPTY + x));
        tc_commit(bar(BAR_SFULL + x));
        return true;
      };
      // O_X += P_X . V[j] ; `last` marks the last reader of V[j]
      auto issue_pv = [&](int x, int j, bool last) -> bool {
        const int s = j % kStages;
        const uint32_t par = ((x ? tiles_b : tiles_a) + j) & 1;
        // The softmax warps publish the first 64 positions of P before they start on the
        // other 64, so that half of this product overlaps their remaining exponentials.
        if (!mbar_wait(bar(BAR_PHALF + x), par, abort_flag, p.error_flag, 10)) return false;
        if (!mbar_wait(bar(BAR_VFULL + s), ((g0 + j) / kStages) & 1, abort_flag, p.error_flag, 6)) return false;
        tc_fence_after();
        const uint32_t pcol = tmem + kColS + 128 * x, ocol = tmem + kColO + 128 * x;
        const uint32_t dv = dv0 + s * kTileStep;
        const uint32_t acc0 = j > 0 ? 1u : 0u;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // 16 positions per step: 8 TMEM columns of packed P, 16 rows (2048 B) of V
          tc_mma_ts(ocol, pcol + 8 * k, dv + k * (2048 >> 4), kDescHi, idesc_pv, k > 0 ? 1u : acc0);
        }
        if (!mbar_wait(bar(BAR_PREADY + x), par, abort_flag, p.error_flag, 5)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 4; k < 8; ++k) tc_mma_ts(ocol, pcol + 8 * k, dv + k * (2048 >> 4), kDescHi, idesc_pv, 1u);
        if (last) tc_commit(bar(BAR_VEMPTY + s));
        tc_commit(bar(BAR_ODONE + x));
        return true;
      };
      // the first Q.K^T products of an item (tile 0, stage 0), once its Q tiles are there
      auto first_products = [&](const Item &it) -> bool {
        if (!mbar_wait(bar(BAR_QFULL + 0), q_par_a, abort_flag, p.error_flag, 3)) return false;
        q_par_a ^= 1u;
        if (!issue_qk(0, 0, !it.has_b, it.nt_a == 1)) return false;
        if (it.has_b) {
          if (!mbar_wait(bar(BAR_QFULL + 1), q_par_b, abort_flag, p.error_flag, 11)) return false;
          q_par_b ^= 1u;
          if (!issue_qk(1, 0, true, it.nt_b == 1)) return false;
        }
        return true;
      };
      Item cur = decode_item(p, kFirstItem);
      bool ok = first_products(cur);
      for (int e = 1; ok; ++e) {
        const int nt = cur.nt, nt_a = cur.nt_a, nt_b = cur.nt_b;
        const bool has_b = cur.has_b;
        // tile B (when present) reads every KV tile that A reads, and reads it after A
        for (int j = 0; ok && j < nt; ++j) {
          if (j < nt_a) {
            ok = issue_pv(0, j, !has_b);
            if (ok && j + 1 < nt_a) ok = issue_qk(0, j + 1, !has_b, j + 2 == nt_a);
          }
          if (ok && has_b) {
            ok = issue_pv(1, j, true);
            if (ok && j + 1 < nt_b) ok = issue_qk(1, j + 1, true, j + 2 == nt_b);
          }
        }
        if (!ok) break;
        tiles_a += nt_a;
        tiles_b += nt_b;
        g0 += nt;
        if (g0 & 1) {
          // the empty slot that pads an odd tile count: release it behind the products issued so far
          if (!(ok = mbar_wait(bar(BAR_KFULL + 1), (g0 / kStages) & 1, abort_flag, p.error_flag, 4))) break;
          tc_commit(bar(BAR_KEMPTY + 1));
          if (!(ok = mbar_wait(bar(BAR_VFULL + 1), (g0 / kStages) & 1, abort_flag, p.error_flag, 6))) break;
          tc_commit(bar(BAR_VEMPTY + 1));
          ++g0;
        }
        // The next item's first products go out right here, behind this item's last P.V: its S_A and S_B
        // are being computed while the softmax warps are in their epilogue.
        const int nid = fetch_item(e);
        if (nid < 0) break;
        cur = decode_item(p, nid);
        if (!cur.valid) break;
        ok = first_products(cur);
      }
    } else if (warp == 3 && lane == 0) {
      // ---------------------------------------------------------- tensor stores of both tiles' output
      // The lane polls the two groups' "staging tile written" barriers in turn and sleeps in between:
      // it is in no hurry, and it shares its scheduler with two softmax warps that are.
      uint32_t n[2] = {0, 0};
      bool live[2] = {true, true};
      long long t0 = clock64();
      while (live[0] || live[1]) {
        bool progress = false;
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (!live[x] || !mbar_try_wait(bar(BAR_STGWR + x), n[x] & 1)) continue;
          progress = true;
          t0 = clock64();
          ++n[x];
          volatile int *coord = stg_coord + 4 * x;
          if (coord[3]) {                // the group has left its loop
            live[x] = false;
            continue;
          }
          tma_store_4d(&map_o, smem_base + kSmemStg, 0, coord[0], coord[1], coord[2]);
          tma_store_4d(&map_o, smem_base + kSmemStg + kHalfTile, 64, coord[0], coord[1], coord[2]);
          bulk_commit();
          bulk_wait_read0();             // the staging tile has been read: the next user may write it
          mbar_arrive(bar(BAR_STGFREE));
          mbar_arrive(bar(BAR_STGDONE + x));
        }
        if (!progress) {
          __nanosleep(200);
          if (*abort_flag) break;
          if (clock64() - t0 > 4000000000LL) {   // bounded like every other wait
            *abort_flag = 1;
            *reinterpret_cast<volatile int *>(p.error_flag) = 18;
            break;
          }
        }
      }
      bulk_wait0();
    }
  } else {
    reg_inc<kRegsSoftmax>();
    // ------------------------------------------------------------ softmax + epilogue of tile X
    const int x = (warp >> 2) - 1;               // 0: tile A (warps 4-7), 1: tile B (warps 8-11)
    const int quad = warp & 3;                   // TMEM lane quadrant this warp may touch
    const int trow = quad * 32 + lane;           // row within the tile = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t scol = tmem + lane_addr + kColS + 128 * x;
    const uint32_t ocol = tmem + lane_addr + kColO + 128 * x;
    const bool elected = quad == 0 && lane == 0; // takes the staging tile for the group
    uint32_t t = 0;                              // tiles this group has processed (barrier parity)
    uint32_t n_epi = 0;                          // epilogues this group has run
    Item cur = decode_item(p, kFirstItem);
    bool ok = true;
    for (int e = 1; ok && cur.valid; ++e) {
      const int ntx = x == 0 ? cur.nt_a : cur.nt_b;
      if (ntx > 0) {
        const int trow0 = cur.row0 + x * kBM;
        const int row = trow0 + trow;                // query token index within the call
        const int vis_end = min(p.n, p.offset + row + 1); // columns < vis_end are visible to this row
        float m_ref = -INFINITY, l = 0.f;
        for (int j = 0; j < ntx; ++j, ++t) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar(BAR_SFULL + x), t & 1, abort_flag, p.error_flag, 7))) {
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
            for (int i = 0; i < 8; ++i)
              mxa[i] = max3(mxa[i], __uint_as_float(su[c + i]), __uint_as_float(su[c + 8 + i]));
          }
          float mx = fmaxf(max3(mxa[0], mxa[1], mxa[2]), fmaxf(max3(mxa[3], mxa[4], mxa[5]), fmaxf(mxa[6], mxa[7])));
          mx *= p.scale_log2;
          // lazy rescale: keep the old reference max unless the new one is much larger
          const bool grow = mx > m_ref + kRescaleThreshold;
          if (__any_sync(0xffffffffu, grow) && j > 0) {
            // O must hold every P.V issued so far before it is rescaled
            if (!__all_sync(0xffffffffu, mbar_wait(bar(BAR_ODONE + x), (t - 1) & 1, abort_flag, p.error_flag, 8))) {
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
            const uint64_t x2 =
                fma2(pack2(__uint_as_float(su[2 * c]), __uint_as_float(su[2 * c + 1])), scale2, neg_m2);
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
        if (!ok) break;
        // ---- epilogue: O / l -> staging tile -> tensor store
        if (!__all_sync(0xffffffffu, mbar_wait(bar(BAR_ODONE + x), (t - 1) & 1, abort_flag, p.error_flag, 9))) {
          ok = false;
          break;
        }
        tc_fence_after();
        // The staging tile is shared by both groups; its users are numbered as they come, and user u
        // waits until user u - 1 has been read out by its tensor store.  A wait on a parity can only
        // tell a barrier's current phase from the one before, so the group first makes sure that its
        // own previous store is done: then every user before u - 1 is done when the number is taken.
        if (elected) {
          bool got = n_epi == 0 || mbar_wait(bar(BAR_STGDONE + x), (n_epi - 1) & 1, abort_flag, p.error_flag, 19);
          if (got) {
            const uint32_t u = atomicAdd(stg_seq, 1u);
            got = u == 0 || mbar_wait(bar(BAR_STGFREE), (u - 1) & 1, abort_flag, p.error_flag, 16);
          }
          if (got) {
            stg_coord[4 * x + 0] = cur.h;
            stg_coord[4 * x + 1] = trow0;
            stg_coord[4 * x + 2] = cur.b;
            mbar_arrive(bar(BAR_STGRDY + x));
          }
        }
        if (!__all_sync(0xffffffffu, mbar_wait(bar(BAR_STGRDY + x), n_epi & 1, abort_flag, p.error_flag, 17))) {
          ok = false;
          break;
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const uint32_t stg_row = smem_base + kSmemStg + trow * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tc_ld32(ocol + 32 * c, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 u4;
            u4.x = Elem<T>::pack(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
            u4.y = Elem<T>::pack(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
            u4.z = Elem<T>::pack(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
            u4.w = Elem<T>::pack(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
            // element d = 32 c + 8 i: half tile c / 2, 16-byte chunk (c & 1) * 4 + i, swizzled by the row
            const uint32_t chunk = static_cast<uint32_t>((c & 1) * 4 + i) ^ static_cast<uint32_t>(trow & 7);
            st_shared_v4(stg_row + (c >> 1) * kHalfTile + (chunk << 4), u4);
          }
        }
        tc_fence_before();          // O_X has been read: the next item's first P.V may overwrite it
        fence_proxy_async_smem();   // the tensor store reads what this thread wrote
        mbar_arrive(bar(BAR_STGWR + x));    // 128 arrivals release the group's store lane
        ++n_epi;
      }
      // next item of this CTA
      // Lane 0 reads the entry; the warp takes it through a warp-wide reduction, whose result the
      // compiler knows to be the same in every lane: the loop bounds, barrier parities and addresses
      // derived from it stay on the uniform datapath, as they do for an item taken from blockIdx.
      int nid = INT_MIN;
      if (lane == 0) nid = fetch_item(e);
      nid = __reduce_max_sync(0xffffffffu, nid);
      if (nid < 0) {
        ok = false;
        break;
      }
      cur = decode_item(p, nid);
    }
    // Tell the group's store lane that nothing more comes -- once it has taken the group's last tile:
    // it tells this arrival from the previous one by the parity alone.
    if (elected) {
      if (n_epi > 0) (void)mbar_wait(bar(BAR_STGDONE + x), (n_epi - 1) & 1, abort_flag, p.error_flag, 19);
      stg_coord[4 * x + 3] = 1;
    }
    __syncwarp();
    mbar_arrive(bar(BAR_STGWR + x));
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
  if (threadIdx.x == 0) {
    // the last CTA to finish leaves the counter pair as it found it
    __threadfence();
    const unsigned int done = atomicAdd(p.ticket + 1, 1u);
    if (done == kGridSize - 1) {
      atomicExch(p.ticket, 0u);
      atomicExch(p.ticket + 1, 0u);
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------

// Counter pairs: a few per (device, stream), used in turn.  Launches on one stream run one after the
// other (a programmatic dependent launch overlaps at most its neighbour), so a pair is back at zero
// long before its turn comes again.  Returns nullptr when no more streams can be served.
constexpr int kPairsPerStream = 4, kMaxStreams = 64, kMaxDevices = 64;
struct StreamSlots {
  cudaStream_t stream;
  int next;
};
struct DeviceSlots {
  unsigned int *base = nullptr;          // kMaxStreams * kPairsPerStream pairs, zeroed once
  std::vector<StreamSlots> streams;
};

unsigned int *ticket_pair(int dev, cudaStream_t stream) {
  static std::mutex mu;
  static DeviceSlots slots[kMaxDevices];
  if (dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lk(mu);
  DeviceSlots &d = slots[dev];
  if (!d.base) {
    const size_t bytes = static_cast<size_t>(kMaxStreams) * kPairsPerStream * 2 * sizeof(unsigned int);
    if (cudaMalloc(reinterpret_cast<void **>(&d.base), bytes) != cudaSuccess) {
      d.base = nullptr;
      (void)cudaGetLastError();
      return nullptr;
    }
    if (cudaMemset(d.base, 0, bytes) != cudaSuccess) return nullptr;
  }
  size_t i = 0;
  for (; i < d.streams.size(); ++i)
    if (d.streams[i].stream == stream) break;
  if (i == d.streams.size()) {
    if (d.streams.size() >= static_cast<size_t>(kMaxStreams)) return nullptr;
    d.streams.push_back(StreamSlots{stream, 0});
  }
  StreamSlots &s = d.streams[i];
  unsigned int *pair = d.base + (i * kPairsPerStream + s.next) * 2;
  s.next = (s.next + 1) % kPairsPerStream;
  return pair;
}

int sm_count(int dev) {
  static int cached[kMaxDevices] = {};
  if (dev < 0 || dev >= kMaxDevices) return 0;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

} // namespace tc5p

cudaError_t launch_attn_prefill_tc5p(const PrefillParams &p, bool bf16, cudaStream_t stream) {
  using namespace tc5p;
  const AttnGeom &g = p.g;
  // A captured launch would be replayed with the counter pair of the capturing stream, possibly next to
  // other work that owns the same pair: leave captures to the non-persistent kernel.
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    (void)cudaGetLastError();
    return cudaErrorNotSupported;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const int sms = sm_count(dev);
  if (sms <= 0) return cudaErrorNotSupported;
  const long nqb = (p.m + 2 * kBM - 1) / (2 * kBM);
  const long n_items = nqb * g.n_heads * g.batch;
  if (n_items <= 0 || n_items > 0x3fffffff) return cudaErrorNotSupported;
  CUtensorMap mq, mk, mv, mk_tail, mv_tail, mo;
  // q / out: (d, head, token, seq); k/v: (d, pos, kv_head, seq), or (d, pos in page, kv_head, page) over a pool
  if (!make_tensor_map_4d(&mq, bf16, p.q, g.n_heads, p.m, g.batch, kHeadDim, g.q_tok, g.q_seq, 1, kBM) ||
      !make_tensor_map_4d(&mo, bf16, p.out, g.n_heads, p.m, g.batch, kHeadDim, g.out_tok, g.out_seq, 1, kBM))
    return cudaErrorNotSupported;
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
  int *err_dev = kernel_error_word_dev();
  if (!err_dev) return cudaErrorNotSupported;
  unsigned int *pair = ticket_pair(dev, stream);
  if (!pair) return cudaErrorNotSupported;
  Params kp{};
  kp.m = p.m;
  kp.n = p.n;
  kp.offset = p.offset;
  kp.group = g.group;
  kp.n_heads = g.n_heads;
  kp.nqb = static_cast<int>(nqb);
  kp.n_items = static_cast<int>(n_items);
  kp.scale_log2 = p.scale_log2;
  kp.error_flag = err_dev;
  kp.ticket = pair;
  kp.page_table = p.pg.table;
  kp.table_stride = p.pg.table_stride;
  kp.page_shift = p.pg.page_shift;
  const dim3 grid(static_cast<unsigned>(n_items < sms ? n_items : sms));
  // the shared-memory opt-in is a property of (function, device): set it on the first launch per device
  static bool attr_set[2][kMaxDevices] = {};
  if (!attr_set[bf16 ? 1 : 0][dev]) {
    // the register budgets inside the kernel assume the allocation the compiler chose for the launch
    cudaFuncAttributes fa{};
    e = bf16 ? cudaFuncGetAttributes(&fa, attn_prefill_tc5p_kernel<__nv_bfloat16>)
             : cudaFuncGetAttributes(&fa, attn_prefill_tc5p_kernel<__half>);
    if (e != cudaSuccess) return e;
    if (fa.numRegs < kRegsLaunch) return cudaErrorNotSupported;
    e = bf16 ? cudaFuncSetAttribute(attn_prefill_tc5p_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal)
             : cudaFuncSetAttribute(attn_prefill_tc5p_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
    if (e != cudaSuccess) return e;
    attr_set[bf16 ? 1 : 0][dev] = true;
  }
  if (bf16)
    attn_prefill_tc5p_kernel<__nv_bfloat16><<<grid, kThreads, kSmemTotal, stream>>>(mq, mk, mv, mk_tail, mv_tail, mo, kp);
  else
    attn_prefill_tc5p_kernel<__half><<<grid, kThreads, kSmemTotal, stream>>>(mq, mk, mv, mk_tail, mv_tail, mo, kp);
  return cudaGetLastError();
}

} // namespace b200attn
