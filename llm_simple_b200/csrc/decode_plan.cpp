// Host-side work partition of a decode step ("plan") for attn_decode_tma_kernel.
//
// Every (sequence, KV head) cache is a run of 64-position tiles; the runs are laid end to end in
// (sequence, KV head) order and the line is cut into n_ctas contiguous shares of equal cost, where
// a tile costs 1 and every piece a CTA starts costs kPieceCost on top (query staging, pipeline
// restart, the combine at its end).  A cut never leaves a piece of a single tile when one more
// tile on the previous share avoids it.  A cache that was cut gets one scratch slot per piece and
// a merge group.  Pure host code: no CUDA call.
#include "kernels.h"

#include <algorithm>
#include <cstring>
#include <vector>

namespace b200attn {

namespace {
constexpr int kTile = 64;
constexpr double kPieceCost = 1.5; // tiles
inline size_t align16(size_t x) { return (x + 15) & ~static_cast<size_t>(15); }
} // namespace

size_t decode_plan_capacity(int batch, int n_kv_heads, int n_ctas) {
  if (batch <= 0 || n_kv_heads <= 0 || n_ctas <= 0) return 0;
  const size_t units = static_cast<size_t>(batch) * n_kv_heads;
  return sizeof(PlanHeader) + align16((static_cast<size_t>(n_ctas) + 1) * 4) +
         (units + static_cast<size_t>(n_ctas)) * sizeof(PlanItem) + align16(units * sizeof(PlanGroup));
}

size_t build_decode_plan(void *blob, size_t capacity, const int32_t *kv_len, int batch, int n_kv_heads, int group,
                         int append, int n_ctas) {
  if (!blob || !kv_len || batch <= 0 || n_kv_heads <= 0 || group <= 0 || n_ctas <= 0) return 0;
  append = append ? 1 : 0;
  long total_tiles = 0;
  int max_total = 0;
  for (int b = 0; b < batch; ++b) {
    if (kv_len[b] < 0) return 0;
    const int total = kv_len[b] + append;
    max_total = std::max(max_total, total);
    total_tiles += static_cast<long>((total + kTile - 1) / kTile) * n_kv_heads;
  }
  // no more CTAs than pairs of tiles: a share below two tiles is all overhead
  const int ctas = static_cast<int>(std::min<long>(n_ctas, std::max<long>(1, total_tiles / 2)));

  std::vector<PlanItem> items;
  std::vector<PlanGroup> groups;
  std::vector<int32_t> cta_begin;
  items.reserve(static_cast<size_t>(batch) * n_kv_heads + ctas);
  cta_begin.reserve(ctas + 1);
  cta_begin.push_back(0);
  int n_slots = 0;
  // Each share's budget is set when the share is opened, from what is left: the tiles not yet
  // handed out, one piece per cache not yet finished and one cut per share still to come.  Errors
  // of the estimate therefore spread over the remaining shares instead of piling up in the last.
  long tiles_left = total_tiles;
  long units_left = static_cast<long>(batch) * n_kv_heads; // caches not yet finished (the one being cut included)
  int cta = 0;
  double used = 0.0, budget = 0.0;
  auto open_cta = [&]() {
    const int ctas_left = ctas - cta;
    budget = (static_cast<double>(tiles_left) + kPieceCost * static_cast<double>(units_left + ctas_left - 1)) / ctas_left;
    used = 0.0;
  };
  auto close_cta = [&]() {
    cta_begin.push_back(static_cast<int32_t>(items.size()));
    ++cta;
    open_cta();
  };
  open_cta();
  for (int b = 0; b < batch; ++b) {
    const int len_old = kv_len[b];
    const int total = len_old + append;
    const int tiles = (total + kTile - 1) / kTile;
    for (int kvh = 0; kvh < n_kv_heads; ++kvh) {
      int t0 = 0;
      const size_t first_item = items.size();
      if (tiles == 0) {
        // an empty cache without a new token: a piece without tiles, which writes a zero result
        // (log-sum-exp -inf) so that every output row of the call is defined
        PlanItem w{};
        w.b = b;
        w.kvh = kvh;
        w.len_old = len_old;
        w.slot = -1;
        items.push_back(w);
        used += kPieceCost;
        --units_left;
        if (cta < ctas - 1 && used >= budget - 0.5) close_cta();
        continue;
      }
      while (t0 < tiles) {
        int take = tiles - t0;
        if (cta < ctas - 1) {
          const double room = budget - (used + kPieceCost);
          int fit = room < 1.0 ? 1 : static_cast<int>(room + 0.5);
          if (fit < take) {
            if (take - fit == 1) fit = take; // do not leave a single tile behind
            take = fit;
          }
        }
        PlanItem w{};
        w.b = b;
        w.kvh = kvh;
        w.pos0 = t0 * kTile;
        w.pos_end = std::min(total, (t0 + take) * kTile);
        w.len_old = len_old;
        w.slot = -1;
        w.has_new = (append && w.pos0 <= len_old && len_old < w.pos_end) ? 1 : 0;
        items.push_back(w);
        used += kPieceCost + take;
        t0 += take;
        tiles_left -= take;
        if (t0 == tiles) --units_left;
        if (cta < ctas - 1 && used >= budget - 0.5) close_cta();
      }
      const int parts = static_cast<int>(items.size() - first_item);
      if (parts > 1) {
        groups.push_back({n_slots, parts, b, kvh});
        for (int i = 0; i < parts; ++i) items[first_item + i].slot = n_slots++;
      }
    }
  }
  while (static_cast<int>(cta_begin.size()) < ctas + 1) cta_begin.push_back(static_cast<int32_t>(items.size()));

  PlanHeader h{};
  h.magic = kPlanMagic;
  h.n_ctas = ctas;
  h.n_items = static_cast<int32_t>(items.size());
  h.n_groups = static_cast<int32_t>(groups.size());
  h.n_slots = n_slots;
  h.batch = batch;
  h.n_kv_heads = n_kv_heads;
  h.group = group;
  h.append = append;
  h.max_total = max_total;
  h.off_cta_begin = static_cast<int32_t>(sizeof(PlanHeader));
  h.off_items = static_cast<int32_t>(h.off_cta_begin + align16(cta_begin.size() * 4));
  h.off_groups = static_cast<int32_t>(h.off_items + items.size() * sizeof(PlanItem));
  h.total_bytes = static_cast<int32_t>(align16(h.off_groups + groups.size() * sizeof(PlanGroup)));
  h.total_tiles = static_cast<int32_t>(total_tiles);
  for (const PlanGroup &g : groups) h.max_parts = std::max(h.max_parts, g.n_parts);
  if (static_cast<size_t>(h.total_bytes) > capacity) return 0;
  unsigned char *out = static_cast<unsigned char *>(blob);
  std::memset(out, 0, static_cast<size_t>(h.total_bytes));
  std::memcpy(out, &h, sizeof h);
  std::memcpy(out + h.off_cta_begin, cta_begin.data(), cta_begin.size() * 4);
  if (!items.empty()) std::memcpy(out + h.off_items, items.data(), items.size() * sizeof(PlanItem));
  if (!groups.empty()) std::memcpy(out + h.off_groups, groups.data(), groups.size() * sizeof(PlanGroup));
  return static_cast<size_t>(h.total_bytes);
}

} // namespace b200attn
