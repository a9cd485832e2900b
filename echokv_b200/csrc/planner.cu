// Host-side plan of one step's KV writes (no device code): the residual-slot allocator, the K_ref ring cursor and the
// per-step plan of echokv_vllm/write_plan.py:98-240 (`WritePlanner.plan`), decision for decision -- the same groups
// finalized, the same residual slots handed out and evicted, the same order of every output list -- so that a plan
// made here and one made by the Python planner are interchangeable.
#include <algorithm>
#include <cstdint>
#include <unordered_map>
#include <utility>
#include <vector>

#include "common.cuh"

namespace echokv {

// A map that remembers the order in which keys were first inserted (what a Python dict iterates in); a later write to
// a key keeps its place and replaces its value.
struct OrderedLog {
  std::vector<std::pair<int64_t, int64_t>> items;
  std::unordered_map<int64_t, size_t> at;
  void put(int64_t k, int64_t v) {
    auto it = at.find(k);
    if (it == at.end()) {
      at.emplace(k, items.size());
      items.emplace_back(k, v);
    } else {
      items[it->second].second = v;
    }
  }
};

struct SlotInfo {
  int64_t block, group, fill, last;
  uint64_t stamp;  // insertion order among the live slots
};

struct Planner {
  int64_t bs, g, num_slots, kref_window;
  std::vector<int64_t> free;                        // popped from the end: 0, 1, 2, ...
  std::unordered_map<int64_t, int64_t> block_slot;  // block -> its residual slot
  std::unordered_map<int64_t, SlotInfo> slot_info;  // live slots
  std::unordered_map<int64_t, int64_t> sealed;      // block -> bitmask of sealed groups
  int64_t step = 0, kref_pos = 0, kref_fill = 0;
  uint64_t stamp = 0;

  void drop(int64_t slot, OrderedLog& blocks) {
    const int64_t block = slot_info.at(slot).block;
    slot_info.erase(slot);
    block_slot.erase(block);
    free.push_back(slot);
    blocks.put(block, -1);
  }
  bool is_sealed(int64_t block, int64_t group) const {
    auto it = sealed.find(block);
    return it != sealed.end() && ((it->second >> group) & 1);
  }
};

}  // namespace echokv

using namespace echokv;

extern "C" {

void* echokv_planner_create(int32_t block_size, int32_t k_group, int32_t residual_slots, int32_t kref_window) {
  if (block_size <= 0 || k_group <= 0 || block_size % k_group || residual_slots < 0 || kref_window < 0) {
    set_error(ECHOKV_E_ARGUMENT, "planner: bad block_size / k_group / residual_slots / kref_window");
    return nullptr;
  }
  Planner* p = new Planner();
  p->bs = block_size; p->g = k_group; p->num_slots = residual_slots; p->kref_window = kref_window;
  for (int64_t s = residual_slots - 1; s >= 0; --s) p->free.push_back(s);
  return p;
}

void echokv_planner_destroy(void* planner) { delete static_cast<Planner*>(planner); }

int64_t echokv_planner_get(void* planner, int32_t what) {
  const Planner* p = static_cast<const Planner*>(planner);
  if (!p) return -1;
  switch (what) {
    case 0: return (int64_t)p->free.size();
    case 1: return p->kref_pos;
    case 2: return p->kref_fill;
    case 3: return p->step;
    case 4: return p->num_slots;
    case 5: return (int64_t)p->slot_info.size();
    default: return -1;
  }
}

int64_t echokv_planner_sealed_mask(void* planner, int64_t block, int64_t otherwise) {
  const Planner* p = static_cast<const Planner*>(planner);
  auto it = p->sealed.find(block);
  return it == p->sealed.end() ? otherwise : it->second;
}

int echokv_planner_plan(void* planner, const int64_t* slots, int64_t n_rows, int64_t* tok, int64_t* fin,
                        int64_t* evictions, int64_t* opened, int64_t* touched, int64_t* touched_fill,
                        int64_t* touched_count, int64_t* map_block, int64_t* map_value, int64_t* grp_slot,
                        int64_t* grp_value, int64_t* counts) {
  Planner* P = static_cast<Planner*>(planner);
  if (!P || (n_rows > 0 && !slots) || !tok || !fin || !evictions || !opened || !touched || !touched_fill ||
      !touched_count || !map_block || !map_value || !grp_slot || !grp_value || !counts)
    return set_error(ECHOKV_E_ARGUMENT, "planner: null pointer");
  P->step += 1;
  const int64_t bs = P->bs, g = P->g, gpb = bs / g, w = 3 + g;
  OrderedLog log_block, log_group;

  // live tokens in row order
  std::vector<int64_t> live;
  live.reserve((size_t)n_rows);
  for (int64_t r = 0; r < n_rows; ++r)
    if (slots[r] >= 0) live.push_back(r);
  const int64_t n = (int64_t)live.size();
  std::vector<int64_t> blk((size_t)n), off((size_t)n), gid((size_t)n), pos((size_t)n);
  for (int64_t i = 0; i < n; ++i) {
    const int64_t s = slots[live[(size_t)i]];
    blk[(size_t)i] = s / bs; off[(size_t)i] = s % bs;
    gid[(size_t)i] = blk[(size_t)i] * gpb + off[(size_t)i] / g;
    pos[(size_t)i] = off[(size_t)i] % g;
  }

  // blocks whose offset 0 is written open: their residual slot and sealed mask go first
  std::vector<int64_t> open_b;
  for (int64_t i = 0; i < n; ++i)
    if (off[(size_t)i] == 0) open_b.push_back(blk[(size_t)i]);
  std::sort(open_b.begin(), open_b.end());
  open_b.erase(std::unique(open_b.begin(), open_b.end()), open_b.end());
  for (int64_t b : open_b) {
    auto it = P->block_slot.find(b);
    if (it != P->block_slot.end()) P->drop(it->second, log_block);
    P->sealed.erase(b);
  }

  // tokens sorted by (group id, position), ties in row order; runs of equal group id are the step's K groups
  std::vector<int64_t> order((size_t)n);
  for (int64_t i = 0; i < n; ++i) order[(size_t)i] = i;
  std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) {
    return gid[(size_t)a] != gid[(size_t)b] ? gid[(size_t)a] < gid[(size_t)b] : pos[(size_t)a] < pos[(size_t)b];
  });
  std::vector<int64_t> first, size;
  for (int64_t i = 0; i < n; ++i) {
    if (i == 0 || gid[(size_t)order[(size_t)i]] != gid[(size_t)order[(size_t)(i - 1)]]) {
      first.push_back(i);
      size.push_back(0);
    }
    size.back() += 1;
  }
  const int64_t ng = (int64_t)first.size();
  std::vector<char> whole((size_t)ng);
  for (int64_t u = 0; u < ng; ++u) {
    const int64_t gd = gid[(size_t)order[(size_t)first[(size_t)u]]];
    whole[(size_t)u] = size[(size_t)u] == g && !(!P->sealed.empty() && P->is_sealed(gd / gpb, gd % gpb));
  }

  // groups that arrive whole are finalized straight from the step's key rows
  int64_t n_fin = 0;
  std::vector<int64_t> whole_blocks;
  for (int64_t u = 0; u < ng; ++u) {
    if (!whole[(size_t)u]) continue;
    const int64_t gd = gid[(size_t)order[(size_t)first[(size_t)u]]];
    int64_t* line = fin + n_fin * w;
    line[0] = gd / gpb; line[1] = gd % gpb; line[2] = -1;
    for (int64_t k = 0; k < g; ++k) line[3 + k] = live[(size_t)order[(size_t)(first[(size_t)u] + k)]];
    whole_blocks.push_back(gd / gpb);
    ++n_fin;
  }
  if (!P->block_slot.empty() && !whole_blocks.empty()) {  // a rewritten group that still owned a slot
    std::unordered_map<int64_t, std::vector<int64_t>> by_block;
    for (int64_t i = 0; i < n_fin; ++i) by_block[fin[i * w]].push_back(fin[i * w + 1]);
    for (int64_t b : whole_blocks) {
      auto it = P->block_slot.find(b);
      if (it == P->block_slot.end()) continue;
      const int64_t grp = P->slot_info.at(it->second).group;
      const auto& gs = by_block[b];
      if (std::find(gs.begin(), gs.end(), grp) != gs.end()) P->drop(it->second, log_block);
    }
  }

  int64_t* tok_slot = tok;
  int64_t* tok_res = tok + n_rows;
  int64_t* tok_sealed = tok + 2 * n_rows;
  int64_t* tok_kref = tok + 3 * n_rows;
  for (int64_t r = 0; r < n_rows; ++r) { tok_slot[r] = slots[r]; tok_res[r] = -1; tok_sealed[r] = 0; tok_kref[r] = -1; }

  // slots of the blocks written in this step are never evicted by it
  std::vector<int64_t> ublk(blk);
  std::sort(ublk.begin(), ublk.end());
  ublk.erase(std::unique(ublk.begin(), ublk.end()), ublk.end());
  std::vector<char> protected_slot((size_t)P->num_slots + 1, 0);
  for (int64_t b : ublk) {
    auto it = P->block_slot.find(b);
    if (it != P->block_slot.end()) protected_slot[(size_t)it->second] = 1;
  }

  int64_t n_evict = 0;
  for (int64_t u = 0; u < ng; ++u) {
    if (whole[(size_t)u]) continue;
    const int64_t f0 = first[(size_t)u], sz = size[(size_t)u];
    const int64_t gd = gid[(size_t)order[(size_t)f0]], b = gd / gpb, gr = gd % gpb;
    if (P->is_sealed(b, gr)) {
      for (int64_t k = 0; k < sz; ++k) tok_sealed[live[(size_t)order[(size_t)(f0 + k)]]] = 1;
      continue;
    }
    int64_t top = 0;
    for (int64_t k = 0; k < sz; ++k) top = std::max(top, pos[(size_t)order[(size_t)(f0 + k)]]);
    int64_t slot = -1;
    {
      auto it = P->block_slot.find(b);
      if (it != P->block_slot.end() && P->slot_info.at(it->second).group == gr) slot = it->second;
    }
    if (top == g - 1) {  // the group completes in this step
      int64_t* line = fin + n_fin * w;
      line[0] = b; line[1] = gr; line[2] = slot;
      for (int64_t k = 0; k < g; ++k) line[3 + k] = -1;
      for (int64_t k = 0; k < sz; ++k) {
        const int64_t i = order[(size_t)(f0 + k)];
        line[3 + pos[(size_t)i]] = live[(size_t)i];
      }
      ++n_fin;
      if (slot >= 0) P->drop(slot, log_block);
      continue;
    }
    if (slot < 0) {
      if (P->free.empty()) {  // evict the least recently written unprotected slot; its group is sealed
        int64_t victim = -1;
        int64_t best_last = 0;
        uint64_t best_stamp = 0;
        for (const auto& kv : P->slot_info) {
          if (protected_slot[(size_t)kv.first]) continue;
          const SlotInfo& si = kv.second;
          if (victim < 0 || si.last < best_last || (si.last == best_last && si.stamp < best_stamp)) {
            victim = kv.first; best_last = si.last; best_stamp = si.stamp;
          }
        }
        if (victim < 0)
          return set_error(ECHOKV_E_UNSUPPORTED, "more than %lld open K groups in one step", (long long)P->num_slots);
        const SlotInfo vi = P->slot_info.at(victim);
        int64_t* ev = evictions + 4 * n_evict++;
        ev[0] = victim; ev[1] = vi.block; ev[2] = vi.group; ev[3] = vi.fill;
        P->sealed[vi.block] |= (int64_t)1 << vi.group;
        P->drop(victim, log_block);
      }
      slot = P->free.back();
      P->free.pop_back();
      P->slot_info[slot] = SlotInfo{b, gr, 0, 0, P->stamp++};
      P->block_slot[b] = slot;
      protected_slot[(size_t)slot] = 1;
      log_block.put(b, slot);
      log_group.put(slot, gr);
    }
    for (int64_t k = 0; k < sz; ++k) tok_res[live[(size_t)order[(size_t)(f0 + k)]]] = slot;
    SlotInfo& si = P->slot_info.at(slot);
    si.fill = std::max(si.fill, top + 1);
    si.last = P->step;
  }

  // per touched block: highest offset written + 1, and how many tokens
  const int64_t n_touched = (int64_t)ublk.size();
  {
    std::unordered_map<int64_t, int64_t> idx;
    for (int64_t i = 0; i < n_touched; ++i) { touched[i] = ublk[(size_t)i]; touched_fill[i] = 0; touched_count[i] = 0; idx[ublk[(size_t)i]] = i; }
    for (int64_t i = 0; i < n; ++i) {
      const int64_t t = idx[blk[(size_t)i]];
      touched_fill[t] = std::max(touched_fill[t], off[(size_t)i] + 1);
      touched_count[t] += 1;
    }
  }

  // the last `kref_window` keys of the step go to the K_ref ring in order
  const int64_t k = std::min(n, P->kref_window);
  for (int64_t i = 0; i < k; ++i) tok_kref[live[(size_t)(n - k + i)]] = (P->kref_pos + i) % P->kref_window;
  if (k) {
    P->kref_pos = (P->kref_pos + k) % P->kref_window;
    P->kref_fill = std::min(P->kref_window, P->kref_fill + k);
  }

  for (size_t i = 0; i < open_b.size(); ++i) opened[i] = open_b[i];
  for (size_t i = 0; i < log_block.items.size(); ++i) { map_block[i] = log_block.items[i].first; map_value[i] = log_block.items[i].second; }
  for (size_t i = 0; i < log_group.items.size(); ++i) { grp_slot[i] = log_group.items[i].first; grp_value[i] = log_group.items[i].second; }
  counts[0] = n_fin; counts[1] = n_evict; counts[2] = (int64_t)open_b.size(); counts[3] = n_touched;
  counts[4] = (int64_t)log_block.items.size(); counts[5] = (int64_t)log_group.items.size(); counts[6] = P->step;
  return ECHOKV_OK;
}

}  // extern "C"
