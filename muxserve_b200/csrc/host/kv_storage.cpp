// Block allocator of the unified KV pool (host side).
//
// Observable behaviour follows KVStorage in the reference
// (csrc/memory_manager.cpp:4-157): a free list that hands out ids from its
// tail, request-keyed ownership, batch allocation that preempts the longest
// suffix of the batch whose blocks make the prefix fit, and the same return
// encodings and counters.  States in which the reference would read outside
// its own vectors (it carries no checks) are rejected here with an error and
// leave the allocator unchanged.
#include <cstdint>
#include <cstring>
#include <unordered_map>
#include <vector>

#include "../../../include/muxb200.h"

struct mux_kv_storage {
  int32_t num_blocks = 0;
  std::vector<int32_t> free_list;  // the back is handed out first
  std::unordered_map<int32_t, std::vector<int32_t>> owned;
  int32_t blocks_allocated = 0;      // running counter with the reference's accounting
  int32_t last_new_blocks = 0;       // new minus freed of the last batch call
};

namespace {

struct BatchPlan {
  std::vector<int64_t> want;         // blocks a request's row asks to see returned
  std::vector<int64_t> need;         // blocks to take from the free list (may be <= 0)
  std::vector<int64_t> held;         // blocks owned when the call started
  std::vector<int64_t> need_prefix;  // inclusive running sum of need
  std::vector<int64_t> want_prefix;  // exclusive running sum of want (size n+1)
  int32_t keep = 0;                  // requests [0, keep) are served, the rest preempted
};

// Sizes every row and finds how many leading requests can be served if the
// trailing ones give their blocks back (memory_manager.cpp:36-72).
BatchPlan plan_batch(const mux_kv_storage& s, const int32_t* info, int32_t n, int64_t per_block) {
  BatchPlan bp;
  bp.want.resize(n);
  bp.need.resize(n);
  bp.held.resize(n);
  bp.need_prefix.resize(n);
  bp.want_prefix.assign(n + 1, 0);
  int64_t run = 0;
  for (int32_t i = 0; i < n; ++i) {
    const int32_t id = info[3 * i];
    const bool has_blocks = info[3 * i + 2] != 0;
    auto it = s.owned.find(id);
    const int64_t holding = it == s.owned.end() ? 0 : (int64_t)it->second.size();
    bp.want[i] = (int64_t)info[3 * i + 1] * per_block;
    bp.held[i] = holding;
    // A request that says it has no blocks yet but is known is topped up to `want`.
    bp.need[i] = has_blocks ? bp.want[i] : bp.want[i] - holding;
    run += bp.need[i];
    bp.need_prefix[i] = run;
    bp.want_prefix[i + 1] = bp.want_prefix[i] + bp.want[i];
  }
  std::vector<int64_t> suffix_held(n + 1, 0);  // blocks held by requests [i, n)
  for (int32_t i = n - 1; i >= 0; --i) suffix_held[i] = suffix_held[i + 1] + bp.held[i];
  int32_t keep = n;
  const int64_t free_now = (int64_t)s.free_list.size();
  while (keep > 0 && bp.need_prefix[keep - 1] > free_now + suffix_held[keep]) --keep;
  bp.keep = keep;
  return bp;
}

}  // namespace

extern "C" {

mux_kv_storage_t* mux_kv_storage_create(int32_t num_blocks) {
  if (num_blocks < 0) return nullptr;
  auto* s = new mux_kv_storage();
  s->num_blocks = num_blocks;
  s->free_list.resize(num_blocks);
  for (int32_t i = 0; i < num_blocks; ++i) s->free_list[i] = i;
  return s;
}

void mux_kv_storage_destroy(mux_kv_storage_t* s) { delete s; }

int mux_kv_storage_allocate(mux_kv_storage_t* s, int32_t size, int32_t* out_ids) {
  if (s == nullptr) return MUX_ERR_BAD_HANDLE;
  if (size < 0 || (size > 0 && out_ids == nullptr)) return MUX_ERR_BAD_SHAPE;
  if ((size_t)size > s->free_list.size()) return MUX_ERR_BUFFER_TOO_SMALL;
  for (int32_t i = 0; i < size; ++i) {
    out_ids[i] = s->free_list.back();
    s->free_list.pop_back();
  }
  return MUX_OK;
}

int mux_kv_storage_allocate_batch(mux_kv_storage_t* s, const int32_t* info, int32_t n,
                                  int32_t num_layers, int32_t num_heads, int32_t* out,
                                  int64_t out_capacity, int64_t* out_len) {
  if (s == nullptr) return MUX_ERR_BAD_HANDLE;
  if (n < 0 || num_layers <= 0 || num_heads <= 0 || (n > 0 && info == nullptr) || out_len == nullptr)
    return MUX_ERR_BAD_SHAPE;
  const int64_t per_block = (int64_t)num_layers * num_heads;
  const BatchPlan bp = plan_batch(*s, info, n, per_block);
  const int32_t keep = bp.keep;
  const int64_t length = keep <= 0 ? 1 : 1 + bp.want_prefix[keep];
  *out_len = length;
  if (out == nullptr) return MUX_OK;  // size query: no state change
  if (out_capacity < length) return MUX_ERR_BUFFER_TOO_SMALL;

  // ---- checks for states the reference cannot handle; nothing is changed before they pass ----
  int64_t take_total = keep > 0 ? bp.need_prefix[keep - 1] : 0;
  if (keep > 0) {
    int64_t positive = 0;
    std::unordered_map<int32_t, int64_t> size_after;  // a request id may repeat in a batch
    for (int32_t i = 0; i < keep; ++i) {
      const int32_t id = info[3 * i];
      auto sa = size_after.find(id);
      int64_t cur = sa == size_after.end() ? bp.held[i] : sa->second;
      if (bp.need[i] > 0) {
        positive += bp.need[i];
        cur += bp.need[i];
      }
      size_after[id] = cur;
      if (bp.want[i] > cur || bp.want[i] < 0) return MUX_ERR_BAD_SHAPE;
    }
    if (take_total < 0 || positive != take_total) return MUX_ERR_BAD_SHAPE;
    // ids named both in the served prefix and the preempted suffix would be freed under their owner
    for (int32_t i = keep; i < n; ++i)
      if (bp.held[i] > 0 && size_after.count(info[3 * i])) return MUX_ERR_BAD_SHAPE;
  }

  // ---- preempt the suffix: its blocks return to the tail of the free list ----
  int64_t freed = 0;
  for (int32_t i = keep; i < n; ++i) {
    if (bp.held[i] <= 0) continue;
    freed += bp.held[i];
    auto it = s->owned.find(info[3 * i]);
    if (it != s->owned.end()) {
      s->free_list.insert(s->free_list.end(), it->second.begin(), it->second.end());
      s->owned.erase(it);
    }
  }
  s->blocks_allocated -= (int32_t)freed;
  s->last_new_blocks = -(int32_t)freed;
  out[0] = keep;
  if (keep <= 0) return MUX_OK;

  // ---- serve the prefix from the last take_total entries, in list order ----
  const size_t first = s->free_list.size() - (size_t)take_total;
  size_t cursor = first;
  int64_t w = 1;
  for (int32_t i = 0; i < keep; ++i) {
    std::vector<int32_t>& mine = s->owned[info[3 * i]];
    if (bp.need[i] > 0) {
      mine.insert(mine.end(), s->free_list.begin() + cursor,
                  s->free_list.begin() + cursor + (size_t)bp.need[i]);
      cursor += (size_t)bp.need[i];
    }
    if (bp.want[i] > 0) {
      std::memcpy(out + w, mine.data() + (mine.size() - (size_t)bp.want[i]),
                  (size_t)bp.want[i] * sizeof(int32_t));
      w += bp.want[i];
    }
  }
  s->free_list.resize(first);
  s->last_new_blocks += (int32_t)take_total;
  s->blocks_allocated += s->last_new_blocks;  // freed blocks are subtracted twice, as in the reference
  return MUX_OK;
}

int64_t mux_kv_storage_free_batch(mux_kv_storage_t* s, const int32_t* request_ids, int32_t n) {
  if (s == nullptr) return MUX_ERR_BAD_HANDLE;
  if (n < 0 || (n > 0 && request_ids == nullptr)) return MUX_ERR_BAD_SHAPE;
  int64_t freed = 0;
  for (int32_t i = 0; i < n; ++i) {
    auto it = s->owned.find(request_ids[i]);
    if (it == s->owned.end()) continue;  // unknown ids are ignored
    freed += (int64_t)it->second.size();
    s->free_list.insert(s->free_list.end(), it->second.begin(), it->second.end());
    s->owned.erase(it);
  }
  s->blocks_allocated -= (int32_t)freed;
  return freed;
}

int32_t mux_kv_storage_new_blocks_allocated(const mux_kv_storage_t* s) {
  return s ? s->last_new_blocks : 0;
}

int32_t mux_kv_storage_num_blocks_allocated(const mux_kv_storage_t* s) {
  return s ? s->blocks_allocated : 0;
}

int64_t mux_kv_storage_num_free(const mux_kv_storage_t* s) {
  return s ? (int64_t)s->free_list.size() : MUX_ERR_BAD_HANDLE;
}

int mux_kv_storage_free_list(const mux_kv_storage_t* s, int32_t* out, int64_t capacity) {
  if (s == nullptr) return MUX_ERR_BAD_HANDLE;
  if ((int64_t)s->free_list.size() > capacity) return MUX_ERR_BUFFER_TOO_SMALL;
  if (!s->free_list.empty())
    std::memcpy(out, s->free_list.data(), s->free_list.size() * sizeof(int32_t));
  return MUX_OK;
}

int mux_kv_storage_check(const mux_kv_storage_t* s) {
  if (s == nullptr) return MUX_ERR_BAD_HANDLE;
  std::vector<uint8_t> seen((size_t)s->num_blocks, 0);
  auto mark = [&](int32_t id) {
    if (id < 0 || id >= s->num_blocks || seen[(size_t)id]) return false;
    seen[(size_t)id] = 1;
    return true;
  };
  for (int32_t id : s->free_list)
    if (!mark(id)) return MUX_ERR_BAD_SHAPE;
  for (const auto& kv : s->owned)
    for (int32_t id : kv.second)
      if (!mark(id)) return MUX_ERR_BAD_SHAPE;
  for (uint8_t f : seen)
    if (!f) return MUX_ERR_BAD_SHAPE;
  return MUX_OK;
}

}  // extern "C"
