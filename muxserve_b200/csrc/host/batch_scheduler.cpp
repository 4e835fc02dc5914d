// Per-model step builder (host side): tracks every request's logical position
// and physical block table and emits the index tensors the kernels consume.
//
// Observable behaviour follows BatchScheduler / Request in the reference
// (csrc/batch_scheduler.h:9-106, csrc/batch_scheduler.cpp:5-199): the same
// try_batch rows, batch info, token / position / context_len / slot_mapping
// values and block-table entries.  Two deliberate differences: block-table
// entries past a request's physical blocks are written as 0 (the reference
// leaves them uninitialised), and ids / sizes are checked instead of trusted.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <memory>
#include <unordered_map>
#include <vector>

#include "../../../include/muxb200.h"

namespace {

struct Seq {
  int32_t id = 0;
  int32_t max_tokens = 0;
  int32_t context_len = 0;
  int32_t phys_blocks = 0;   // physical blocks granted so far (per layer-head)
  int32_t logical_idx = 0;   // index of the logical block holding the last token
  int32_t logical_off = 0;   // offset of the last token inside it
  std::vector<int32_t> prompt;
  std::vector<int32_t> outputs;
  std::vector<int32_t> table;  // [max_blocks][L][H]
};

}  // namespace

struct mux_batch_scheduler {
  int32_t L = 0, H = 0, max_seq_len = 0, block = 0, max_blocks = 0;
  std::unordered_map<int32_t, std::unique_ptr<Seq>> seqs;
  std::vector<int32_t> preempted;
  std::vector<int32_t> prompt_info;
  std::vector<int32_t> batch_reqs;  // pairs

  Seq* find(int32_t id) const {
    auto it = seqs.find(id);
    return it == seqs.end() ? nullptr : it->second.get();
  }
};

namespace {

// Shared body of the two get_batch forms.  `layered` selects the block-table
// layout: false = [token, block, L, H] (reference), true = [L, seq, H, block].
int build_batch(mux_batch_scheduler* b, const int32_t* req, int32_t n, const int32_t* block_info,
                int64_t block_info_len, int32_t* tokens, int32_t* positions, int32_t padded_len,
                int32_t* context_lens, int32_t num_contexts, int32_t* block_tables,
                int64_t block_tables_len, int64_t* slot_mapping, int64_t slot_mapping_len,
                bool layered) {
  if (b == nullptr) return MUX_ERR_BAD_HANDLE;
  if (n < 0 || block_info == nullptr || block_info_len < 1 || (n > 0 && req == nullptr))
    return MUX_ERR_BAD_SHAPE;
  const int32_t keep = std::min(block_info[0], n);
  const int64_t LH = (int64_t)b->L * b->H;

  // ---- pass 1: sizes, and everything that can fail, before any state changes ----
  int64_t num_tokens = 0, num_ctx = 0;
  int32_t max_blocks_per_seq = 0;
  bool any_prefill = false;
  for (int32_t i = 0; i < std::max(keep, 0); ++i) {
    const Seq* s = b->find(req[3 * i]);
    if (s == nullptr) return MUX_ERR_UNKNOWN_REQUEST;
    if (!s->outputs.empty()) {
      if (s->phys_blocks < 1) return MUX_ERR_BAD_SHAPE;  // a decode row needs a block to write to
      max_blocks_per_seq = std::max(max_blocks_per_seq, s->phys_blocks);
      num_tokens += 1;
      num_ctx += 1;
    } else {
      any_prefill = true;
      if ((int64_t)(s->prompt.size() + b->block - 1) / b->block > s->phys_blocks)
        return MUX_ERR_BAD_SHAPE;  // prompt slots would index blocks never granted
      num_tokens += (int64_t)s->prompt.size();
    }
  }
  if (layered && any_prefill) return MUX_ERR_BAD_SHAPE;
  if (num_tokens > padded_len || num_ctx > num_contexts) return MUX_ERR_BUFFER_TOO_SMALL;
  if (num_tokens * LH > slot_mapping_len) return MUX_ERR_BUFFER_TOO_SMALL;
  const int64_t table_len = num_tokens * max_blocks_per_seq * LH;
  if (table_len > block_tables_len) return MUX_ERR_BUFFER_TOO_SMALL;
  if ((num_tokens > 0 && (!tokens || !positions || !slot_mapping)) ||
      (num_ctx > 0 && !context_lens) || (table_len > 0 && !block_tables))
    return MUX_ERR_NULL_POINTER;
  if (max_blocks_per_seq > 0) {
    // the table holds one row per token, rows [0, keep) are written (batch_scheduler.cpp:159-168)
    if (keep > num_tokens) return MUX_ERR_BAD_SHAPE;
    for (int32_t i = 0; i < keep; ++i)
      if (b->find(req[3 * i])->phys_blocks > max_blocks_per_seq) return MUX_ERR_BAD_SHAPE;
  }

  // ---- pass 2 ----
  b->preempted.clear();
  b->prompt_info.clear();
  b->batch_reqs.clear();
  int64_t tok = 0, ctx_i = 0, slot_i = 0;
  int32_t max_context_len = 0;
  for (int32_t i = 0; i < n; ++i) {
    const int32_t id = req[3 * i];
    if (i >= keep) {  // preempted by the allocator: forget the request
      b->preempted.push_back(id);
      b->seqs.erase(id);
      continue;
    }
    Seq* s = b->find(id);
    if (!s->outputs.empty()) {
      tokens[tok] = s->outputs.back();
      positions[tok] = s->context_len - 1;
      context_lens[ctx_i++] = s->context_len;
      max_context_len = std::max(max_context_len, s->context_len);
      const int32_t* last = s->table.data() + (int64_t)(s->phys_blocks - 1) * LH;
      for (int64_t j = 0; j < LH; ++j)
        slot_mapping[slot_i++] = (int64_t)last[j] * b->block + s->logical_off;
      tok += 1;
    } else {
      const int64_t plen = (int64_t)s->prompt.size();
      for (int64_t t = 0; t < plen; ++t) {
        tokens[tok + t] = s->prompt[(size_t)t];
        positions[tok + t] = (int32_t)t;
        const int32_t* blk = s->table.data() + (t / b->block) * LH;
        const int64_t off = t % b->block;
        for (int64_t j = 0; j < LH; ++j) slot_mapping[slot_i++] = (int64_t)blk[j] * b->block + off;
      }
      b->prompt_info.push_back((int32_t)plen);
      tok += plen;
    }
    b->batch_reqs.push_back(id);
    b->batch_reqs.push_back(s->max_tokens);
  }
  b->prompt_info.push_back(max_context_len);
  for (int64_t t = tok; t < padded_len; ++t) tokens[t] = positions[t] = 0;

  if (max_blocks_per_seq > 0) {
    std::memset(block_tables, 0, (size_t)table_len * sizeof(int32_t));
    const int64_t S = num_tokens;
    for (int32_t i = 0; i < keep; ++i) {
      const Seq* s = b->find(req[3 * i]);
      const int64_t cnt = (int64_t)s->phys_blocks * LH;
      if (!layered) {
        std::memcpy(block_tables + (int64_t)i * max_blocks_per_seq * LH, s->table.data(),
                    (size_t)cnt * sizeof(int32_t));
      } else {
        for (int32_t l = 0; l < b->L; ++l)
          for (int32_t h = 0; h < b->H; ++h) {
            int32_t* dst = block_tables + (((int64_t)l * S + i) * b->H + h) * max_blocks_per_seq;
            const int32_t* src = s->table.data() + (int64_t)l * b->H + h;
            for (int32_t j = 0; j < s->phys_blocks; ++j) dst[j] = src[(int64_t)j * LH];
          }
      }
    }
  }
  return MUX_OK;
}

int32_t copy_out(const std::vector<int32_t>& v, int32_t* out, int32_t capacity) {
  const int32_t n = (int32_t)v.size();
  if (out != nullptr && capacity > 0)
    std::memcpy(out, v.data(), (size_t)std::min(n, capacity) * sizeof(int32_t));
  return n;
}

}  // namespace

extern "C" {

mux_batch_scheduler_t* mux_batch_scheduler_create(int32_t num_layers, int32_t num_heads,
                                                  int32_t max_seq_len, int32_t block_size) {
  if (num_layers <= 0 || num_heads <= 0 || max_seq_len <= 0 || block_size <= 0) return nullptr;
  auto* b = new mux_batch_scheduler();
  b->L = num_layers;
  b->H = num_heads;
  b->max_seq_len = max_seq_len;
  b->block = block_size;
  b->max_blocks = (max_seq_len + block_size - 1) / block_size;
  return b;
}

void mux_batch_scheduler_destroy(mux_batch_scheduler_t* b) { delete b; }

int mux_batch_scheduler_add_request(mux_batch_scheduler_t* b, const int32_t* prompt,
                                    int32_t prompt_len, int32_t req_id, int32_t max_tokens) {
  if (b == nullptr) return MUX_ERR_BAD_HANDLE;
  if (prompt_len < 0 || (prompt_len > 0 && prompt == nullptr)) return MUX_ERR_BAD_SHAPE;
  auto s = std::make_unique<Seq>();
  s->id = req_id;
  s->max_tokens = max_tokens;
  s->prompt.assign(prompt, prompt + prompt_len);
  s->context_len = prompt_len;
  // integer forms of batch_scheduler.h:25-27 (C++ division truncates towards zero)
  s->logical_idx = (prompt_len + b->block - 1) / b->block - 1;
  s->logical_off = (prompt_len - 1) % b->block;
  s->table.assign((size_t)b->max_blocks * b->L * b->H, 0);
  b->seqs[req_id] = std::move(s);  // re-adding an id starts it from scratch
  return MUX_OK;
}

int mux_batch_scheduler_try_batch(mux_batch_scheduler_t* b, const int32_t* req_ids, int32_t n,
                                  const int32_t* last_tokens, int32_t n_last, int32_t* out) {
  if (b == nullptr) return MUX_ERR_BAD_HANDLE;
  if (n < 0 || n_last < 0 || out == nullptr || (n > 0 && req_ids == nullptr)) return MUX_ERR_BAD_SHAPE;
  const bool decoding = n_last > 0;
  if (decoding && (n_last < n || last_tokens == nullptr)) return MUX_ERR_BAD_SHAPE;
  for (int32_t i = 0; i < n; ++i)
    if (b->find(req_ids[i]) == nullptr) return MUX_ERR_UNKNOWN_REQUEST;
  int32_t total = 0;
  for (int32_t i = 0; i < n; ++i) {
    Seq* s = b->find(req_ids[i]);
    int32_t needed;
    if (decoding) {
      // the new token is accounted for before the allocator has answered
      s->outputs.push_back(last_tokens[i]);
      s->context_len += 1;
      if (++s->logical_off == b->block) {
        s->logical_off = 0;
        s->logical_idx += 1;
      }
      needed = s->logical_idx + 1 - s->phys_blocks;
    } else {
      needed = s->logical_idx + 1;
    }
    out[3 * i] = s->id;
    out[3 * i + 1] = needed;
    out[3 * i + 2] = std::min(s->phys_blocks, 1);
    total += needed;
  }
  out[3 * n] = total;
  return MUX_OK;
}

int mux_batch_scheduler_get_batch_info(mux_batch_scheduler_t* b, const int32_t* req, int32_t n,
                                       const int32_t* block_info, int64_t block_info_len,
                                       int32_t* out, int32_t out_capacity, int32_t* out_len) {
  if (b == nullptr) return MUX_ERR_BAD_HANDLE;
  if (n < 0 || block_info == nullptr || block_info_len < 1 || out == nullptr || out_len == nullptr ||
      (n > 0 && req == nullptr))
    return MUX_ERR_BAD_SHAPE;
  const int32_t keep = std::min(block_info[0], n);
  const int64_t LH = (int64_t)b->L * b->H;
  // everything that can fail first
  int64_t consumed = 1;
  int32_t prompts = 0;
  for (int32_t i = 0; i < keep; ++i) {
    const Seq* s = b->find(req[3 * i]);
    if (s == nullptr) return MUX_ERR_UNKNOWN_REQUEST;
    const int64_t grant = (int64_t)req[3 * i + 1] * LH;
    if (grant > 0) {
      consumed += grant;
      if ((int64_t)s->phys_blocks + req[3 * i + 1] > b->max_blocks) return MUX_ERR_TOO_LARGE;
    }
    if (s->outputs.empty()) ++prompts;
  }
  if (consumed > block_info_len) return MUX_ERR_BAD_SHAPE;
  *out_len = 6 + prompts;
  if (out_capacity < 6 + prompts) return MUX_ERR_BUFFER_TOO_SMALL;

  int32_t num_tokens = 0, num_contexts = 0, max_context_len = 0, max_blocks_per_seq = 0;
  int64_t cursor = 1;
  int32_t w = 6;
  for (int32_t i = 0; i < keep; ++i) {
    Seq* s = b->find(req[3 * i]);
    const int64_t grant = (int64_t)req[3 * i + 1] * LH;
    if (grant > 0) {
      std::memcpy(s->table.data() + (int64_t)s->phys_blocks * LH, block_info + cursor,
                  (size_t)grant * sizeof(int32_t));
      cursor += grant;
      s->phys_blocks += req[3 * i + 1];
    }
    if (!s->outputs.empty()) {
      max_blocks_per_seq = std::max(max_blocks_per_seq, s->phys_blocks);
      max_context_len = std::max(max_context_len, s->context_len);
      num_contexts += 1;
      num_tokens += 1;
    } else {
      out[w++] = (int32_t)s->prompt.size();
      num_tokens += (int32_t)s->prompt.size();
    }
  }
  out[0] = num_tokens;
  out[1] = num_contexts;
  out[2] = max_context_len;
  out[3] = max_blocks_per_seq;
  out[4] = b->L;
  out[5] = b->H;
  return MUX_OK;
}

int mux_batch_scheduler_get_batch(mux_batch_scheduler_t* b, const int32_t* req, int32_t n,
                                  const int32_t* block_info, int64_t block_info_len,
                                  int32_t* tokens, int32_t* positions, int32_t padded_len,
                                  int32_t* context_lens, int32_t num_contexts,
                                  int32_t* block_tables, int64_t block_tables_len,
                                  int64_t* slot_mapping, int64_t slot_mapping_len) {
  return build_batch(b, req, n, block_info, block_info_len, tokens, positions, padded_len,
                     context_lens, num_contexts, block_tables, block_tables_len, slot_mapping,
                     slot_mapping_len, false);
}

int mux_batch_scheduler_get_batch_decode_layered(
    mux_batch_scheduler_t* b, const int32_t* req, int32_t n, const int32_t* block_info,
    int64_t block_info_len, int32_t* tokens, int32_t* positions, int32_t padded_len,
    int32_t* context_lens, int32_t num_contexts, int32_t* block_tables, int64_t block_tables_len,
    int64_t* slot_mapping, int64_t slot_mapping_len) {
  return build_batch(b, req, n, block_info, block_info_len, tokens, positions, padded_len,
                     context_lens, num_contexts, block_tables, block_tables_len, slot_mapping,
                     slot_mapping_len, true);
}

int mux_batch_scheduler_release_requests(mux_batch_scheduler_t* b, const int32_t* req_ids, int32_t n) {
  if (b == nullptr) return MUX_ERR_BAD_HANDLE;
  if (n < 0 || (n > 0 && req_ids == nullptr)) return MUX_ERR_BAD_SHAPE;
  for (int32_t i = 0; i < n; ++i) b->seqs.erase(req_ids[i]);
  return MUX_OK;
}

int32_t mux_batch_scheduler_preempt_requests(const mux_batch_scheduler_t* b, int32_t* out, int32_t capacity) {
  return b ? copy_out(b->preempted, out, capacity) : MUX_ERR_BAD_HANDLE;
}

int32_t mux_batch_scheduler_prompt_info(const mux_batch_scheduler_t* b, int32_t* out, int32_t capacity) {
  return b ? copy_out(b->prompt_info, out, capacity) : MUX_ERR_BAD_HANDLE;
}

int32_t mux_batch_scheduler_batch_reqs(const mux_batch_scheduler_t* b, int32_t* out, int32_t capacity) {
  return b ? copy_out(b->batch_reqs, out, capacity) : MUX_ERR_BAD_HANDLE;
}

int mux_batch_scheduler_request_state(const mux_batch_scheduler_t* b, int32_t req_id, int32_t out[5]) {
  if (b == nullptr) return MUX_ERR_BAD_HANDLE;
  const Seq* s = b->find(req_id);
  if (s == nullptr) return MUX_ERR_UNKNOWN_REQUEST;
  out[0] = s->context_len;
  out[1] = s->phys_blocks;
  out[2] = s->logical_idx;
  out[3] = s->logical_off;
  out[4] = (int32_t)s->outputs.size();
  return MUX_OK;
}

int mux_batch_scheduler_get_batch_mixed(const mux_mixed_model_t* models, int32_t num_models, int32_t tp,
                                        int32_t tp_rank, int32_t max_blocks, int32_t* item_context_len,
                                        int32_t* item_q_row, int32_t* item_group, float* item_scale,
                                        int32_t* block_tables, int64_t block_tables_len, mux_mixed_span_t* spans,
                                        int32_t* totals) {
  if (models == nullptr || spans == nullptr || totals == nullptr) return MUX_ERR_NULL_POINTER;
  if (num_models <= 0 || tp < 1 || tp_rank < 0 || tp_rank >= tp || max_blocks < 0) return MUX_ERR_BAD_SHAPE;
  // ---- everything that can fail, and the sizes ----
  std::vector<int32_t> order((size_t)num_models);
  for (int32_t m = 0; m < num_models; ++m) {
    const mux_mixed_model_t& md = models[m];
    if (md.scheduler == nullptr) return MUX_ERR_BAD_HANDLE;
    if (md.num_requests < 0 || (md.num_requests > 0 && md.request_ids == nullptr)) return MUX_ERR_BAD_SHAPE;
    const int32_t H = md.scheduler->H;
    if (md.num_q_heads <= 0 || md.num_q_heads % H != 0 || md.num_q_heads / H > 8) return MUX_ERR_BAD_GROUP;
    for (int32_t i = 0; i < md.num_requests; ++i) {
      const Seq* sq = md.scheduler->find(md.request_ids[i]);
      if (sq == nullptr) return MUX_ERR_UNKNOWN_REQUEST;
      if (sq->outputs.empty() || sq->phys_blocks < 1) return MUX_ERR_BAD_SHAPE;  // decode rows only
      if (sq->phys_blocks > max_blocks) return MUX_ERR_BUFFER_TOO_SMALL;
    }
    order[(size_t)m] = m;
  }
  // deepest model first: the models that still have layer l are always a prefix of the items and rows
  std::stable_sort(order.begin(), order.end(),
                   [&](int32_t a, int32_t b) { return models[a].scheduler->L > models[b].scheduler->L; });
  int64_t items = 0, rows = 0;
  int32_t max_layers = 0, max_ctx = 0, max_group = 1;
  for (int32_t k = 0; k < num_models; ++k) {
    const mux_mixed_model_t& md = models[order[(size_t)k]];
    mux_mixed_span_t& sp = spans[k];
    sp.model = order[(size_t)k];
    sp.first_item = (int32_t)items;
    sp.num_items = md.num_requests * md.scheduler->H;
    sp.first_row = (int32_t)rows;
    sp.num_rows = md.num_requests * md.num_q_heads * tp;
    sp.num_layers = md.scheduler->L;
    items += sp.num_items;
    rows += sp.num_rows;
    max_layers = std::max(max_layers, sp.num_layers);
    max_group = std::max(max_group, md.num_q_heads / md.scheduler->H);
  }
  if (items > 0x7fffffffLL || rows > 0x7fffffffLL) return MUX_ERR_TOO_LARGE;
  totals[0] = (int32_t)items;
  totals[1] = (int32_t)rows;
  totals[2] = max_layers;
  totals[3] = max_group;
  if (block_tables == nullptr) {  // sizing call
    totals[4] = 0;
    return MUX_OK;
  }
  if (!item_context_len || !item_q_row || !item_group || !item_scale) return MUX_ERR_NULL_POINTER;
  if ((int64_t)max_layers * items * max_blocks > block_tables_len) return MUX_ERR_BUFFER_TOO_SMALL;
  std::memset(block_tables, 0, (size_t)((int64_t)max_layers * items * max_blocks) * sizeof(int32_t));
  for (int32_t k = 0; k < num_models; ++k) {
    const mux_mixed_model_t& md = models[spans[k].model];
    const mux_batch_scheduler* b = md.scheduler;
    const int32_t H = b->H, G = md.num_q_heads / H;
    const int64_t LH = (int64_t)b->L * H;
    for (int32_t i = 0; i < md.num_requests; ++i) {
      const Seq* sq = b->find(md.request_ids[i]);
      max_ctx = std::max(max_ctx, sq->context_len);
      for (int32_t h = 0; h < H; ++h) {
        const int64_t item = spans[k].first_item + (int64_t)i * H + h;
        item_context_len[item] = sq->context_len;
        // this rank's heads sit at their global position inside the model's [S, tp * local heads] rows
        item_q_row[item] = spans[k].first_row + i * (md.num_q_heads * tp) + tp_rank * md.num_q_heads + h * G;
        item_group[item] = G;
        item_scale[item] = md.scale;
        for (int32_t l = 0; l < b->L; ++l) {
          int32_t* dst = block_tables + ((int64_t)l * items + item) * max_blocks;
          const int32_t* src = sq->table.data() + (int64_t)l * H + h;
          for (int32_t j = 0; j < sq->phys_blocks; ++j) dst[j] = src[(int64_t)j * LH];
        }
      }
    }
  }
  totals[4] = max_ctx;
  return MUX_OK;
}

}  // extern "C"
