// Definitions shared by the attention kernels: launch parameters, per-item
// lookup and the q / out row resolution of one head tile.
#pragma once
#include <cstdint>

#include "internal.h"
#include "ptx.cuh"
#include "rope.cuh"

namespace mux {

constexpr int kHeadSize = 128;
constexpr int kConsumerWarps = 4;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;  // + producer warp
constexpr int kMaxStages = 16;
constexpr int kRedStride = kHeadSize + 4;  // padded row of the cross-warp reduction
constexpr int kMaxSmemBytes = 227 * 1024;
constexpr int kMaxDevicesTracked = 64;

struct AttnParams {
  const void* q;
  void* out;
  const void* kc;
  const void* vc;
  const int* block_tables;
  const int* context_lens;
  const int* head_mapping;
  const int* seq_rows;   // optional: row of each sequence in a persistent block table
  const int* item_ctx;
  const int* item_q_row;
  const int* item_group;
  const float* item_scale;
  long long q_s0, q_s1, o_s0, o_s1;  // single model: seq, head strides; mixed: s1 = row stride
  long long bt_s0, bt_s1;            // single model: seq, head strides; mixed: s0 = item stride
  float* ws_acc;
  float* ws_ml;
  unsigned* status;
  long long num_blocks;
  float scale;
  int num_q_heads, num_kv_heads, group;
  int gs;          // head columns kept in shared memory (1..8)
  int head_tiles;  // ceil(group / 8)
  int pb;          // partition size in blocks
  int max_parts;
  int max_context_len;
  int nst;         // ring depth in tiles
  int prod_lanes;  // lanes of the producer warp that issue tiles (divides nst)
  // fused cache write (decode step): the new token's K/V rows, one per (sequence, kv head)
  const void* k_new;
  const void* v_new;
  long long kn_s0, kn_s1, vn_s0, vn_s1;  // single model: seq, head strides; mixed: s0 = item (row) stride
  int new_tokens;                        // fused decode step: rows appended per (sequence, kv head), 1..16
  const void* rope_cache;                // fused decode step only: [max_position][64 cos | 64 sin], or nullptr
  long long rope_max_position;
  long long num_items;                   // (sequence, kv head) items of the launch
  const int* units;                      // optional list of item | partition << 24, one CTA each
  int flags;                             // MUX_ATTN_* bits of the call
#ifdef MUX_TRACE
  unsigned long long* trace;             // scratch builds only: clock64 stamps of CTA 0
#endif
};

// Scratch builds (-DMUX_TRACE) stamp the phases of CTA 0 with clock64; product builds compile this away.
#ifdef MUX_TRACE
#define MUX_TRACE_AT(slot, who)                                                   \
  do {                                                                            \
    if (p.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == (who)) p.trace[slot] = clock64(); \
  } while (0)
#else
#define MUX_TRACE_AT(slot, who) \
  do {                          \
  } while (0)
#endif

// Shared-memory carve-up, identical on host (sizing) and device.
struct SmemLayout {
  int ring, s, ids, newrows, info, bars, total;
  int srow;
};

__host__ __device__ inline SmemLayout smem_layout(int block_size, int pb, int gs, int nst) {
  SmemLayout L;
  const int tile = kHeadSize * block_size * 2;
  const int P = pb * block_size;
  L.srow = P + 16;  // rows 64 bytes apart modulo 128: conflict-free 16-byte reads of the weights
  int off = 0;
  L.ring = off;
  off += nst * tile;
  L.s = off;
  int s_bytes = gs * L.srow * 4;
  int red_bytes = kConsumerWarps * gs * kRedStride * 4;
  off += (s_bytes > red_bytes ? s_bytes : red_bytes);
  off = (off + 15) & ~15;
  L.ids = off;
  off += pb * 4;
  off = (off + 15) & ~15;
  L.newrows = off;   // fused decode step: the new K row (256 B) and V row (256 B), staged by the producer warp
  off += 512;
  L.info = off;
  off += 8 * 8 + 8 * 8 + 8 * 2 * 4 + 16;  // qoff, ooff, ml, geff
  L.bars = off;
  off += (2 * kMaxStages + 1) * 8;  // full[], empty[], and one barrier for the staged new rows
  L.total = off;
  return L;
}

struct ItemInfo {
  long long qoff[8];
  long long ooff[8];
  float ml[8][2];
  int geff;
  int pad[3];
};

struct ItemDesc {
  int ctx, G, seq, kvh;
  float scale;
  const int* bt_row;
};

template <bool MIXED>
__device__ __forceinline__ ItemDesc load_item(const AttnParams& p, int item) {
  ItemDesc d;
  if (MIXED) {
    d.ctx = p.item_ctx[item];
    d.G = p.item_group[item];
    d.scale = p.item_scale[item];
    d.bt_row = p.block_tables + (long long)item * p.bt_s0;
    d.seq = 0;
    d.kvh = 0;
  } else {
    d.seq = item / p.num_kv_heads;
    d.kvh = item - d.seq * p.num_kv_heads;
    d.ctx = p.context_lens[d.seq];
    d.G = p.group;
    d.scale = p.scale;
    const long long row = p.seq_rows != nullptr ? p.seq_rows[d.seq] : d.seq;
    d.bt_row = p.block_tables + row * p.bt_s0 + (long long)d.kvh * p.bt_s1;
  }
  return d;
}

// Executed by one full warp: element offsets of the (up to 8) q / out rows of
// this head tile, and how many of them exist.
template <bool MIXED>
__device__ __forceinline__ void resolve_heads(const AttnParams& p, const ItemDesc& d, int item,
                                              int htile, ItemInfo* info, int lane) {
  if (MIXED) {
    if (lane < 8) {
      long long row = (long long)p.item_q_row[item] + htile * 8 + lane;
      info->qoff[lane] = row * p.q_s1;
      info->ooff[lane] = row * p.o_s1;
    }
    if (lane == 0) {
      // Shared memory holds p.gs head columns: a group read from device data never widens the tile.
      if (d.G < 1 || d.G > p.gs * p.head_tiles) atomicOr(p.status, MUX_DEV_BAD_GROUP);
      info->geff = max(0, min(p.gs, d.G - htile * 8));
    }
  } else if (p.head_mapping == nullptr) {
    if (lane < 8) {
      long long hq = (long long)d.kvh * d.G + htile * 8 + lane;
      info->qoff[lane] = (long long)d.seq * p.q_s0 + hq * p.q_s1;
      info->ooff[lane] = (long long)d.seq * p.o_s0 + hq * p.o_s1;
    }
    if (lane == 0) info->geff = max(0, min(p.gs, d.G - htile * 8));
  } else {
    // General head_mapping: ordered compaction of the q heads mapped to this kv head.
    int count = 0;
    for (int base = 0; base < p.num_q_heads; base += 32) {
      int hq = base + lane;
      bool match = hq < p.num_q_heads && p.head_mapping[hq] == d.kvh;
      unsigned bal = __ballot_sync(0xffffffffu, match);
      int pos = count + __popc(bal & ((1u << lane) - 1u)) - htile * 8;
      if (match && pos >= 0 && pos < 8) {
        info->qoff[pos] = (long long)d.seq * p.q_s0 + (long long)hq * p.q_s1;
        info->ooff[pos] = (long long)d.seq * p.o_s0 + (long long)hq * p.o_s1;
      }
      count += __popc(bal);
    }
    if (lane == 0) {
      if (count != d.G) atomicOr(p.status, MUX_DEV_BAD_HEAD_MAPPING);
      // A kv head given more q heads than the group keeps only the first `group` of them (status bit above):
      // the tile never grows beyond the p.gs columns that shared memory and the workspace were sized for.
      info->geff = max(0, min(p.gs, min(count, d.G) - htile * 8));
    }
  }
}

}  // namespace mux
