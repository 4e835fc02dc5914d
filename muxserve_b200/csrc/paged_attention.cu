// Decode-phase paged attention over a head-granular unified KV pool (sm_100a).
//
// Work unit = one partition (<= partition_size tokens) of one (sequence, kv head)
// item.  One CTA per unit: a producer warp walks the item's block list and
// streams every 16-token K block and V block (head_size*block_size*2 bytes, one
// contiguous piece of the pool) into a shared-memory ring with 1-D bulk (TMA)
// copies completed on mbarriers; four consumer warps take the staged blocks in
// turn.  The grouped query heads of the item (1 for MHA, up to 8 for GQA) form
// the N=8 dimension of m16n8k16 tensor-core MMAs whose M dimension is the 16
// tokens of a block: the pool's own layouts, K [d/8][token][8] and V [d][token],
// are exactly the row-major A operands of K.Q^T and V^T.P^T, so the staged
// bytes are used as they arrive.
//
//   phase 1  logits[h][t] = scale * K[t,:] . q[h,:]   for all K blocks of the unit
//   softmax  over the unit (max, exp, sum); the weights stay fp32 in place of the logits
//            and are split into hi + lo parts of the KV dtype when they are loaded as MMA
//            operands (two MMAs per tile: fp32-level accuracy of P with 16-bit operands)
//   phase 2  out^T[d][h] += V^T[d,t] P^T[t,h]         for all V blocks of the unit
//
// A unit that covers its whole context writes `out`; otherwise it writes an
// un-normalised fp32 partial (acc, max, sum) to the workspace and a second
// small kernel merges the partitions (flash-decoding).
#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <mutex>

#include "attn_common.cuh"

namespace mux {

constexpr int kMergeWarps = 4;
constexpr int kMergeChunk = 128;  // partitions whose weights are staged at a time

// One warp merges the partitions of one q head of one (item, head tile): the lanes reduce (max, sum)
// over the partitions, turn them into one weight per partition (staged in `wts`, kMergeChunk floats of
// shared memory owned by the warp) and then each lane accumulates four output elements from 16-byte
// loads, eight partitions in flight.
template <typename T>
__device__ __forceinline__ void merge_one(const AttnParams& p, long long slot0, int n, int nparts, long long ooff,
                                          float* wts, int lane) {
  // Everything a warp needs comes from L2, and what costs is the number of DEPENDENT round trips, not the bytes
  // (this kernel sits between two attention launches): lane k takes partition k's (max, sum) pair in one 8-byte
  // load, and the accumulators of the first eight partitions are requested at the same time — they do not depend
  // on the weights.  Items with more than 32 partitions take the general path for the rest.
  const float* src = p.ws_acc + (slot0 * p.gs + n) * kHeadSize + 4 * lane;
  const long long stride = (long long)p.gs * kHeadSize;
  float2 ml0 = make_float2(-INFINITY, 0.f);
  if (lane < nparts) ml0 = __ldcg(reinterpret_cast<const float2*>(p.ws_ml + ((slot0 + lane) * p.gs + n) * 2));
  constexpr int kPre = 8;
  float4 pre[kPre];
#pragma unroll
  for (int k = 0; k < kPre; ++k)
    if (k < nparts) pre[k] = __ldcg(reinterpret_cast<const float4*>(src + k * stride));
  float M = ml0.x;
  for (int k = lane + 32; k < nparts; k += 32) M = fmaxf(M, __ldcg(p.ws_ml + ((slot0 + k) * p.gs + n) * 2));
  M = warp_max(M);
  float lsum = ml0.y * __expf(ml0.x - M);  // lanes past nparts: 0 * exp(-inf) = 0
  for (int k = lane + 32; k < nparts; k += 32) {
    const long long r = (slot0 + k) * p.gs + n;
    lsum += __ldcg(p.ws_ml + r * 2 + 1) * __expf(__ldcg(p.ws_ml + r * 2) - M);
  }
  lsum = warp_sum(lsum);
  const float inv = 1.f / lsum;
  const float w_lane = __expf(ml0.x - M) * inv;  // weight of partition `lane`
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const int head = min(nparts, 32);
#pragma unroll
  for (int k = 0; k < kPre; ++k) {
    const float w = __shfl_sync(0xffffffffu, w_lane, k);
    if (k < head) {
      acc.x = fmaf(w, pre[k].x, acc.x);
      acc.y = fmaf(w, pre[k].y, acc.y);
      acc.z = fmaf(w, pre[k].z, acc.z);
      acc.w = fmaf(w, pre[k].w, acc.w);
    }
  }
#pragma unroll 8
  for (int k = kPre; k < head; ++k) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(src + k * stride));
    const float w = __shfl_sync(0xffffffffu, w_lane, k);
    acc.x = fmaf(w, a.x, acc.x);
    acc.y = fmaf(w, a.y, acc.y);
    acc.z = fmaf(w, a.z, acc.z);
    acc.w = fmaf(w, a.w, acc.w);
  }
  for (int k0 = 32; k0 < nparts; k0 += kMergeChunk) {
    const int cnt = min(kMergeChunk, nparts - k0);
    for (int k = lane; k < cnt; k += 32) wts[k] = __expf(__ldcg(p.ws_ml + ((slot0 + k0 + k) * p.gs + n) * 2) - M) * inv;
    __syncwarp();
#pragma unroll 8
    for (int k = 0; k < cnt; ++k) {
      const float4 a = __ldcg(reinterpret_cast<const float4*>(src + (k0 + k) * stride));
      const float w = wts[k];
      acc.x = fmaf(w, a.x, acc.x);
      acc.y = fmaf(w, a.y, acc.y);
      acc.z = fmaf(w, a.z, acc.z);
      acc.w = fmaf(w, a.w, acc.w);
    }
    __syncwarp();
  }
  T* dst = static_cast<T*>(p.out) + ooff + 4 * lane;
  const T o0 = from_float<T>(acc.x), o1 = from_float<T>(acc.y), o2 = from_float<T>(acc.z), o3 = from_float<T>(acc.w);
  if ((reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
    uint2 w;
    w.x = (uint32_t)(*reinterpret_cast<const unsigned short*>(&o0)) | ((uint32_t)(*reinterpret_cast<const unsigned short*>(&o1)) << 16);
    w.y = (uint32_t)(*reinterpret_cast<const unsigned short*>(&o2)) | ((uint32_t)(*reinterpret_cast<const unsigned short*>(&o3)) << 16);
    *reinterpret_cast<uint2*>(dst) = w;
  } else {
    dst[0] = o0;
    dst[1] = o1;
    dst[2] = o2;
    dst[3] = o3;
  }
}

// FUSE != 0: the call is a whole decode step, the new tokens' K/V rows are appended by the launch itself.
//   1  one new token per sequence (what the reference's decode step appends): the CTA that owns the item's last
//      partition patches the staged copy of the last K and V block in shared memory with the new rows, so the
//      attention sees them, and writes them to the pool; the rows reach shared memory beside the KV stream.
//   2  several new tokens: the producer warp of the CTA whose partition holds their positions writes the rows
//      into the pool first (rotary applied to K) and only then issues the bulk copies of the blocks that received
//      them; about 1 us more on that CTA's path, no extra shared memory whatever the token count.
template <typename T, int BS, bool MIXED, int FUSE>
__global__ void __launch_bounds__(kThreads, 6)  // six CTAs per SM: at most 64 registers per thread
paged_attn_kernel(const __grid_constant__ AttnParams p) {
  constexpr int TILE = kHeadSize * BS * 2;       // bytes of one K or V block
  constexpr int MT = BS >= 16 ? BS / 16 : 1;     // 16-token m-tiles per K block
  constexpr int KSTEPS = BS >= 16 ? BS / 16 : 1; // 16-token k-steps per V block
  constexpr int CHUNK = BS * 16;                 // bytes of one 8-wide d chunk row of K
  constexpr int VROW = BS * 2;                   // bytes of one d row of V

  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int item = blockIdx.x, part = blockIdx.y;
  const int htile = blockIdx.z;
  if (p.units != nullptr) {  // the host listed the real (item, partition) pairs
    const int u = p.units[blockIdx.x];
    if (u < 0) return;  // padding of a list kept at a fixed length (launch dimensions frozen in a CUDA graph)
    item = u & 0xffffff;
    part = (int)((unsigned)u >> 24);
    if (item >= p.num_items) {  // a list that does not belong to this launch: nothing is read through it
      if (threadIdx.x == 0) atomicOr(p.status, MUX_DEV_BAD_CONTEXT);
      return;
    }
  }
  const int P = p.pb * BS;
  MUX_TRACE_AT(0, 0);

  // Programmatic dependent launch.  Normally nothing is read before every earlier kernel of the stream
  // has completed.  With MUX_ATTN_EARLY_KV the caller vouches that the launch's index data and the KV
  // blocks it names are not being written by the kernels just ahead of it, so this CTA resolves its item,
  // fetches its block ids and fills its ring with the first KV blocks while those kernels drain; only
  // q, the new K/V rows and every write (pool, workspace, out) stay behind the wait.
  const bool early = (p.flags & MUX_ATTN_EARLY_KV) != 0;
  if (!early) {
    griddep_wait();
    griddep_launch_dependents();  // the next kernel may start being scheduled behind this grid
  }
  ItemDesc d = load_item<MIXED>(p, item);
  // The producer warp asks for the partition's first 32 block ids at once, before the context length
  // has arrived: entries below ceil(max_context_len / BS) exist in every block list whatever its length
  // (unused ones may hold anything and are dropped below), so the two loads overlap.
  int spec_id = 0;
  if (warp == kConsumerWarps && lane < p.pb && part * p.pb + lane < (p.max_context_len + BS - 1) / BS)
    spec_id = d.bt_row[part * p.pb + lane];
  if (d.ctx < 0 || d.ctx > p.max_context_len || (FUSE == 2 && d.ctx > 0 && d.ctx < p.new_tokens)) {
    if (tid == 0) atomicOr(p.status, MUX_DEV_BAD_CONTEXT);  // (a decode step's context counts its new tokens)
    d.ctx = d.ctx < 0 ? 0 : min(max(d.ctx, FUSE == 2 ? p.new_tokens : 0), p.max_context_len);
  }
  const int nparts = (d.ctx + P - 1) / P;
  if (part >= nparts && !(d.ctx == 0 && part == 0)) return;

  const SmemLayout L = smem_layout(BS, p.pb, p.gs, p.nst);
  ItemInfo* info = reinterpret_cast<ItemInfo*>(smem + L.info);
  const uint32_t bars = smem_u32(smem + L.bars);  // full[i] at +8i, empty[i] at +8(kMaxStages+i)
  const int nst = p.nst;

  if (warp == 0) resolve_heads<MIXED>(p, d, item, htile, info, lane);
  if (tid == kConsumerThreads) {
    for (int i = 0; i < nst; ++i) {
      mbar_init(bars + 8 * i, 1);
      mbar_init(bars + 8 * (kMaxStages + i), 1);
    }
    mbar_init(bars + 8 * (2 * kMaxStages), 1);  // the staged new rows are in shared memory
    mbar_init_fence();
  }
  __syncthreads();
  MUX_TRACE_AT(1, 0);

  const int geff = info->geff;
  if (geff <= 0) return;
  T* out = static_cast<T*>(p.out);
  if (d.ctx == 0) {  // empty context: defined output (zeros), nothing to attend to
    if (early) {
      griddep_wait();
      griddep_launch_dependents();
    }
    if (tid < kHeadSize)
      for (int n = 0; n < geff; ++n) out[info->ooff[n] + tid] = from_float<T>(0.f);
    return;
  }

  const int tok0 = part * P;
  const int ntok = min(d.ctx - tok0, P);
  const int nblk = (ntok + BS - 1) / BS;
  const uint32_t ring = smem_u32(smem + L.ring);

  if (warp == kConsumerWarps) {
    // ---------------- producer warp ----------------
    int* ids = reinterpret_cast<int*>(smem + L.ids);
    for (int i = lane; i < nblk; i += 32) {
      int id = i < 32 ? spec_id : d.bt_row[part * p.pb + i];
      if (id < 0 || id >= p.num_blocks) {
        atomicOr(p.status, MUX_DEV_BAD_BLOCK_ID);
        id = -1;  // block 0 is read in its place; nothing is ever written through it
      }
      ids[i] = id;
    }
    __syncwarp();
    MUX_TRACE_AT(10, kConsumerThreads);
    const unsigned char* kc = static_cast<const unsigned char*>(p.kc);
    const unsigned char* vc = static_cast<const unsigned char*>(p.vc);
    const int ntiles = 2 * nblk;
    const int first = min(ntiles, nst);  // the ring's first filling needs no free-stage wait
    const int nl = p.prod_lanes;         // lanes that issue tiles (a divisor of nst): lane l takes tiles l, l + nl, ...
    // FUSE == 2: the new tokens' positions that fall into this partition, [lo, hi), and the first block they touch.
    // In the ring's first filling (any order is fine there) the tiles of earlier blocks go out at once; those of
    // the blocks that receive new rows follow when the rows are in the pool.
    int lo = 0, hi = 0;
    if (FUSE == 2) {
      lo = max(d.ctx - p.new_tokens, tok0);
      hi = min(d.ctx, tok0 + ntok);
    }
    const bool has_new = FUSE == 2 && lo < hi;
    const int jb_new = has_new ? (lo - tok0) / BS : nblk;
    if (lane < nl) {
      for (int j = lane; j < first; j += nl) {
        const int jb = j < nblk ? j : j - nblk;
        if (jb >= jb_new) continue;
        const unsigned char* src = (j < nblk ? kc : vc) + (long long)max(ids[jb], 0) * TILE;
        mbar_arrive_expect_tx(bars + 8 * j, TILE);
        bulk_g2s(ring + j * TILE, src, TILE, bars + 8 * j);
      }
    }
    __syncwarp();
    MUX_TRACE_AT(11, kConsumerThreads);
    if (early) {
      griddep_wait();
      griddep_launch_dependents();
    }
    if (has_new) {
      // ---- append: K rows as 16 pieces of 16 bytes (two rows per pass, one per half-warp), V rows as 128 single
      // elements (the pool keeps V token-minor), four per lane ----
      const int first_new = d.ctx - p.new_tokens;
      const int half = lane >> 4, l = lane & 15;
      unsigned char* kcw = static_cast<unsigned char*>(const_cast<void*>(p.kc));
      unsigned short* vcw = reinterpret_cast<unsigned short*>(const_cast<void*>(p.vc));
      for (int r0 = lo; r0 < hi; r0 += 2) {
        const bool live = r0 + half < hi;
        const int r = live ? r0 + half : hi - 1;  // the idle half still takes part in the shuffles of the rotation
        const long long row = MIXED ? ((long long)item * p.new_tokens + (r - first_new)) * p.kn_s0
                                    : ((long long)d.seq * p.new_tokens + (r - first_new)) * p.kn_s0 + (long long)d.kvh * p.kn_s1;
        uint4 knew = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.k_new) + row + 8 * l);
        if (p.rope_cache != nullptr) {
          const long long pos = min((long long)r, p.rope_max_position - 1);
          knew = rope_row16<T>(knew, l, static_cast<const T*>(p.rope_cache) + pos * kHeadSize);
        }
        const int id = ids[(r - tok0) / BS];
        if (live && id >= 0)
          *reinterpret_cast<uint4*>(kcw + (long long)id * TILE + l * CHUNK + ((r - tok0) % BS) * 16) = knew;
      }
      for (int r = lo; r < hi; ++r) {
        const long long row = MIXED ? ((long long)item * p.new_tokens + (r - first_new)) * p.vn_s0
                                    : ((long long)d.seq * p.new_tokens + (r - first_new)) * p.vn_s0 + (long long)d.kvh * p.vn_s1;
        const uint2 vnew = *reinterpret_cast<const uint2*>(static_cast<const T*>(p.v_new) + row + 4 * lane);
        const int id = ids[(r - tok0) / BS];
        if (id >= 0) {
          unsigned short* dst = vcw + (long long)id * (TILE / 2) + (4 * lane) * BS + (r - tok0) % BS;
          dst[0] = (unsigned short)(vnew.x & 0xffffu);
          dst[BS] = (unsigned short)(vnew.x >> 16);
          dst[2 * BS] = (unsigned short)(vnew.y & 0xffffu);
          dst[3 * BS] = (unsigned short)(vnew.y >> 16);
        }
      }
      // the rows must be in the pool before the bulk copies (another proxy) of their blocks read it: every lane
      // orders its own writes before later async-proxy accesses, the warp barrier carries that to the issuing lanes
      fence_proxy_async_global();
      __syncwarp();
    }
    if (has_new && lane < nl) {
      for (int j = lane; j < first; j += nl) {
        const int jb = j < nblk ? j : j - nblk;
        if (jb < jb_new) continue;
        const unsigned char* src = (j < nblk ? kc : vc) + (long long)max(ids[jb], 0) * TILE;
        mbar_arrive_expect_tx(bars + 8 * j, TILE);
        bulk_g2s(ring + j * TILE, src, TILE, bars + 8 * j);
      }
    }
    if (FUSE == 1 && part == nparts - 1 && lane >= 16) {
      // The upper half-warp brings the decode step's new K/V rows of this item to shared memory (rotary
      // applied to K) while lane 0 keeps issuing tiles; the consumer warp that appends them waits on
      // their barrier.
      const int l = lane - 16;
      const long long ko = MIXED ? (long long)item * p.kn_s0 : (long long)d.seq * p.kn_s0 + (long long)d.kvh * p.kn_s1;
      const long long vo = MIXED ? (long long)item * p.vn_s0 : (long long)d.seq * p.vn_s0 + (long long)d.kvh * p.vn_s1;
      uint4 knew = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.k_new) + ko + 8 * l);
      const uint4 vnew = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.v_new) + vo + 8 * l);
      if (p.rope_cache != nullptr) {
        long long pos = min((long long)d.ctx - 1, p.rope_max_position - 1);
        knew = rope_row16<T>(knew, l, static_cast<const T*>(p.rope_cache) + pos * kHeadSize, 0xffff0000u);
      }
      unsigned char* nr = smem + L.newrows;
      *reinterpret_cast<uint4*>(nr + 16 * l) = knew;
      *reinterpret_cast<uint4*>(nr + 256 + 16 * l) = vnew;
      __syncwarp(0xffff0000u);
      if (l == 0) mbar_arrive(bars + 8 * (2 * kMaxStages));
    }
    if (lane < nl) {
      // tiles nst + lane, nst + lane + nl, ...: stage and the parity of its previous use are kept incrementally
      int stage = lane;
      uint32_t parity = 0;
      for (int j = nst + lane; j < ntiles; j += nl) {
        const long long bid = max(ids[j < nblk ? j : j - nblk], 0);
        const unsigned char* src = (j < nblk ? kc : vc) + bid * TILE;
        mbar_wait(bars + 8 * (kMaxStages + stage), parity, p.status, MUX_DEV_WAIT_TIMEOUT);
        mbar_arrive_expect_tx(bars + 8 * stage, TILE);
        bulk_g2s(ring + stage * TILE, src, TILE, bars + 8 * stage);
        stage += nl;
        if (stage >= nst) {
          stage -= nst;
          parity ^= 1u;
        }
      }
    }
    MUX_TRACE_AT(12, kConsumerThreads);
    return;
  }

  // ---------------- consumer warps ----------------
  if (early) {  // q (and everything written below) may depend on the kernels ahead
    griddep_wait();
    griddep_launch_dependents();
  }
  const int g = lane >> 2, tq = lane & 3;
  float* S = reinterpret_cast<float*>(smem + L.s);
  const int SROW = L.srow;

  // FUSE: the warp that consumes the block holding the new token also appends it (the producer warp
  // has staged the new rows in shared memory by then).
  const int new_local = d.ctx - 1 - tok0;  // the appended token's index inside this partition
  const int jl = new_local / BS, ol = new_local % BS;
  const bool appends = FUSE == 1 && part == nparts - 1 && (jl & (kConsumerWarps - 1)) == warp;
  const int* ids_c = reinterpret_cast<const int*>(smem + L.ids);
  // Rotary embedding of the decode step: the query and the new key sit at position ctx - 1.
  const T* rope_row = nullptr;
  if (FUSE && p.rope_cache != nullptr) {
    long long pos = d.ctx - 1;
    if (pos >= p.rope_max_position) {
      if (tid == 0) atomicOr(p.status, MUX_DEV_BAD_CONTEXT);
      pos = p.rope_max_position - 1;
    }
    rope_row = static_cast<const T*>(p.rope_cache) + pos * kHeadSize;
  }
  // q as the B operand (k = d, n = head): b0 = q[g][16ks + 2tq, +1], b1 = q[g][16ks + 8 + 2tq, +1]
  uint32_t qf[8][2];
  {
    const T* q = static_cast<const T*>(p.q);
    if (g < geff) {
      const T* qr = q + info->qoff[g];
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        qf[ks][0] = ldg32_nc(qr + ks * 16 + 2 * tq);
        qf[ks][1] = ldg32_nc(qr + ks * 16 + 8 + 2 * tq);
      }
      if (FUSE && rope_row != nullptr) {  // element d < 64 is in qf[ks][r], its partner d + 64 in qf[ks + 4][r]
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int dd = ks * 16 + r * 8 + 2 * tq;
            rope_words<T>(qf[ks][r], qf[ks + 4][r], ldg32_nc(rope_row + dd), ldg32_nc(rope_row + 64 + dd));
          }
      }
    } else {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) qf[ks][0] = qf[ks][1] = 0u;
    }
  }

  MUX_TRACE_AT(2, 0);
  // ---- phase 1: logits ----
  {
    const int n0 = 2 * tq;
    const int lm_tok = (lane & 7) + (BS >= 16 ? ((lane >> 3) & 1) * 8 : 0);
    const int lm_chunk = lane >> 4;
    for (int jb = warp; jb < nblk; jb += kConsumerWarps) {
      const int stage = jb % nst, use = jb / nst;
      mbar_wait(bars + 8 * stage, use & 1, p.status, MUX_DEV_WAIT_TIMEOUT);
      if (jb == 0) MUX_TRACE_AT(3, 0);
      const uint32_t tile = ring + stage * TILE;
      if (FUSE == 1 && appends && jb == jl) {  // K row of the new token: 16 pieces of 16 bytes
        mbar_wait(bars + 8 * (2 * kMaxStages), 0, p.status, MUX_DEV_WAIT_TIMEOUT);
        if (lane < 16) {
          const uint4 knew = *reinterpret_cast<const uint4*>(smem + L.newrows + 16 * lane);
          const uint32_t off = lane * CHUNK + ol * 16;
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(tile + off), "r"(knew.x), "r"(knew.y),
                       "r"(knew.z), "r"(knew.w) : "memory");
          if (ids_c[jl] >= 0)
            *reinterpret_cast<uint4*>(static_cast<unsigned char*>(const_cast<void*>(p.kc)) +
                                      (long long)ids_c[jl] * TILE + off) = knew;
        }
        fence_proxy_async_smem();
        __syncwarp();
      }
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          uint32_t a[4];
          ldmatrix_x4(a, tile + (2 * ks + lm_chunk) * CHUNK + (mt * 16 + lm_tok) * 16);
          mma_16816<T>(c, a, qf[ks][0], qf[ks][1]);
        }
        const int tok = jb * BS + mt * 16 + g;
        if (n0 < geff) {
          S[n0 * SROW + tok] = c[0] * d.scale;
          if (BS >= 16) S[n0 * SROW + tok + 8] = c[2] * d.scale;
        }
        if (n0 + 1 < geff) {
          S[(n0 + 1) * SROW + tok] = c[1] * d.scale;
          if (BS >= 16) S[(n0 + 1) * SROW + tok + 8] = c[3] * d.scale;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * (kMaxStages + stage));
    }
  }
  MUX_TRACE_AT(4, 0);
  named_bar_sync(1, kConsumerThreads);
  MUX_TRACE_AT(5, 0);

  // ---- softmax over the unit ----
  for (int n = warp; n < geff; n += kConsumerWarps) {
    const float* srow = S + n * SROW;
    float m = -INFINITY;
    for (int t = lane; t < ntok; t += 32) m = fmaxf(m, srow[t]);
    m = warp_max(m);
    float l = 0.f;
    float* prow = S + n * SROW;  // exp(logit - max) overwrites the logit
    for (int t = lane; t < nblk * BS; t += 32) {
      const float pv = t < ntok ? __expf(srow[t] - m) : 0.f;
      l += pv;
      prow[t] = pv;
    }
    l = warp_sum(l);
    if (lane == 0) {
      info->ml[n][0] = m;
      info->ml[n][1] = l;
    }
  }
  named_bar_sync(1, kConsumerThreads);
  MUX_TRACE_AT(6, 0);

  // ---- phase 2: out^T[d][h] = sum_t V^T[d][t] P^T[t][h] ----
  float acc[8][4];
#pragma unroll
  for (int mt = 0; mt < 8; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
  {
    const bool lane_has = (BS >= 16) || (tq < 2);
    for (int jb = warp; jb < nblk; jb += kConsumerWarps) {
      const int j = nblk + jb;
      const int stage = j % nst, use = j / nst;
      mbar_wait(bars + 8 * stage, use & 1, p.status, MUX_DEV_WAIT_TIMEOUT);
      if (jb == 0) MUX_TRACE_AT(7, 0);
      const uint32_t tile = ring + stage * TILE;
      if (FUSE == 1 && appends && jb == jl) {  // V column of the new token: 128 single elements
        const uint2 vnew = *reinterpret_cast<const uint2*>(smem + L.newrows + 256 + 8 * lane);
        const unsigned short e[4] = {(unsigned short)(vnew.x & 0xffffu), (unsigned short)(vnew.x >> 16),
                                     (unsigned short)(vnew.y & 0xffffu), (unsigned short)(vnew.y >> 16)};
        unsigned short* gdst = reinterpret_cast<unsigned short*>(
            static_cast<unsigned char*>(const_cast<void*>(p.vc)) + (long long)max(ids_c[jl], 0) * TILE);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t off = (4 * lane + i) * VROW + ol * 2;
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(tile + off), "h"(e[i]) : "memory");
          if (ids_c[jl] >= 0) gdst[off >> 1] = e[i];
        }
        fence_proxy_async_smem();
        __syncwarp();
      }
      const int rem = ntok - jb * BS;  // valid tokens of this block
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        // This lane's four tokens of the k-step: slots {2tq,2tq+1} and {8+2tq,9+2tq}
        // of the MMA are tokens t0..t0+3 (same mapping in A and B).
        const int t0 = ks * 16 + 4 * tq;
        uint32_t b0 = 0u, b1 = 0u, c0 = 0u, c1 = 0u;
        if (g < geff && lane_has) {
          const float4 pw = *reinterpret_cast<const float4*>(S + g * SROW + jb * BS + t0);
          split_pair<T>(pw.x, pw.y, b0, c0);
          split_pair<T>(pw.z, pw.w, b1, c1);
        }
        uint32_t mlo = 0xffffffffu, mhi = 0xffffffffu;
        if (rem < BS) {  // stale tail of the last block may hold anything, NaN included
          mlo = (t0 < rem ? 0x0000ffffu : 0u) | (t0 + 1 < rem ? 0xffff0000u : 0u);
          mhi = (t0 + 2 < rem ? 0x0000ffffu : 0u) | (t0 + 3 < rem ? 0xffff0000u : 0u);
        }
        if (!lane_has) mlo = mhi = 0u;
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
          const int row = mt * 16 + g;
          uint2 r0 = lds64(tile + row * VROW + t0 * 2);
          uint2 r1 = lds64(tile + (row + 8) * VROW + t0 * 2);
          uint32_t a[4] = {r0.x & mlo, r1.x & mlo, r0.y & mhi, r1.y & mhi};
          mma_16816<T>(acc[mt], a, b0, b1);
          mma_16816<T>(acc[mt], a, c0, c1);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + 8 * (kMaxStages + stage));
    }
  }

  MUX_TRACE_AT(8, 0);
  // ---- cross-warp reduction.  It reuses the buffer of the softmax weights, which the other
  // warps may still be reading: wait for all of them to finish phase 2 first.
  named_bar_sync(1, kConsumerThreads);
  float* red = S;
  {
    const int n0 = 2 * tq;
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      const int d0 = mt * 16 + g;
      if (n0 < geff) {
        red[(warp * p.gs + n0) * kRedStride + d0] = acc[mt][0];
        red[(warp * p.gs + n0) * kRedStride + d0 + 8] = acc[mt][2];
      }
      if (n0 + 1 < geff) {
        red[(warp * p.gs + n0 + 1) * kRedStride + d0] = acc[mt][1];
        red[(warp * p.gs + n0 + 1) * kRedStride + d0 + 8] = acc[mt][3];
      }
    }
  }
  named_bar_sync(1, kConsumerThreads);
  {
    const int dd = tid;  // 0..127
    const long long slot = ((long long)item * p.head_tiles + htile) * p.max_parts + part;
    for (int n = 0; n < geff; ++n) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) s += red[(w * p.gs + n) * kRedStride + dd];
      if (nparts == 1) {
        out[info->ooff[n] + dd] = from_float<T>(s / info->ml[n][1]);
      } else {
        p.ws_acc[(slot * p.gs + n) * kHeadSize + dd] = s;
        if (dd == 0) {
          p.ws_ml[(slot * p.gs + n) * 2] = info->ml[n][0];
          p.ws_ml[(slot * p.gs + n) * 2 + 1] = info->ml[n][1];
        }
      }
    }
  }
  MUX_TRACE_AT(9, 0);
}

// Merges the partitions of every item that has more than one: one warp per (item, head tile, q head of
// the group), see merge_one.
template <typename T, int BS, bool MIXED>
__global__ void __launch_bounds__(kMergeWarps * 32)
paged_attn_merge_kernel(const __grid_constant__ AttnParams p) {
  __shared__ ItemInfo infos[kMergeWarps];
  __shared__ float wts[kMergeWarps][kMergeChunk];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int P = p.pb * BS;
  // The kernel behind this one may be scheduled at once: every kernel of this library waits for its predecessors
  // itself before it touches what they write.  Ahead of its own wait this kernel reads at most the launch's index
  // data (context lengths, head mappings), and only when the caller has said that the kernels ahead do not write it.
  griddep_launch_dependents();
  const bool early = (p.flags & MUX_ATTN_EARLY_KV) != 0;  // index data is not written by the kernels just ahead
  if (!early) griddep_wait();
  const long long unit = (long long)blockIdx.x * kMergeWarps + warp;
  if (unit >= p.num_items * p.head_tiles * p.gs) return;
  const int n = (int)(unit % p.gs);
  const long long ih = unit / p.gs;
  const int htile = (int)(ih % p.head_tiles);
  const int item = (int)(ih / p.head_tiles);
  ItemDesc d = load_item<MIXED>(p, item);
  if (d.ctx < 0) d.ctx = 0;
  if (d.ctx > p.max_context_len) d.ctx = p.max_context_len;
  const int nparts = (d.ctx + P - 1) / P;
  if (nparts <= 1) return;
  ItemInfo* info = &infos[warp];
  resolve_heads<MIXED>(p, d, item, htile, info, lane);
  __syncwarp();
  if (n >= info->geff) return;
  if (early) griddep_wait();  // the partial results and `out` belong to the attention kernel ahead
  const long long slot0 = ((long long)item * p.head_tiles + htile) * p.max_parts;
  merge_one<T>(p, slot0, n, nparts, info->ooff[n], wts[warp], lane);
}

// ------------------------------------------------------------------ host side

#ifdef MUX_TRACE
static unsigned long long* g_trace_ptr = nullptr;
}  // namespace mux
extern "C" void mux_debug_set_trace(void* p) { mux::g_trace_ptr = static_cast<unsigned long long*>(p); }
namespace mux {
#endif

struct Plan {
  int pb, max_parts, gs, head_tiles, nst, smem;
  size_t ws_acc_bytes, ws_ml_bytes;
  size_t total() const { return ws_acc_bytes + ws_ml_bytes; }
};

static int default_stages(int block_size, int gs) {
  // 32 KiB of staged blocks per CTA; 16 KiB for grouped heads, whose logits and softmax
  // weights already take tens of KiB (more resident CTAs beat a deeper ring there).
  int tile = kHeadSize * block_size * 2;
  int n = ((gs > 2 ? 16 : 32) * 1024) / tile;
  return std::max(kConsumerWarps, std::min(kMaxStages, n));
}

static Plan make_plan(long long items, int group, int block_size, int max_context_len,
                      int partition_size, int num_stages) {
  Plan pl;
  int psize = partition_size > 0 ? partition_size : 512;
  psize = std::max(block_size, (psize / block_size) * block_size);
  pl.pb = psize / block_size;
  pl.max_parts = std::max(1, (max_context_len + psize - 1) / psize);
  pl.gs = std::min(8, std::max(1, group));
  pl.head_tiles = (std::max(1, group) + 7) / 8;
  // The ring depth must be a multiple of the consumer-warp count: then every
  // stage is always consumed by the same warp, whose mbarrier parity waits are
  // therefore never more than one phase apart.
  pl.nst = num_stages > 0 ? num_stages : default_stages(block_size, pl.gs);
  pl.nst = std::min(kMaxStages, std::max(kConsumerWarps, (pl.nst / kConsumerWarps) * kConsumerWarps));
  pl.smem = smem_layout(block_size, pl.pb, pl.gs, pl.nst).total;
  if (pl.max_parts > 1) {
    size_t slots = (size_t)items * pl.head_tiles * pl.max_parts * pl.gs;
    pl.ws_acc_bytes = slots * kHeadSize * sizeof(float);
    pl.ws_ml_bytes = slots * 2 * sizeof(float);
  } else {
    pl.ws_acc_bytes = pl.ws_ml_bytes = 0;
  }
  return pl;
}

static int plan_limits(const Plan& pl, long long items) {
  if (pl.smem > kMaxSmemBytes) return MUX_ERR_BAD_SHAPE;  // partition too large for one SM
  if (items > 0x7fffffffLL || pl.max_parts > 65535) return MUX_ERR_BAD_SHAPE;
  return MUX_OK;
}

struct DeviceInfo {
  int sms = 0;
};
static int device_info(int* dev_out, DeviceInfo* info) {
  static DeviceInfo cache[kMaxDevicesTracked];
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return record_cuda_error(e);
  if (dev < 0 || dev >= kMaxDevicesTracked) return record_cuda_error(cudaErrorInvalidDevice);
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev].sms == 0) {
    e = cudaDeviceGetAttribute(&cache[dev].sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return record_cuda_error(e);
  }
  *dev_out = dev;
  *info = cache[dev];
  return MUX_OK;
}

template <typename K>
static int ensure_smem(K kern, int smem, int dev, int* granted) {
  if (granted[dev] < smem) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return record_cuda_error(e);
    granted[dev] = smem;
  }
  return MUX_OK;
}

template <typename T, int BS, bool MIXED, int FUSE>
static int launch_typed(AttnParams& prm, const Plan& pl, long long items, cudaStream_t stream, int num_units) {
  int dev = 0;
  DeviceInfo di;
  int st = device_info(&dev, &di);
  if (st != MUX_OK) return st;
  cudaError_t e;
  auto kern = paged_attn_kernel<T, BS, MIXED, FUSE>;
  static int granted[kMaxDevicesTracked] = {};  // per instantiation, per device
  if ((st = ensure_smem(kern, pl.smem, dev, granted)) != MUX_OK) return st;
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = prm.units != nullptr ? dim3((unsigned)num_units, 1u, (unsigned)pl.head_tiles)
                                     : dim3((unsigned)items, (unsigned)pl.max_parts, (unsigned)pl.head_tiles);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = (size_t)pl.smem;
  cfg.stream = stream;
  cfg.attrs = pdl;
  cfg.numAttrs = 1;
  prm.num_items = items;
#ifdef MUX_TRACE
  prm.trace = g_trace_ptr;
  if (const char* e = getenv("MUX_PROD_LANES")) prm.prod_lanes = atoi(e);
#endif
  if ((e = cudaLaunchKernelEx(&cfg, kern, prm)) != cudaSuccess) return record_cuda_error(e);
  if (pl.max_parts > 1) {
    static bool carve[kMaxDevicesTracked] = {};
    if (!carve[dev]) {  // same shared-memory carve-out as the main kernel: no SM reconfiguration between them
      cudaFuncSetAttribute(paged_attn_merge_kernel<T, BS, MIXED>, cudaFuncAttributePreferredSharedMemoryCarveout,
                           cudaSharedmemCarveoutMaxShared);
      carve[dev] = true;
    }
    const long long units = items * pl.head_tiles * pl.gs;
    cfg.gridDim = dim3((unsigned)((units + kMergeWarps - 1) / kMergeWarps));
    cfg.blockDim = dim3(kMergeWarps * 32);
    cfg.dynamicSmemBytes = 0;
    if ((e = cudaLaunchKernelEx(&cfg, paged_attn_merge_kernel<T, BS, MIXED>, prm)) != cudaSuccess)
      return record_cuda_error(e);
  }
  return MUX_OK;
}

template <bool MIXED>
static int launch(AttnParams& prm, const Plan& pl, long long items, int dtype, int block_size,
                  cudaStream_t stream, int num_units = 0) {
  const int fuse = prm.k_new == nullptr ? 0 : (prm.new_tokens > 1 ? 2 : 1);
#define MUX_CASE(T, BS)                                                                \
  return fuse == 0   ? launch_typed<T, BS, MIXED, 0>(prm, pl, items, stream, num_units) \
         : fuse == 1 ? launch_typed<T, BS, MIXED, 1>(prm, pl, items, stream, num_units) \
                     : launch_typed<T, BS, MIXED, 2>(prm, pl, items, stream, num_units)
  if (dtype == MUX_DTYPE_F16) {
    if (block_size == 8) MUX_CASE(__half, 8);
    if (block_size == 16) MUX_CASE(__half, 16);
    MUX_CASE(__half, 32);
  } else {
    if (block_size == 8) MUX_CASE(__nv_bfloat16, 8);
    if (block_size == 16) MUX_CASE(__nv_bfloat16, 16);
    MUX_CASE(__nv_bfloat16, 32);
  }
#undef MUX_CASE
}

// Splits the caller's workspace into the two partial arrays.
static void bind_workspace(AttnParams& prm, const Plan& pl, void* workspace) {
  char* base = static_cast<char*>(workspace);
  prm.ws_acc = pl.ws_acc_bytes ? reinterpret_cast<float*>(base) : nullptr;
  prm.ws_ml = pl.ws_ml_bytes ? reinterpret_cast<float*>(base + pl.ws_acc_bytes) : nullptr;
}

static int check_common(int dtype, int head_size, int block_size) {
  if (dtype != MUX_DTYPE_F16 && dtype != MUX_DTYPE_BF16) return MUX_ERR_BAD_DTYPE;
  if (head_size != kHeadSize) return MUX_ERR_BAD_HEAD_SIZE;
  if (block_size != 8 && block_size != 16 && block_size != 32) return MUX_ERR_BAD_BLOCK_SIZE;
  return MUX_OK;
}

static int validate(const mux_attn_args_t* a) {
  if (a == nullptr) return MUX_ERR_NULL_POINTER;
  int st = check_common(a->dtype, a->head_size, a->block_size);
  if (st != MUX_OK) return st;
  if (a->num_seqs < 0 || a->num_q_heads <= 0 || a->num_kv_heads <= 0 || a->max_context_len < 0 ||
      a->num_blocks <= 0 || a->partition_size < 0 || a->num_stages < 0 || (a->flags & ~MUX_ATTN_EARLY_KV) != 0)
    return MUX_ERR_BAD_SHAPE;
  if (a->partition_size % a->block_size != 0) return MUX_ERR_BAD_SHAPE;
  if (a->num_q_heads % a->num_kv_heads != 0) return MUX_ERR_BAD_GROUP;
  if (a->num_seqs == 0) return MUX_OK;
  if (!a->out || !a->q || !a->key_cache || !a->value_cache || !a->block_tables || !a->context_lens)
    return MUX_ERR_NULL_POINTER;
  if (!aligned16(a->key_cache) || !aligned16(a->value_cache) || !aligned16(a->q) || !aligned16(a->out))
    return MUX_ERR_MISALIGNED;
  // q rows are staged with 16-byte bulk copies: every row must start on a 16-byte boundary.
  if ((a->q_seq_stride & 7) || (a->q_head_stride & 7)) return MUX_ERR_MISALIGNED;
  if (a->bt_seq_stride < 0 || a->bt_head_stride < 0) return MUX_ERR_BAD_SHAPE;
  return MUX_OK;
}

static int validate(const mux_attn_mixed_args_t* a) {
  if (a == nullptr) return MUX_ERR_NULL_POINTER;
  int st = check_common(a->dtype, a->head_size, a->block_size);
  if (st != MUX_OK) return st;
  if (a->num_items < 0 || a->max_context_len < 0 || a->num_blocks <= 0 || a->partition_size < 0 ||
      a->num_stages < 0 || (a->flags & ~MUX_ATTN_EARLY_KV) != 0)
    return MUX_ERR_BAD_SHAPE;
  if (a->partition_size % a->block_size != 0) return MUX_ERR_BAD_SHAPE;
  if (a->max_group < 1 || a->max_group > 8) return MUX_ERR_BAD_GROUP;
  if (a->num_items == 0) return MUX_OK;
  if (!a->out || !a->q || !a->key_cache || !a->value_cache || !a->block_tables ||
      !a->item_context_len || !a->item_q_row || !a->item_group || !a->item_scale)
    return MUX_ERR_NULL_POINTER;
  if (!aligned16(a->key_cache) || !aligned16(a->value_cache) || !aligned16(a->q) || !aligned16(a->out))
    return MUX_ERR_MISALIGNED;
  if (a->q_row_stride & 7) return MUX_ERR_MISALIGNED;
  if (a->bt_item_stride < 0) return MUX_ERR_BAD_SHAPE;
  return MUX_OK;
}

static Plan plan_of(const mux_attn_args_t* a) {
  return make_plan((long long)a->num_seqs * a->num_kv_heads, a->num_q_heads / a->num_kv_heads,
                   a->block_size, a->max_context_len, a->partition_size, a->num_stages);
}

static Plan plan_of(const mux_attn_mixed_args_t* a) {
  return make_plan(a->num_items, a->max_group, a->block_size, a->max_context_len, a->partition_size,
                   a->num_stages);
}

static int check_workspace(const Plan& pl, const void* workspace, size_t workspace_bytes) {
  const size_t need = pl.total();
  if (need > 0 && (workspace == nullptr || workspace_bytes < need)) return MUX_ERR_WORKSPACE_TOO_SMALL;
  if (need > 0 && !aligned16(workspace)) return MUX_ERR_MISALIGNED;
  return MUX_OK;
}

}  // namespace mux

extern "C" {

size_t mux_paged_attention_workspace_size(const mux_attn_args_t* a) {
  if (mux::validate(a) != MUX_OK || a->num_seqs == 0) return 0;
  return mux::plan_of(a).total();
}

}  // extern "C"

namespace mux {

struct NewRows {  // the decode step's new K/V rows; k == nullptr: plain attention
  const void* k = nullptr;
  const void* v = nullptr;
  long long k_s0 = 0, k_s1 = 0, v_s0 = 0, v_s1 = 0;
  const void* rope_cache = nullptr;   // optional rotary embedding of q and the new k
  long long rope_max_position = 0;
  int new_tokens = 1;                 // rows per (sequence, kv head)
};

static int validate_new_rows(const NewRows& n) {
  if (n.k == nullptr && n.v == nullptr) return MUX_OK;
  if (n.k == nullptr || n.v == nullptr) return MUX_ERR_NULL_POINTER;
  if (!aligned16(n.k) || !aligned16(n.v)) return MUX_ERR_MISALIGNED;
  if ((n.k_s0 & 7) || (n.k_s1 & 7) || (n.v_s0 & 7) || (n.v_s1 & 7)) return MUX_ERR_MISALIGNED;
  if (n.rope_cache != nullptr && (!aligned16(n.rope_cache) || n.rope_max_position <= 0)) return MUX_ERR_BAD_SHAPE;
  if (n.new_tokens < 1 || n.new_tokens > MUX_MAX_FUSED_NEW_TOKENS) return MUX_ERR_BAD_SHAPE;
  return MUX_OK;
}

static int run_single(const mux_attn_args_t* a, const NewRows& rows, void* workspace,
                      size_t workspace_bytes, void* cuda_stream) {
  int st = mux::validate(a);
  if (st != MUX_OK) return st;
  if ((st = validate_new_rows(rows)) != MUX_OK) return st;
  if (a->num_seqs == 0) return MUX_OK;
  const long long items = (long long)a->num_seqs * a->num_kv_heads;
  const mux::Plan pl = mux::plan_of(a);
  if ((st = mux::plan_limits(pl, items)) != MUX_OK) return st;
  if ((st = mux::check_workspace(pl, workspace, workspace_bytes)) != MUX_OK) return st;
  unsigned* status = mux::device_status_ptr();
  if (status == nullptr) return MUX_ERR_CUDA;

  mux::AttnParams prm = {};
  prm.q = a->q;
  prm.out = a->out;
  prm.kc = a->key_cache;
  prm.vc = a->value_cache;
  prm.block_tables = a->block_tables;
  prm.context_lens = a->context_lens;
  prm.head_mapping = a->head_mapping;
  prm.seq_rows = a->seq_rows;
  prm.q_s0 = a->q_seq_stride;
  prm.q_s1 = a->q_head_stride;
  prm.o_s0 = a->out_seq_stride;
  prm.o_s1 = a->out_head_stride;
  prm.bt_s0 = a->bt_seq_stride;
  prm.bt_s1 = a->bt_head_stride;
  prm.status = status;
  prm.num_blocks = a->num_blocks;
  prm.scale = a->scale;
  prm.num_q_heads = a->num_q_heads;
  prm.num_kv_heads = a->num_kv_heads;
  prm.group = a->num_q_heads / a->num_kv_heads;
  prm.gs = pl.gs;
  prm.head_tiles = pl.head_tiles;
  prm.pb = pl.pb;
  prm.max_parts = pl.max_parts;
  prm.max_context_len = a->max_context_len;
  prm.nst = pl.nst;
  prm.prod_lanes = 2;
  prm.flags = a->flags;
  prm.k_new = rows.k;
  prm.v_new = rows.v;
  prm.kn_s0 = rows.k_s0;
  prm.kn_s1 = rows.k_s1;
  prm.vn_s0 = rows.v_s0;
  prm.vn_s1 = rows.v_s1;
  prm.rope_cache = rows.rope_cache;
  prm.rope_max_position = rows.rope_max_position;
  prm.new_tokens = rows.new_tokens;
  mux::bind_workspace(prm, pl, workspace);
  if (a->num_units < 0) return MUX_ERR_BAD_SHAPE;
  if (a->num_units > 0) {
    if (a->units == nullptr) return MUX_ERR_NULL_POINTER;
    if (a->partition_size <= 0 || items >= (1 << 24) || pl.max_parts > 128) return MUX_ERR_BAD_SHAPE;
    prm.units = a->units;
  }
  return mux::launch<false>(prm, pl, items, a->dtype, a->block_size,
                            static_cast<cudaStream_t>(cuda_stream), a->num_units);
}

}  // namespace mux

extern "C" {

int mux_paged_attention(const mux_attn_args_t* a, void* workspace, size_t workspace_bytes,
                        void* cuda_stream) {
  return mux::run_single(a, mux::NewRows(), workspace, workspace_bytes, cuda_stream);
}

int mux_decode_attention(const mux_decode_args_t* a, void* workspace, size_t workspace_bytes,
                         void* cuda_stream) {
  if (a == nullptr) return MUX_ERR_NULL_POINTER;
  if (a->attn.num_seqs > 0 && (a->k == nullptr || a->v == nullptr)) return MUX_ERR_NULL_POINTER;
  // One new row per (sequence, kv head): with a shared block list the kv heads would all append to one slot.
  if (a->attn.bt_head_stride == 0 && a->attn.num_kv_heads > 1) return MUX_ERR_BAD_SHAPE;
  mux::NewRows rows;
  rows.k = a->k;
  rows.v = a->v;
  rows.k_s0 = a->k_seq_stride;
  rows.k_s1 = a->k_head_stride;
  rows.v_s0 = a->v_seq_stride;
  rows.v_s1 = a->v_head_stride;
  rows.rope_cache = a->cos_sin_cache;
  rows.rope_max_position = a->max_position;
  rows.new_tokens = a->new_tokens > 0 ? a->new_tokens : 1;
  return mux::run_single(&a->attn, rows, workspace, workspace_bytes, cuda_stream);
}

size_t mux_paged_attention_mixed_workspace_size(const mux_attn_mixed_args_t* a) {
  if (mux::validate(a) != MUX_OK || a->num_items == 0) return 0;
  return mux::plan_of(a).total();
}

}  // extern "C"

namespace mux {

static int run_mixed(const mux_attn_mixed_args_t* a, const NewRows& rows, void* workspace,
                     size_t workspace_bytes, void* cuda_stream) {
  int st = mux::validate(a);
  if (st != MUX_OK) return st;
  if ((st = validate_new_rows(rows)) != MUX_OK) return st;
  if (a->num_items == 0) return MUX_OK;
  const mux::Plan pl = mux::plan_of(a);
  if ((st = mux::plan_limits(pl, a->num_items)) != MUX_OK) return st;
  if ((st = mux::check_workspace(pl, workspace, workspace_bytes)) != MUX_OK) return st;
  unsigned* status = mux::device_status_ptr();
  if (status == nullptr) return MUX_ERR_CUDA;

  mux::AttnParams prm = {};
  prm.q = a->q;
  prm.out = a->out;
  prm.kc = a->key_cache;
  prm.vc = a->value_cache;
  prm.block_tables = a->block_tables;
  prm.item_ctx = a->item_context_len;
  prm.item_q_row = a->item_q_row;
  prm.item_group = a->item_group;
  prm.item_scale = a->item_scale;
  prm.q_s1 = a->q_row_stride;
  prm.o_s1 = a->out_row_stride;
  prm.bt_s0 = a->bt_item_stride;
  prm.status = status;
  prm.num_blocks = a->num_blocks;
  prm.gs = pl.gs;
  prm.head_tiles = 1;
  prm.pb = pl.pb;
  prm.max_parts = pl.max_parts;
  prm.max_context_len = a->max_context_len;
  prm.nst = pl.nst;
  prm.prod_lanes = 2;
  prm.flags = a->flags;
  prm.k_new = rows.k;
  prm.v_new = rows.v;
  prm.kn_s0 = rows.k_s0;
  prm.vn_s0 = rows.v_s0;
  prm.rope_cache = rows.rope_cache;
  prm.rope_max_position = rows.rope_max_position;
  prm.new_tokens = rows.new_tokens;
  mux::bind_workspace(prm, pl, workspace);
  if (a->num_units < 0) return MUX_ERR_BAD_SHAPE;
  if (a->num_units > 0) {
    if (a->units == nullptr) return MUX_ERR_NULL_POINTER;
    if (a->partition_size <= 0 || a->num_items >= (1 << 24) || pl.max_parts > 128) return MUX_ERR_BAD_SHAPE;
    prm.units = a->units;
  }
  return mux::launch<true>(prm, pl, a->num_items, a->dtype, a->block_size,
                           static_cast<cudaStream_t>(cuda_stream), a->num_units);
}

}  // namespace mux

extern "C" {

int mux_paged_attention_mixed(const mux_attn_mixed_args_t* a, void* workspace,
                              size_t workspace_bytes, void* cuda_stream) {
  return mux::run_mixed(a, mux::NewRows(), workspace, workspace_bytes, cuda_stream);
}

int mux_decode_attention_mixed(const mux_decode_mixed_args_t* a, void* workspace,
                               size_t workspace_bytes, void* cuda_stream) {
  if (a == nullptr) return MUX_ERR_NULL_POINTER;
  if (a->attn.num_items > 0 && (a->k == nullptr || a->v == nullptr)) return MUX_ERR_NULL_POINTER;
  mux::NewRows rows;
  rows.k = a->k;
  rows.v = a->v;
  rows.k_s0 = a->k_row_stride;
  rows.v_s0 = a->v_row_stride;
  rows.rope_cache = a->cos_sin_cache;
  rows.rope_max_position = a->max_position;
  rows.new_tokens = a->new_tokens > 0 ? a->new_tokens : 1;
  return mux::run_mixed(&a->attn, rows, workspace, workspace_bytes, cuda_stream);
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Allocation-free variant of mux_paged_attention.
//
// Some hosts of this library may not call cudaMalloc once they are running: a
// serving worker whose memory budget was fixed at start-up (FlexStore gives the
// KV pool a set fraction of HBM and the rest is spoken for), a process that
// shares the GPU with others under MPS and must not grow, or code on a path
// where allocation calls are simply not allowed.  For them the split-K scratch
// lives in a fixed array inside the library image instead of a caller buffer.
// Every GPU that loads the library carries the array until the process exits.
namespace mux {

constexpr size_t kStaticScratchBytes = MUX_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime's symbol
// table, not something a kernel can dereference; the real device address is
// looked up once per device (with that device current) and remembered.
static void* g_static_scratch_addr[kMaxDevicesTracked] = {};
static std::mutex g_static_scratch_mutex;

static int static_scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return record_cuda_error(e);
  if (dev < 0 || dev >= kMaxDevicesTracked) return record_cuda_error(cudaErrorInvalidDevice);
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
    if (e != cudaSuccess) return record_cuda_error(e);
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return MUX_OK;
}

}  // namespace mux

extern "C" int mux_paged_attention_static_scratch(const mux_attn_args_t* a, void* cuda_stream) {
  int st = mux::validate(a);
  if (st != MUX_OK) return st;
  if (a->num_seqs == 0) return MUX_OK;
  const size_t need = mux_paged_attention_workspace_size(a);
  if (need > mux::kStaticScratchBytes) return MUX_ERR_TOO_LARGE;  // use mux_paged_attention with your own buffer
  void* scratch = nullptr;
  st = mux::static_scratch_address(&scratch);
  if (st != MUX_OK) return st;
  // Nothing in the scratch has to be cleared: every partial that the merge kernel
  // reads is written by the attention kernel of the same call first.
  return mux_paged_attention(a, scratch, mux::kStaticScratchBytes, cuda_stream);
}
