// Persistent form of the paged attention kernel.
//
// The grid is one wave of CTAs (SMs x resident CTAs).  Every CTA first builds,
// in shared memory, a coarse prefix sum of the work units of all items (a unit
// = one partition of one (item, head tile)), then its producer warp repeatedly
// takes the next unit index from a global queue word, maps it to (item, tile,
// partition), reads that unit's block ids and streams its K and V blocks into
// the shared-memory ring, always one unit ahead of the four consumer warps.
// The last unit of an item to finish (a ticket counter per item, no spinning)
// merges the item's partitions, so one launch does all of attention.
//
// Queue, exit and ticket words are plain 32-bit counters advanced with
// atomicAdd (a compare-and-swap loop on one hot word completes only one
// increment per round trip when hundreds of CTAs contend).  They must be zero
// when the kernel starts; the merging unit and the last CTA to leave put them
// back to zero, so a clean workspace stays clean from launch to launch.
#pragma once
#include "attn_common.cuh"

namespace mux {

constexpr int kMaxChunks = 1024;   // 32 items each: at most 32768 items per launch
constexpr int kMaxPB = 256;        // blocks per partition
constexpr int kMaxTickets = 65536; // (item, head tile) pairs per launch
// The scheduling words sit at the front of the workspace in a region of fixed size, so that
// the partials behind them never overlap words of a launch with another shape.
constexpr size_t kSchedBytes = ((2 + (size_t)kMaxTickets) * 4 + 255) & ~(size_t)255;

struct UnitDesc {
  ItemInfo info;        // q / out row offsets of the head tile, (max, sum) per head, geff
  long long ws_slot0;   // first partial slot of this (item, tile)
  int item;             // < 0: no more work
  int htile, part, nparts, ntok, nblk;
  float scale;
  int ids[1];           // pb entries follow (the descriptor stride is desc_stride(pb))
};

// A descriptor slot = header + pb block ids, then the unit's q rows (gs x 128 elements),
// which the producer stages with bulk copies so that the consumers never wait on global memory.
__host__ __device__ inline int desc_q_offset(int pb) {
  return ((int)sizeof(UnitDesc) + (pb - 1) * 4 + 15) & ~15;
}
__host__ __device__ inline int desc_stride(int pb, int gs) {
  return desc_q_offset(pb) + gs * kHeadSize * 2;
}

struct PSmemLayout {
  int ring, s, pm, desc, cum, flag, bars, total;
  int srow, prow;
};

__host__ __device__ inline PSmemLayout psmem_layout(int block_size, int pb, int gs, int nst, int num_chunks) {
  PSmemLayout L;
  const int tile = kHeadSize * block_size * 2;
  const int P = pb * block_size;
  L.srow = P + 8;
  L.prow = P + 16;
  int off = 0;
  L.ring = off;
  off += nst * tile;
  L.s = off;
  const int s_bytes = gs * L.srow * 4;
  const int red_bytes = kConsumerWarps * gs * kRedStride * 4;
  off += (s_bytes > red_bytes ? s_bytes : red_bytes);
  off = (off + 15) & ~15;
  L.pm = off;
  off += 2 * gs * L.prow * 2;
  off = (off + 15) & ~15;
  L.desc = off;
  off += 2 * desc_stride(pb, gs);
  L.cum = off;
  off += (num_chunks + 1) * 4;
  off = (off + 15) & ~15;
  L.flag = off;
  off += 16;
  L.bars = off;
  off += (2 * kMaxStages + 4) * 8;
  L.total = off;
  return L;
}

template <bool MIXED>
__device__ __forceinline__ int item_context(const AttnParams& p, int item) {
  int ctx = MIXED ? p.item_ctx[item] : p.context_lens[item / p.num_kv_heads];
  return ctx < 0 ? 0 : (ctx > p.max_context_len ? p.max_context_len : ctx);
}

template <bool MIXED>
__device__ __forceinline__ int item_units(const AttnParams& p, int item, int P) {
  const int ctx = item_context<MIXED>(p, item);
  const int parts = ctx == 0 ? 1 : (ctx + P - 1) / P;   // an empty context still gets a unit (writes zeros)
  return parts * (MIXED ? 1 : p.head_tiles);
}

template <typename T, int BS, bool MIXED>
__global__ void __launch_bounds__(kThreads)
paged_attn_persistent_kernel(const __grid_constant__ AttnParams p) {
  constexpr int TILE = kHeadSize * BS * 2;
  constexpr int MT = BS >= 16 ? BS / 16 : 1;
  constexpr int KSTEPS = BS >= 16 ? BS / 16 : 1;
  constexpr int CHUNK = BS * 16;
  constexpr int VROW = BS * 2;

  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int P = p.pb * BS;
  const int nst = p.nst;
  const PSmemLayout L = psmem_layout(BS, p.pb, p.gs, nst, p.num_chunks);
  unsigned char* desc_base = smem + L.desc;
  const int dstride = desc_stride(p.pb, p.gs);
  const int dq_off = desc_q_offset(p.pb);
  unsigned* cum = reinterpret_cast<unsigned*>(smem + L.cum);   // cum[c] = units before chunk c
  int* flag = reinterpret_cast<int*>(smem + L.flag);
  const uint32_t bars = smem_u32(smem + L.bars);
  const uint32_t bar_full = bars, bar_empty = bars + 8 * kMaxStages;
  const uint32_t bar_dfull = bars + 16 * kMaxStages, bar_dempty = bar_dfull + 16;
  const uint32_t ring = smem_u32(smem + L.ring);

  if (tid == 0) {
    for (int i = 0; i < nst; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_dfull + 8 * i, 1);
      mbar_init(bar_dempty + 8 * i, 1);
    }
    mbar_init_fence();
  }
  for (int i = tid; i <= p.num_chunks; i += kThreads) cum[i] = 0u;
  __syncthreads();
  // Nothing above touched global memory.  From here on inputs written by
  // earlier kernels of the stream are read.
  griddep_wait();
  griddep_launch_dependents();

  for (int i = tid; i < p.num_items; i += kThreads)
    atomicAdd(&cum[(i >> 5) + 1], (unsigned)item_units<MIXED>(p, i, P));
  __syncthreads();
  if (warp == 0) {  // in-place inclusive scan of cum[1..num_chunks]
    const int per = (p.num_chunks + 31) / 32;
    const int c0 = 1 + lane * per, c1 = min(c0 + per, p.num_chunks + 1);
    unsigned local = 0;
    for (int c = c0; c < c1; ++c) local += cum[c];
    unsigned incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      unsigned y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    unsigned run = incl - local;
    for (int c = c0; c < c1; ++c) {
      run += cum[c];
      cum[c] = run;
    }
  }
  __syncthreads();
  const unsigned U = cum[p.num_chunks];

  if (warp == kConsumerWarps) {
    // ------------------------------ producer warp ------------------------------
    const unsigned char* kc = static_cast<const unsigned char*>(p.kc);
    const unsigned char* vc = static_cast<const unsigned char*>(p.vc);
    unsigned u_next = 0;               // next unit of this CTA (lane 0)
    unsigned pos = 0;                  // next ring stage (lane 0)
    unsigned e_used = 0, e_par = 0;    // per stage: used before / parity of the next empty wait (lane 0)
    for (unsigned k = 0;; ++k) {
      const int slot = k & 1;
      UnitDesc* d = reinterpret_cast<UnitDesc*>(desc_base + slot * dstride);
      if (k >= 2) mbar_wait(bar_dempty + 8 * slot, ((k >> 1) - 1) & 1, p.status, MUX_DEV_WAIT_TIMEOUT);
      // the first unit of a CTA is its own index; later ones come from the queue (taken by
      // lane 0 one unit early, so the round trip overlaps the previous unit's copies)
      const unsigned u = k == 0 ? blockIdx.x : __shfl_sync(0xffffffffu, u_next, 0);
      if (u >= U) {
        if (lane == 0) {
          d->item = -1;
          mbar_arrive(bar_dfull + 8 * slot);
        }
        break;
      }
      // unit -> chunk of 32 items (shared prefix sums) -> item (one coalesced load + warp scan)
      int lo = 0, hi = p.num_chunks;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (cum[mid] <= u) lo = mid; else hi = mid;
      }
      const int cand = lo * 32 + lane;
      const unsigned n = cand < p.num_items ? (unsigned)item_units<MIXED>(p, cand, P) : 0u;
      unsigned incl = n;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        unsigned y = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += y;
      }
      const unsigned before = cum[lo] + incl - n;
      const unsigned hit = __ballot_sync(0xffffffffu, n > 0 && before <= u && u < before + n);
      const int src = hit ? __ffs(hit) - 1 : 0;
      const int item = lo * 32 + src;
      const unsigned sub = u - __shfl_sync(0xffffffffu, before, src);

      ItemDesc it = load_item<MIXED>(p, item);
      if (it.ctx < 0 || it.ctx > p.max_context_len) {
        if (lane == 0) atomicOr(p.status, MUX_DEV_BAD_CONTEXT);
        it.ctx = it.ctx < 0 ? 0 : p.max_context_len;
      }
      const int nparts = it.ctx == 0 ? 1 : (it.ctx + P - 1) / P;
      const int htile = (int)(sub / (unsigned)nparts), part = (int)(sub % (unsigned)nparts);
      int ntok = it.ctx == 0 ? 0 : min(it.ctx - part * P, P);
      int nblk = (ntok + BS - 1) / BS;
      resolve_heads<MIXED>(p, it, item, htile, &d->info, lane);
      __syncwarp();
      if (d->info.geff <= 0) ntok = nblk = 0;  // no q head in this tile: nothing is streamed
      for (int i = lane; i < nblk; i += 32) {
        int id = it.bt_row[part * p.pb + i];
        if (id < 0 || id >= p.num_blocks) {
          atomicOr(p.status, MUX_DEV_BAD_BLOCK_ID);
          id = 0;
        }
        d->ids[i] = id;
      }
      if (lane == 0) {
        d->item = item;
        d->htile = htile;
        d->part = part;
        d->nparts = nparts;
        d->ntok = ntok;
        d->nblk = nblk;
        d->scale = it.scale;
        d->ws_slot0 = ((long long)item * p.head_tiles + htile) * p.max_parts;
      }
      __syncwarp();
      if (lane == 0) {
        // publish the descriptor; the unit's q rows (256 B each) ride on the same barrier
        const int gq = nblk > 0 ? d->info.geff : 0;
        if (gq > 0) {
          mbar_arrive_expect_tx(bar_dfull + 8 * slot, gq * kHeadSize * 2);
          const uint32_t qdst = smem_u32(reinterpret_cast<unsigned char*>(d) + dq_off);
          for (int n = 0; n < gq; ++n)
            bulk_g2s(qdst + n * kHeadSize * 2, static_cast<const T*>(p.q) + d->info.qoff[n], kHeadSize * 2,
                     bar_dfull + 8 * slot);
        } else {
          mbar_arrive(bar_dfull + 8 * slot);
        }
        u_next = gridDim.x + atomicAdd(p.sched, 1u);
        // K blocks, then V blocks.  Each phase starts on a ring position that is a multiple
        // of 4, so block j of a phase always sits in a stage congruent to j mod 4 and is
        // consumed by warp j mod 4: a stage has one fixed consumer warp.
#pragma unroll 1
        for (int phase = 0; phase < 2 && nblk > 0; ++phase) {
          pos = (pos + 3u) & ~3u;
          if (pos >= (unsigned)nst) pos = 0;
          const unsigned char* base = phase == 0 ? kc : vc;
          for (int j = 0; j < nblk; ++j) {
            const unsigned bit = 1u << pos;
            if (e_used & bit) {  // wait for the consumer to release the stage's previous use
              mbar_wait(bar_empty + 8 * pos, (e_par >> pos) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
              e_par ^= bit;
            } else {
              e_used |= bit;
            }
            mbar_arrive_expect_tx(bar_full + 8 * pos, TILE);
            bulk_g2s(ring + pos * TILE, base + (long long)d->ids[j] * TILE, TILE, bar_full + 8 * pos);
            pos = pos + 1u == (unsigned)nst ? 0u : pos + 1u;
          }
        }
      }
      __syncwarp();
    }
    return;
  }

  // ------------------------------ consumer warps ------------------------------
  const int g = lane >> 2, tq = lane & 3;
  float* S = reinterpret_cast<float*>(smem + L.s);
  T* Pm = reinterpret_cast<T*>(smem + L.pm);
  const int SROW = L.srow, PROW = L.prow;
  const uint32_t pm_base = smem_u32(Pm);
  T* out = static_cast<T*>(p.out);
  unsigned pos = 0;     // ring stage where the next phase starts (same sequence as the producer's)
  unsigned f_par = 0;   // per stage owned by this warp: parity of its next full wait

  for (unsigned k = 0;; ++k) {
    const int slot = k & 1;
    UnitDesc* d = reinterpret_cast<UnitDesc*>(desc_base + slot * dstride);
    mbar_wait(bar_dfull + 8 * slot, (k >> 1) & 1, p.status, MUX_DEV_WAIT_TIMEOUT);
    if (d->item < 0) break;
    ItemInfo* info = &d->info;
    const int geff = info->geff;
    const int ntok = d->ntok, nblk = d->nblk, nparts = d->nparts, part = d->part;
    const float scale = d->scale;

    if (geff > 0 && ntok == 0) {  // empty context: defined output, nothing to read
      if (tid < kHeadSize)
        for (int n = 0; n < geff; ++n) out[info->ooff[n] + tid] = from_float<T>(0.f);
    } else if (geff > 0) {
      uint32_t qf[8][2];
      if (g < geff) {
        const T* qr = reinterpret_cast<const T*>(reinterpret_cast<const unsigned char*>(d) + dq_off) + g * kHeadSize;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          qf[ks][0] = *reinterpret_cast<const uint32_t*>(qr + ks * 16 + 2 * tq);
          qf[ks][1] = *reinterpret_cast<const uint32_t*>(qr + ks * 16 + 8 + 2 * tq);
        }
      } else {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) qf[ks][0] = qf[ks][1] = 0u;
      }

      // ---- phase 1: logits.  Warp w takes blocks w, w+4, ... of the unit; they sit in stages
      // congruent to w mod 4, which no other warp ever waits on, so the parity of a stage's next
      // completion is simply flipped after every use (f_par).
      pos = (pos + 3u) & ~3u;
      if (pos >= (unsigned)nst) pos = 0;
      {
        const int n0 = 2 * tq;
        const int lm_tok = (lane & 7) + (BS >= 16 ? ((lane >> 3) & 1) * 8 : 0);
        const int lm_chunk = lane >> 4;
        for (int jb = warp; jb < nblk; jb += kConsumerWarps) {
          const unsigned stage = (pos + (unsigned)jb) % (unsigned)nst;
          mbar_wait(bar_full + 8 * stage, (f_par >> stage) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
          f_par ^= 1u << stage;
          const uint32_t tile = ring + stage * TILE;
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
              S[n0 * SROW + tok] = c[0] * scale;
              if (BS >= 16) S[n0 * SROW + tok + 8] = c[2] * scale;
            }
            if (n0 + 1 < geff) {
              S[(n0 + 1) * SROW + tok] = c[1] * scale;
              if (BS >= 16) S[(n0 + 1) * SROW + tok + 8] = c[3] * scale;
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
        }
      }
      pos = (pos + (unsigned)nblk) % (unsigned)nst;
      named_bar_sync(1, kConsumerThreads);

      // ---- softmax over the unit ----
      for (int n = warp; n < geff; n += kConsumerWarps) {
        const float* srow = S + n * SROW;
        float m = -INFINITY;
        for (int t = lane; t < ntok; t += 32) m = fmaxf(m, srow[t]);
        m = warp_max(m);
        float l = 0.f;
        T* prow = Pm + n * PROW;
        T* prow_lo = prow + p.gs * PROW;
        for (int t = lane; t < nblk * BS; t += 32) {
          const float pv = t < ntok ? __expf(srow[t] - m) : 0.f;
          l += pv;
          const T hi = from_float<T>(pv);
          prow[t] = hi;
          prow_lo[t] = from_float<T>(pv - to_float(hi));
        }
        l = warp_sum(l);
        if (lane == 0) {
          info->ml[n][0] = m;
          info->ml[n][1] = l;
        }
      }
      named_bar_sync(1, kConsumerThreads);

      // ---- phase 2: out^T[d][h] += V^T[d][t] P^T[t][h] ----
      float acc[8][4];
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
      {
        const bool lane_has = (BS >= 16) || (tq < 2);
        pos = (pos + 3u) & ~3u;
        if (pos >= (unsigned)nst) pos = 0;
        for (int jb = warp; jb < nblk; jb += kConsumerWarps) {
          const unsigned stage = (pos + (unsigned)jb) % (unsigned)nst;
          mbar_wait(bar_full + 8 * stage, (f_par >> stage) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
          f_par ^= 1u << stage;
          const uint32_t tile = ring + stage * TILE;
          const int rem = ntok - jb * BS;
#pragma unroll
          for (int ks = 0; ks < KSTEPS; ++ks) {
            const int t0 = ks * 16 + 4 * tq;
            uint32_t b0 = 0u, b1 = 0u, c0 = 0u, c1 = 0u;
            if (g < geff && lane_has) {
              const uint32_t pa = pm_base + (g * PROW + jb * BS + t0) * 2;
              uint2 pv = lds64(pa);
              b0 = pv.x;
              b1 = pv.y;
              pv = lds64(pa + p.gs * PROW * 2);
              c0 = pv.x;
              c1 = pv.y;
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
              const uint2 r0 = lds64(tile + row * VROW + t0 * 2);
              const uint2 r1 = lds64(tile + (row + 8) * VROW + t0 * 2);
              const uint32_t a[4] = {r0.x & mlo, r1.x & mlo, r0.y & mhi, r1.y & mhi};
              mma_16816<T>(acc[mt], a, b0, b1);
              mma_16816<T>(acc[mt], a, c0, c1);
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_empty + 8 * stage);
        }
      }

      pos = (pos + (unsigned)nblk) % (unsigned)nst;

      // ---- cross-warp reduction (aliases the logits, dead by now) ----
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
      for (int n = 0; n < geff; ++n) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) s += red[(w * p.gs + n) * kRedStride + tid];
        if (nparts == 1) {
          out[info->ooff[n] + tid] = from_float<T>(s / info->ml[n][1]);
        } else {
          const long long r = (d->ws_slot0 + part) * p.gs + n;
          p.ws_acc[r * kHeadSize + tid] = s;
          if (tid == 0) {
            p.ws_ml[r * 2] = info->ml[n][0];
            p.ws_ml[r * 2 + 1] = info->ml[n][1];
          }
        }
      }

      // ---- the last partition of the item to get here merges them all ----
      if (nparts > 1) {
        __threadfence();
        named_bar_sync(1, kConsumerThreads);
        if (tid == 0) {
          unsigned* ticket = p.sched + 2 + ((long long)d->item * p.head_tiles + d->htile);
          const unsigned tk = atomicAdd(ticket, 1u);
          const int last = tk == (unsigned)(nparts - 1);
          if (last) *ticket = 0u;  // nobody else touches it any more in this launch
          *flag = last;
        }
        named_bar_sync(1, kConsumerThreads);
        if (*flag) {
          __threadfence();
          for (int n = 0; n < geff; ++n) {
            float M = -INFINITY;
            for (int q = 0; q < nparts; ++q) M = fmaxf(M, __ldcg(p.ws_ml + ((d->ws_slot0 + q) * p.gs + n) * 2));
            float a = 0.f, lsum = 0.f;
            for (int q = 0; q < nparts; ++q) {
              const long long r = (d->ws_slot0 + q) * p.gs + n;
              const float w = __expf(__ldcg(p.ws_ml + r * 2) - M);
              lsum += __ldcg(p.ws_ml + r * 2 + 1) * w;
              a += __ldcg(p.ws_acc + r * kHeadSize + tid) * w;
            }
            out[info->ooff[n] + tid] = from_float<T>(a / lsum);
          }
        }
      }
    }
    named_bar_sync(1, kConsumerThreads);  // the unit's buffers and descriptor are free again
    if (tid == 0) mbar_arrive(bar_dempty + 8 * slot);
  }

  // The last CTA to leave clears the queue and exit words for the next launch.
  if (tid == 0) {
    const unsigned gone = atomicAdd(p.sched + 1, 1u);
    if (gone == gridDim.x - 1) {
      p.sched[0] = 0u;
      p.sched[1] = 0u;
    }
  }
}

}  // namespace mux
