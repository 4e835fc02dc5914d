// Row-parallel o_proj GEMM of a tensor-parallel rank fused with the all-reduce of its result (sm_100a).
//
// The reference's attention layer ends in ParallelLinear.row: every TP rank multiplies its heads'
// attention output by its slice of the o_proj weight and the [tokens, hidden] partial results are
// summed over the ranks by an NCCL all-reduce (muxserve/flexserver/models/llama.py:131-137,162).
// Here ONE kernel per rank does both: a tcgen05 GEMM (TMA-staged 128 x 64 operand slabs, fp32
// accumulators in tensor memory) whose epilogue is the exchange, tile by tile, so that the tiles that
// finish first cross NVLink while the others still multiply:
//
//   CTA j owns output columns [64 j, 64 j + 64).  Small messages ((world - 1) * bytes <= 4 MiB) go one-shot:
//   every rank's CTA j rounds its partial tile to the tensor type, pushes it (plain peer stores) into area
//   [rank] of every rank's exchange buffer and raises a flag there; it then waits for the world's flags in
//   its own buffer and sums the world's tiles from LOCAL memory in rank order (fp32, one rounding) into `out`.
//   Larger messages go through the tile's OWNER, rank j mod world:
//   1. every rank's CTA j pushes its partial tile into the owner's buffer and raises a flag there;
//   2. the owner's CTA j waits for the world's flags, sums the world's partial tiles from local memory,
//      pushes the sum to every rank and raises a second flag;
//   3. every rank's CTA j waits for that flag and copies the 128 x 64 result to `out`.
//
// Flags carry a per-CTA call counter kept in the exchange buffer (every call on a communicator has the
// same grid, so the counters agree across ranks without atomics); data areas alternate with its parity.
// Every wait is bounded (MUX_DEV_WAIT_TIMEOUT), TMEM is freed on every path.  No multimem, no cluster
// multicast, no TMA over peer memory: the tensor maps cover only this rank's own operands.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdint>
#include <mutex>
#include <type_traits>

#include "internal.h"
#include "ptx.cuh"

namespace mux {
namespace oproj {

constexpr int kBM = 128;                 // rows of a tile (tokens; at most 128 per call)
constexpr int kBN = 64;                  // output columns per CTA
constexpr int kBK = 64;                  // k elements per stage: one 128-byte swizzled slab
constexpr int kABytes = kBM * 128;       // 16 KiB
constexpr int kBBytes = kBN * 128;       // 8 KiB
constexpr int kStageBytes = kABytes + kBBytes;
// One ring of 8 (A + W) stages.  Measured alternatives on B200 (m 128, n 8192, k 4096), all slower or equal: separate A
// and W rings with their own barriers (two waits and two commits per k-block in the issuing thread: +20 %), fewer A
// and more W stages (6 x 12 ... 4 x 16: the A boxes, although they hit L2, see 2-4 us of latency under this load
// like the W boxes from DRAM), every CTA starting at a different k-block (no hot spot to spread), weights repacked
// into contiguous 8 KiB pieces fetched by one bulk copy each (the row-segment access pattern is not the limit).
constexpr int kStages = 8;
constexpr int kThreads = 192;            // warps 0-3 epilogue (one thread per row), 4 TMA producer, 5 MMA issuer
constexpr int kProdWarp = 4, kMmaWarp = 5;
constexpr uint32_t kTmemCols = 64;
constexpr int kMaxTiles = MUX_TP_OPROJ_MAX_COLS / kBN;   // 256
constexpr int kMaxWorld = MUX_TP_MAX_WORLD;
constexpr unsigned kWaitLimit = 1u << 23;
constexpr size_t kCtrlOffset = 8192;     // the fused op's control block follows the plain all-reduce's
constexpr size_t kCtrlTotal = MUX_TP_CTRL_BYTES;

struct FusedCtrl {
  unsigned epoch[kMaxTiles];               // per CTA: calls completed on this rank
  unsigned ready[kMaxWorld][kMaxTiles];    // on the owner: partial tile of [source rank][tile] has arrived
  unsigned done[kMaxTiles];                // on every rank: the owner's sum of the tile has arrived
};
static_assert(kCtrlOffset + sizeof(FusedCtrl) <= kCtrlTotal, "control blocks");

struct Params {
  unsigned char* buf[kMaxWorld];   // exchange buffers (world > 1)
  void* out[kMaxWorld];            // real launch: [rank]; emulated launch: one per rank
  long long out_stride[kMaxWorld]; // elements
  long long slot_bytes;
  unsigned* status;
  int m, n, k;
  int world, rank;
  int one_shot;                    // exchange form (see the top of the file)
  int early_w;                     // weight tiles may be fetched before the kernels ahead have completed
};

constexpr int smem_bytes() { return kStages * kStageBytes + 1024 + 256; }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Shared-memory matrix descriptor, 128-byte swizzle, K-major slab: rows 128 B apart, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)((16u >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((1024u >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// fp32 accumulator, A and B of one 16-bit format (0 f16, 1 bf16), both K-major, M = 128.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt, uint32_t n) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
#define MUX_OF4(a, i) "=f"(a[i]), "=f"(a[i + 1]), "=f"(a[i + 2]), "=f"(a[i + 3])
// This warp's 32 TMEM lanes x 32 consecutive fp32 columns -> 32 registers per thread (thread = lane = row).
template <int OFF, int N>
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&s)[N]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : MUX_OF4(s, OFF), MUX_OF4(s, OFF + 4), MUX_OF4(s, OFF + 8), MUX_OF4(s, OFF + 12), MUX_OF4(s, OFF + 16),
        MUX_OF4(s, OFF + 20), MUX_OF4(s, OFF + 24), MUX_OF4(s, OFF + 28)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ uint4 ld_vol(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_flag(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_flag(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// One thread waits until *f has reached `epoch` (bounded).
__device__ __forceinline__ void wait_flag(const unsigned* f, unsigned epoch, unsigned* status) {
  unsigned i = 0;
  while ((int)(ld_flag(f) - epoch) < 0) {
    if (++i >= kWaitLimit || ((i & 1023u) == 0 && (*reinterpret_cast<volatile unsigned*>(status) & MUX_DEV_WAIT_TIMEOUT))) {
      atomicOr(status, MUX_DEV_WAIT_TIMEOUT);
      break;
    }
  }
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t w);
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
}

enum Bar { FULL = 0, EMPTY = kStages, ACC = 2 * kStages, NUM_BARS = 2 * kStages + 1 };

// EMU: all ranks of a world in one cooperative grid on one GPU (blockIdx.y = rank), for tests.
template <typename T, bool EMU>
__global__ void __launch_bounds__(kThreads, 1)
oproj_allreduce_kernel(const __grid_constant__ CUtensorMap tma_a0, const __grid_constant__ CUtensorMap tma_w0,
                       const CUtensorMap* __restrict__ emu_maps, const __grid_constant__ Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x;
  const int rank = EMU ? (int)blockIdx.y : p.rank;
  const CUtensorMap* tma_a = EMU ? emu_maps + 2 * rank : &tma_a0;
  const CUtensorMap* tma_w = EMU ? emu_maps + 2 * rank + 1 : &tma_w0;
  const uint32_t raw = smem_u32(smem_raw);
  if (raw & 1023u) {  // the swizzle pattern needs the declared alignment
    if (tid == 0) atomicOr(p.status, MUX_DEV_INTERNAL);
    return;
  }
  const uint32_t sBar = raw + kStages * kStageBytes;
  auto bar = [&](int i) { return sBar + 8u * (uint32_t)i; };
  const uint32_t sSlot = sBar + 8u * NUM_BARS;
  volatile uint32_t* slot = reinterpret_cast<volatile uint32_t*>(smem_raw + (sSlot - raw));
  const int nkb = p.k / kBK;

  if (tid == kProdWarp * 32) {
    prefetch_tensormap(tma_a);
    prefetch_tensormap(tma_w);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar(FULL + i), 1);
      mbar_init(bar(EMPTY + i), 1);
    }
    mbar_init(bar(ACC), 1);
    mbar_init_fence();
  }
  // The weight slice is a constant of the model; the activations and the call counter come from the kernels ahead.
  // With early_w only the threads that touch those (producer lanes before their first A tile, the epilogue) wait.
  if (!p.early_w) griddep_wait();
  griddep_launch_dependents();
  __syncthreads();
  uint32_t tmem = 0;
  if (warp == kMmaWarp) tmem_alloc(sSlot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  tmem = *slot;

  if (warp == kProdWarp) {
    // lane s owns stage s (k-blocks s, s + kStages, ...): a single issuing thread pays the barrier and copy-issue
    // latency of every stage in turn, which alone is longer than the weight stream of one CTA per SM needs
    if (lane < kStages) {
      const int st = lane;
      const uint32_t dst = raw + st * kStageBytes;
      uint32_t parity = 0;
      for (int kb = st; kb < nkb; kb += kStages) {
        if (kb >= kStages) {
          mbar_wait_sleepy(bar(EMPTY + st), parity, p.status, MUX_DEV_WAIT_TIMEOUT);
          parity ^= 1u;
        }
        mbar_arrive_expect_tx(bar(FULL + st), kStageBytes);
        tma_load_2d(dst + kABytes, tma_w, kb * kBK, tile * kBN, bar(FULL + st));
        if (p.early_w && kb == st) griddep_wait();
        tma_load_2d(dst, tma_a, kb * kBK, 0, bar(FULL + st));                       // rows past m read as zeros
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc = instr_desc(fmt, kBN);
      for (int kb = 0; kb < nkb; ++kb) {
        const int st = kb % kStages;
        // (the wait tests the phase before it suspends: the ring runs ahead of this thread, and a suspended wait costs
        // a few hundred cycles of wake-up even when the phase is already complete — 18 % of this GEMM's time)
        mbar_wait_sleepy(bar(FULL + st), (uint32_t)(kb / kStages) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
        tc_fence_after();
        const uint64_t dA = smem_desc(raw + st * kStageBytes);
        const uint64_t dB = smem_desc(raw + st * kStageBytes + kABytes);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)   // a 16-element k-step is 32 bytes inside the swizzled 128-byte row
          umma_f16_ss(tmem, dA + (uint64_t)(ks * 2), dB + (uint64_t)(ks * 2), idesc, (kb > 0 || ks > 0) ? 1u : 0u);
        umma_commit(bar(EMPTY + st));
      }
      umma_commit(bar(ACC));
    }
  } else {
    // ------------------------------------------------------------------ epilogue: TMEM lane = output row
    const int row = warp * 32 + lane;
    if (p.early_w) griddep_wait();
    mbar_wait_sleepy(bar(ACC), 0, p.status, MUX_DEV_WAIT_TIMEOUT);  // 128 threads waiting out the whole main loop: asleep, not polling
    __syncwarp();
    tc_fence_after();
    float acc[64];
    const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
    tmem_ld32<0>(taddr, acc);
    tmem_ld32<32>(taddr + 32, acc);
    tmem_wait_ld();
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i].x = pack2<T>(acc[8 * i], acc[8 * i + 1]);
      v[i].y = pack2<T>(acc[8 * i + 2], acc[8 * i + 3]);
      v[i].z = pack2<T>(acc[8 * i + 4], acc[8 * i + 5]);
      v[i].w = pack2<T>(acc[8 * i + 6], acc[8 * i + 7]);
    }
    T* out = static_cast<T*>(p.out[rank]);
    // The tile goes through shared memory (the operand stages are free once the accumulator barrier has fired) so
    // that every global and peer access below is whole 128-byte rows: thread t then owns the 16-byte chunk
    // c = t % 8 of rows t / 8 + 16 j.  Chunks are XOR-swizzled by row to keep both sides free of bank conflicts.
    uint4* stg = reinterpret_cast<uint4*>(smem_raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) stg[row * 8 + (i ^ (row & 7))] = v[i];
    named_bar_sync(1, 128);
    const int c = tid & 7, r0 = tid >> 3;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int r = j * 16 + r0;
      v[j] = stg[r * 8 + (c ^ (r & 7))];
    }
    auto cell_of = [&](int j) {   // chunk (row j * 16 + r0, c) of this tile inside a [m, n] message
      return ((size_t)(j * 16 + r0) * p.n + (size_t)tile * kBN) * sizeof(T) + (size_t)c * 16;
    };
    auto out_of = [&](int j) {
      return reinterpret_cast<uint4*>(out + (long long)(j * 16 + r0) * p.out_stride[rank] + tile * kBN) + c;
    };
    auto sum_world = [&](const unsigned char* base, int j) {   // fixed rank order: every rank gets the same bits
      float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int q = 0; q < p.world; ++q) {
        const uint4 x = ld_vol(base + (size_t)q * ((size_t)p.m * p.n * sizeof(T)) + cell_of(j));
        const float2 a = unpack2<T>(x.x), b = unpack2<T>(x.y), cc = unpack2<T>(x.z), d = unpack2<T>(x.w);
        s[0] += a.x; s[1] += a.y; s[2] += b.x; s[3] += b.y; s[4] += cc.x; s[5] += cc.y; s[6] += d.x; s[7] += d.y;
      }
      uint4 r;
      r.x = pack2<T>(s[0], s[1]);
      r.y = pack2<T>(s[2], s[3]);
      r.z = pack2<T>(s[4], s[5]);
      r.w = pack2<T>(s[6], s[7]);
      return r;
    };
    const int nj = (p.m - r0 + 15) / 16;   // rows j * 16 + r0 < m
    if (p.world == 1) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (j < nj) *out_of(j) = v[j];
    } else {
      FusedCtrl* my = reinterpret_cast<FusedCtrl*>(p.buf[rank] + kCtrlOffset);
      const unsigned epoch = *reinterpret_cast<volatile unsigned*>(&my->epoch[tile]) + 1u;
      const size_t slot_off = kCtrlTotal + (size_t)(epoch & 1u) * (size_t)p.slot_bytes;
      const size_t msg_bytes = (size_t)p.m * p.n * sizeof(T);
      const int owner = tile % p.world;
      if (p.one_shot) {
        for (int q = 0; q < p.world; ++q) {
          unsigned char* dst = p.buf[q] + slot_off + (size_t)rank * msg_bytes;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < nj) *reinterpret_cast<uint4*>(dst + cell_of(j)) = v[j];
        }
        named_bar_sync(1, 128);  // the releasing flag stores are cumulative over the chunks pushed by the other threads
        if (tid < p.world) st_flag(&reinterpret_cast<FusedCtrl*>(p.buf[tid] + kCtrlOffset)->ready[rank][tile], epoch);
        if (tid < p.world) wait_flag(&my->ready[tid][tile], epoch, p.status);
        named_bar_sync(1, 128);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < nj) *out_of(j) = sum_world(p.buf[rank] + slot_off, j);
        if (tid == 0) my->epoch[tile] = epoch;
      } else {
        // 1. my partial tile -> the owner's area [rank]
        {
          unsigned char* dst = p.buf[owner] + slot_off + (size_t)rank * msg_bytes;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < nj) *reinterpret_cast<uint4*>(dst + cell_of(j)) = v[j];
        }
        named_bar_sync(1, 128);  // the releasing flag store is cumulative over the chunks pushed by the other threads
        if (tid == 0) st_flag(&reinterpret_cast<FusedCtrl*>(p.buf[owner] + kCtrlOffset)->ready[rank][tile], epoch);
        // 2. the owner sums the world's partial tiles and hands the sum to everybody
        if (owner == rank) {
          if (tid < p.world) wait_flag(&my->ready[tid][tile], epoch, p.status);
          named_bar_sync(1, 128);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < nj) v[j] = sum_world(p.buf[rank] + slot_off, j);
          // the sum goes where the owner's own partial lay, on every rank (elsewhere that cell is unused)
          for (int q = 0; q < p.world; ++q) {
            unsigned char* dst = p.buf[q] + slot_off + (size_t)rank * msg_bytes;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (j < nj) *reinterpret_cast<uint4*>(dst + cell_of(j)) = v[j];
          }
          named_bar_sync(1, 128);
          if (tid < p.world) st_flag(&reinterpret_cast<FusedCtrl*>(p.buf[tid] + kCtrlOffset)->done[tile], epoch);
        }
        // 3. everybody takes the sum from its own buffer
        if (tid == 0) wait_flag(&my->done[tile], epoch, p.status);
        named_bar_sync(1, 128);
        const unsigned char* src = p.buf[rank] + slot_off + (size_t)owner * msg_bytes;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < nj) *out_of(j) = ld_vol(src + cell_of(j));
        if (tid == 0) my->epoch[tile] = epoch;
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// ---- host side -------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int encode_fn(EncodeTiledFn* out) {
  static EncodeTiledFn fn = nullptr;
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res);
    if (e != cudaSuccess) return record_cuda_error(e);
    if (res != cudaDriverEntryPointSuccess || ptr == nullptr) return record_cuda_error(cudaErrorSymbolNotFound);
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  *out = fn;
  return MUX_OK;
}

// [rows][cols] with `row_stride` elements between rows, fetched in boxes of 64 columns x box_rows rows with the
// 128-byte swizzle; rows past the end read as zeros.
static int make_map(EncodeTiledFn enc, CUtensorMap* map, const void* ptr, int dtype, int64_t rows, int64_t cols,
                    int64_t row_stride, int box_rows) {
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, dtype == MUX_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                         2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MUX_OK : record_cuda_error(cudaErrorInvalidValue);
}

static int validate(const mux_oproj_args_t* a) {
  if (a == nullptr) return MUX_ERR_NULL_POINTER;
  if (a->dtype != MUX_DTYPE_F16 && a->dtype != MUX_DTYPE_BF16) return MUX_ERR_BAD_DTYPE;
  if (a->m < 0 || a->m > kBM || a->n <= 0 || a->k <= 0) return MUX_ERR_BAD_SHAPE;
  if (a->algo != MUX_TP_AUTO && a->algo != MUX_TP_ONE_SHOT && a->algo != MUX_TP_TWO_SHOT) return MUX_ERR_BAD_SHAPE;
  if ((a->flags & ~MUX_OPROJ_EARLY_W) != 0) return MUX_ERR_BAD_SHAPE;
  if (a->n % kBN != 0 || a->n > MUX_TP_OPROJ_MAX_COLS || a->k % kBK != 0) return MUX_ERR_BAD_SHAPE;
  if (a->m == 0) return MUX_OK;
  if (!a->a || !a->w || !a->out) return MUX_ERR_NULL_POINTER;
  if (!aligned16(a->a) || !aligned16(a->w) || !aligned16(a->out)) return MUX_ERR_MISALIGNED;
  if ((a->a_row_stride & 7) || (a->w_row_stride & 7) || (a->out_row_stride & 7)) return MUX_ERR_MISALIGNED;
  if (a->a_row_stride < a->k || a->w_row_stride < a->k || a->out_row_stride < a->n) return MUX_ERR_BAD_SHAPE;
  return MUX_OK;
}

// `which` tells the four instantiations apart (they share one function-pointer type).
template <typename K>
static int ensure_smem(K kern, int which, int dev) {
  static std::mutex mu;
  static bool done[4][64] = {};
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < 64 && !done[which][dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes());
    if (e != cudaSuccess) return record_cuda_error(e);
    done[which][dev] = true;
  }
  return MUX_OK;
}

static int fill_exchange(Params& prm, int world, void* const* buffers, long long buffer_bytes, const mux_oproj_args_t* a) {
  if (world < 2 || world > kMaxWorld) return MUX_ERR_BAD_SHAPE;
  if (buffers == nullptr) return MUX_ERR_NULL_POINTER;
  for (int q = 0; q < world; ++q) {
    if (buffers[q] == nullptr) return MUX_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(buffers[q]) & 255u) != 0) return MUX_ERR_MISALIGNED;
    prm.buf[q] = static_cast<unsigned char*>(buffers[q]);
  }
  prm.slot_bytes = (buffer_bytes - (long long)kCtrlTotal) / 2 / 256 * 256;
  const size_t need = (size_t)world * a->m * a->n * 2;
  if (prm.slot_bytes <= 0 || need > (size_t)prm.slot_bytes) return MUX_ERR_TOO_LARGE;
  prm.one_shot = a->algo == MUX_TP_ONE_SHOT   ? 1
                 : a->algo == MUX_TP_TWO_SHOT ? 0
                 : ((size_t)(world - 1) * a->m * a->n * 2 <= (size_t)MUX_TP_ONE_SHOT_MAX_PUSH_BYTES ? 1 : 0);
  return MUX_OK;
}

}  // namespace oproj
}  // namespace mux

extern "C" {

int mux_tp_oproj_allreduce(const mux_tp_comm_t* comm, const mux_oproj_args_t* a, void* cuda_stream) {
  using namespace mux::oproj;
  int st = validate(a);
  if (st != MUX_OK) return st;
  if (a->m == 0) return MUX_OK;
  Params prm = {};
  prm.world = 1;
  prm.rank = 0;
  if (comm != nullptr && comm->world > 1) {
    if (comm->rank < 0 || comm->rank >= comm->world) return MUX_ERR_BAD_SHAPE;
    if ((st = fill_exchange(prm, comm->world, comm->buffers, comm->buffer_bytes, a)) != MUX_OK) return st;
    prm.world = comm->world;
    prm.rank = comm->rank;
  }
  prm.m = a->m;
  prm.n = a->n;
  prm.k = a->k;
  prm.early_w = (a->flags & MUX_OPROJ_EARLY_W) ? 1 : 0;
  prm.out[prm.rank] = a->out;
  prm.out_stride[prm.rank] = a->out_row_stride;
  prm.status = mux::device_status_ptr();
  if (prm.status == nullptr) return MUX_ERR_CUDA;
  EncodeTiledFn enc;
  if ((st = encode_fn(&enc)) != MUX_OK) return st;
  CUtensorMap ma, mw;
  if ((st = make_map(enc, &ma, a->a, a->dtype, a->m, a->k, a->a_row_stride, kBM)) != MUX_OK) return st;
  if ((st = make_map(enc, &mw, a->w, a->dtype, a->n, a->k, a->w_row_stride, kBN)) != MUX_OK) return st;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return mux::record_cuda_error(e);
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(a->n / kBN));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = (size_t)smem_bytes();
  cfg.stream = static_cast<cudaStream_t>(cuda_stream);
  cfg.attrs = pdl;
  cfg.numAttrs = 1;
  const CUtensorMap* none = nullptr;
  if (a->dtype == MUX_DTYPE_F16) {
    auto kern = oproj_allreduce_kernel<__half, false>;
    if ((st = ensure_smem(kern, 0, dev)) != MUX_OK) return st;
    e = cudaLaunchKernelEx(&cfg, kern, ma, mw, none, prm);
  } else {
    auto kern = oproj_allreduce_kernel<__nv_bfloat16, false>;
    if ((st = ensure_smem(kern, 1, dev)) != MUX_OK) return st;
    e = cudaLaunchKernelEx(&cfg, kern, ma, mw, none, prm);
  }
  return e == cudaSuccess ? MUX_OK : mux::record_cuda_error(e);
}

int mux_tp_oproj_allreduce_emulated(int32_t world, void* const* buffers, int64_t buffer_bytes,
                                    const mux_oproj_args_t* args, void* maps_scratch, void* cuda_stream) {
  using namespace mux::oproj;
  if (args == nullptr || maps_scratch == nullptr) return MUX_ERR_NULL_POINTER;
  if (world < 2 || world > kMaxWorld) return MUX_ERR_BAD_SHAPE;
  int st;
  for (int q = 0; q < world; ++q) {
    if ((st = validate(&args[q])) != MUX_OK) return st;
    if (args[q].m != args[0].m || args[q].n != args[0].n || args[q].k != args[0].k || args[q].dtype != args[0].dtype ||
        args[q].algo != args[0].algo)
      return MUX_ERR_BAD_SHAPE;
  }
  if (args[0].m == 0) return MUX_OK;
  Params prm = {};
  if ((st = fill_exchange(prm, world, buffers, buffer_bytes, &args[0])) != MUX_OK) return st;
  prm.world = world;
  prm.m = args[0].m;
  prm.n = args[0].n;
  prm.k = args[0].k;
  prm.status = mux::device_status_ptr();
  if (prm.status == nullptr) return MUX_ERR_CUDA;
  EncodeTiledFn enc;
  if ((st = encode_fn(&enc)) != MUX_OK) return st;
  CUtensorMap host_maps[2 * kMaxWorld];
  for (int q = 0; q < world; ++q) {
    prm.out[q] = args[q].out;
    prm.out_stride[q] = args[q].out_row_stride;
    if ((st = make_map(enc, &host_maps[2 * q], args[q].a, args[q].dtype, args[q].m, args[q].k, args[q].a_row_stride, kBM)) != MUX_OK) return st;
    if ((st = make_map(enc, &host_maps[2 * q + 1], args[q].w, args[q].dtype, args[q].n, args[q].k, args[q].w_row_stride, kBN)) != MUX_OK) return st;
  }
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  cudaError_t e = cudaMemcpyAsync(maps_scratch, host_maps, sizeof(CUtensorMap) * 2 * world, cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);  // host_maps is a stack array
  if (e != cudaSuccess) return mux::record_cuda_error(e);
  int dev = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return mux::record_cuda_error(e);
  const CUtensorMap* dmaps = static_cast<const CUtensorMap*>(maps_scratch);
  void* kargs[] = {&host_maps[0], &host_maps[1], &dmaps, &prm};
  const dim3 grid((unsigned)(prm.n / kBN), (unsigned)world);
  const void* fn;
  if (args[0].dtype == MUX_DTYPE_F16) {
    auto kern = oproj_allreduce_kernel<__half, true>;
    if ((st = ensure_smem(kern, 2, dev)) != MUX_OK) return st;
    fn = (const void*)kern;
  } else {
    auto kern = oproj_allreduce_kernel<__nv_bfloat16, true>;
    if ((st = ensure_smem(kern, 3, dev)) != MUX_OK) return st;
    fn = (const void*)kern;
  }
  // the ranks' CTAs wait on one another: the cooperative launch fails unless the whole grid is resident at once
  e = cudaLaunchCooperativeKernel(fn, grid, dim3(kThreads), kargs, (size_t)smem_bytes(), s);
  return e == cudaSuccess ? MUX_OK : mux::record_cuda_error(e);
}

}  // extern "C"
