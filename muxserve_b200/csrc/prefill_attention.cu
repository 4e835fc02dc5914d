// Prompt-phase (prefill) attention: causal self-attention of every prompt of a batch over its
// own tokens, the step PagedAttentionWithRoPE runs for the prompt rows of a batch before their
// K/V are written to the pool (muxserve/flexserver/models/llama.py:160-161 with
// input_metadata.prompt_lens from muxserve/flexserver/llm_runtime.py:298-330).
//
// This is the one GEMM-shaped kernel of the library, so it runs on the 5th-generation tensor
// cores: one CTA owns 128 query rows of one (prompt, q head) and walks the key/value tiles of
// 128 tokens up to the diagonal.
//   warp 8 (one lane)  TMA producer: Q once, then K and V tiles through a 3-stage ring
//                      (cp.async.bulk.tensor, 128-byte swizzle, completion on mbarriers)
//   warp 9 (one lane)  issues tcgen05.mma with A in tensor memory: S = Q.K^T into one of two TMEM
//                      buffers, O += P.V into a third; tcgen05.commit signals the mbarriers
//   warps 0-7          two threads per query row (64 columns each): tcgen05.ld of the S row, scale,
//                      causal mask, online softmax (lazy rescaling of O), P written back to tensor
//                      memory in place of the logits (the A operand of P.V), final O / l to global memory
// bf16 rounds P to 8 bits, which breaks the 2e-3 tolerance on short prompts with cancelling
// values; there P is split into hi + lo parts and P.V takes two MMAs per step.
// Every wait is bounded (ptx.cuh); TMEM is freed on every path that allocated it.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <type_traits>

#include "internal.h"
#include "ptx.cuh"

namespace mux {
namespace prefill {

constexpr int kTile = 128;                   // query rows per CTA = tokens per K/V tile
constexpr int kSlabBytes = kTile * 128;      // 128 rows x 64 elements: one 128-byte-swizzled slab
constexpr int kTileBytes = 2 * kSlabBytes;   // head size 128 = two slabs
constexpr int kHalf = kTile / 2;              // columns of a tile one softmax thread handles
constexpr int kSoftmaxWarps = 8;
constexpr int kProducerWarp = 8, kMmaWarp = 9;
constexpr int kThreads = 320;
constexpr uint32_t kTmemCols = 512;          // S0 | S1 | O | Q (448 columns used), power of two
constexpr float kRescaleStep = 8.f;          // O is rescaled only when the running max grows by 2^8

constexpr int kStages = 3;                    // K/V ring: two tiles in flight while one is consumed

enum Bar {
  Q_FULL = 0,                  // TMA bytes of Q have landed
  QT_FULL = 1,                 // the softmax warps have moved Q to tensor memory
  P_FULL = 2,
  KV_FULL = 3,                 // + ring stage
  S_FULL = KV_FULL + kStages,
  PV_DONE = S_FULL + kStages,
  NUM_BARS = PV_DONE + kStages
};

struct Params {
  void* out;
  int64_t out_seq_stride, out_head_stride;  // elements
  const int32_t* cu_seqlens;                // [num_seqs + 1]
 int total_tokens;
  int max_prompt_len;
  int group;                                // q heads per kv head
  float scale_log2;                         // scale * log2(e)
  unsigned* status;
};

template <bool SPLIT>
constexpr int smem_bytes() {
  // Q + K/V ring + barriers + the softmax halves' exchange buffer
  return kTileBytes * (1 + 2 * kStages) + 256 + 4 * kTile * 4;
}

// ---- tcgen05 / TMA building blocks -----------------------------------------------------------

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// All earlier tcgen05.mma of this thread arrive on `bar` when they complete.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem], 128 x 128 x 16, 16-bit operands, fp32 accumulate.  Row i of A lies in
// lane i, two 16-bit elements per 32-bit column, so a 16-element k-step is 8 columns.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle: start address, leading / stride byte offsets
// (all in 16-byte units), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor: fp32 accumulator, formats of A and of B (0 f16, 1 bf16), B major (0 K, 1 MN),
// N = 128, M = 128.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t a_fmt, uint32_t b_fmt, uint32_t b_mn_major) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (b_mn_major << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
}

#define MUX_F4(a, i) "=f"(a[i]), "=f"(a[i + 1]), "=f"(a[i + 2]), "=f"(a[i + 3])
#define MUX_F4I(a, i) "f"(a[i]), "f"(a[i + 1]), "f"(a[i + 2]), "f"(a[i + 3])

// This warp's 32 TMEM lanes x 32 consecutive fp32 columns -> 32 registers per thread (thread = lane = row).
template <int OFF, int N>
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&s)[N]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : MUX_F4(s, OFF), MUX_F4(s, OFF + 4), MUX_F4(s, OFF + 8), MUX_F4(s, OFF + 12), MUX_F4(s, OFF + 16),
        MUX_F4(s, OFF + 20), MUX_F4(s, OFF + 24), MUX_F4(s, OFF + 28)
      : "r"(taddr)
      : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&s)[N]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
      ::MUX_F4I(s, 0), MUX_F4I(s, 4), MUX_F4I(s, 8), MUX_F4I(s, 12), MUX_F4I(s, 16), MUX_F4I(s, 20),
        MUX_F4I(s, 24), MUX_F4I(s, 28), "r"(taddr)
      : "memory");
}

#define MUX_R4I(a, i) "r"(a[i]), "r"(a[i + 1]), "r"(a[i + 2]), "r"(a[i + 3])
__device__ __forceinline__ void tmem_st32u(uint32_t taddr, const uint32_t (&s)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
      ::MUX_R4I(s, 0), MUX_R4I(s, 4), MUX_R4I(s, 8), MUX_R4I(s, 12), MUX_R4I(s, 16), MUX_R4I(s, 20),
        MUX_R4I(s, 24), MUX_R4I(s, 28), "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void lds128(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr) : "memory");
}

template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack_pair<__half>(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// ---- the kernel ------------------------------------------------------------------------------
//
// Tensor memory (512 columns x 128 lanes, lane = query row):
//   [0,128) and [128,256)  logits S of tile j in buffer j & 1; the softmax threads overwrite them with the
//                          16-bit weights P (64 columns hi [+ 64 columns lo]), the A operand of P.V
//   [256,384)              O accumulator
//   [384,448)              Q, 16-bit pairs: the A operand of Q.K^T (read from shared memory once)
// Barriers (index = ring stage j % kStages unless noted):
//   KV_FULL   TMA bytes of K and V of tile j have landed
//   S_FULL    Q.K^T of tile j has completed: logits readable
//   P_FULL    (single) all 8 softmax warps have written P of tile j (they loaded S of tile j before)
//   PV_DONE   P.V of tile j has completed: the stage's shared memory is free, O holds tiles 0..j
// The issuing thread never needs an "S buffer free" signal: it issues Q.K^T of tile j + 1 after it has
// seen P_FULL of tile j - 1 and after it has issued P.V of tile j - 1, and tcgen05.mma of one thread
// execute in issue order.

template <typename T, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 1)
prefill_attn_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                    const __grid_constant__ CUtensorMap tmv, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];  // the swizzle pattern repeats every 1024 bytes
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq = blockIdx.z, head = blockIdx.y;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;  // the tiles with the most work start first

  griddep_wait();
  const int start = p.cu_seqlens[seq];
  const int len = p.cu_seqlens[seq + 1] - start;
  if (start < 0 || len < 0 || len > p.max_prompt_len || start + len > p.total_tokens) {
    if (tid == 0) atomicOr(p.status, MUX_DEV_BAD_CONTEXT);  // nothing of this prompt is read or written
    return;
  }
  if (qt * kTile >= len) return;
  const int n = qt + 1;  // key/value tiles 0..qt; the last one is the diagonal

  const uint32_t raw = smem_u32(smem_raw);
  if (raw & 1023u) {  // the tiles' swizzle needs the declared alignment; never seen violated, never worked around
    if (tid == 0) atomicOr(p.status, MUX_DEV_WAIT_TIMEOUT);
    return;
  }
  const uint32_t sQ = raw;
  const uint32_t sKV = sQ + kTileBytes;  // stage: K tile, then V tile
  const uint32_t sBar = sKV + kStages * 2 * kTileBytes;
  auto bar = [&](int i) { return sBar + 8u * (uint32_t)i; };
  const uint32_t sSlot = sBar + 8u * NUM_BARS;
  volatile uint32_t* slot = reinterpret_cast<volatile uint32_t*>(smem_raw + (sSlot - raw));
  float* xchg = reinterpret_cast<float*>(smem_raw + (sSlot + 16 - raw));  // [2][2][kTile]: row maxima / sums of the halves

  if (tid == 0) {
    mbar_init(bar(Q_FULL), 1);
    mbar_init(bar(QT_FULL), kSoftmaxWarps);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar(KV_FULL + i), 1);
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(PV_DONE + i), 1);
    }
    mbar_init(bar(P_FULL), kSoftmaxWarps);
    mbar_init_fence();
  }
  if (warp == kMmaWarp) tmem_alloc(sSlot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *slot;
  griddep_launch_dependents();

  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      const int kvh = head / p.group;
      const int q0 = start + qt * kTile;
      mbar_arrive_expect_tx(bar(Q_FULL), kTileBytes);
      tma_load_3d(sQ, &tmq, 0, head, q0, bar(Q_FULL));
      tma_load_3d(sQ + kSlabBytes, &tmq, 64, head, q0, bar(Q_FULL));
      for (int j = 0; j < n; ++j) {
        const int st = j % kStages;
        const uint32_t ph = (uint32_t)(j / kStages) & 1u;
        const int t0 = start + j * kTile;
        const uint32_t dst = sKV + st * 2 * kTileBytes;
        mbar_wait(bar(PV_DONE + st), ph ^ 1u, p.status, MUX_DEV_WAIT_TIMEOUT);  // P.V of tile j - kStages
        mbar_arrive_expect_tx(bar(KV_FULL + st), 2 * kTileBytes);
        tma_load_3d(dst, &tmk, 0, kvh, t0, bar(KV_FULL + st));
        tma_load_3d(dst + kSlabBytes, &tmk, 64, kvh, t0, bar(KV_FULL + st));
        tma_load_3d(dst + kTileBytes, &tmv, 0, kvh, t0, bar(KV_FULL + st));
        tma_load_3d(dst + kTileBytes + kSlabBytes, &tmv, 64, kvh, t0, bar(KV_FULL + st));
      }
      // No copy of this CTA may still be in flight when it ends (matters only after a failed wait).
      for (int j = (n > kStages ? n - kStages : 0); j < n; ++j)
        mbar_wait(bar(KV_FULL + j % kStages), (uint32_t)(j / kStages) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc_qk = instr_desc(fmt, fmt, 0);  // S = Q K^T: K tile K-major (d contiguous)
      // O = P V: V is MN-major (d contiguous, tokens = K).  A and B must have ONE format: fp16 weights over
      // bf16 values (a_fmt 0, b_fmt 1) raise "illegal instruction" on B200, hence the hi/lo split for bf16.
      constexpr uint32_t idesc_pv = instr_desc(fmt, fmt, 1);
      const uint32_t tS = tmem, tO = tmem + 256, tQ = tmem + 384;
      mbar_wait(bar(QT_FULL), 0, p.status, MUX_DEV_WAIT_TIMEOUT);
      auto issue_qk = [&](int j) {
        const int st = j % kStages;
        mbar_wait(bar(KV_FULL + st), (uint32_t)(j / kStages) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
        tc_fence_after();
        // K-major slab: rows 128 B apart, 8-row groups 1024 B apart; a 16-element k-step is 32 B inside the
        // swizzled row, the second 64-element slab 16 KiB further.  A: 8 columns of Q per k-step.
        const uint64_t dK = smem_desc(sKV + st * 2 * kTileBytes, 16, 1024);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_f16_ts(tS + (j & 1) * 128, tQ + ks * 8, dK + (uint64_t)((ks >> 2) * (kSlabBytes >> 4) + (ks & 3) * 2),
                      idesc_qk, ks > 0 ? 1u : 0u);
        umma_commit(bar(S_FULL + st));
      };
      issue_qk(0);
      for (int j = 0; j < n; ++j) {
        if (j + 1 < n) issue_qk(j + 1);  // runs while the softmax warps work on tile j
        const int st = j % kStages;
        mbar_wait(bar(P_FULL), (uint32_t)j & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
        tc_fence_after();
        // MN-major slab of V: 64 d-elements contiguous (128 B), 8-token groups 1024 B apart (stride offset),
        // the other 64 d-elements 16 KiB further (leading offset); a k-step is 16 tokens = 2048 B.
        const uint64_t dV = smem_desc(sKV + st * 2 * kTileBytes + kTileBytes, kSlabBytes, 1024);
        const uint32_t tP = tS + (j & 1) * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_f16_ts(tO, tP + ks * 8, dV + (uint64_t)(ks * (2048 >> 4)), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        if (SPLIT) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_f16_ts(tO, tP + 64 + ks * 8, dV + (uint64_t)(ks * (2048 >> 4)), idesc_pv, 1u);
        }
        umma_commit(bar(PV_DONE + st));
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax: two threads per query row
    // Warps w and w + 4 own the same 32 rows (TMEM lanes 32 (w % 4) ...) and split the 128 columns of a tile
    // in halves, so that every scheduler has two softmax warps to interleave.  The halves share the running
    // maximum (one exchange through shared memory per tile) and keep partial sums until the end.
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;
    const int col0 = half * kHalf;
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t tO = lane_base + 256 + (uint32_t)col0;
    float* xmax = xchg + half * kTile + row;             // [parity][half][row]
    const float* xmax_other = xchg + (half ^ 1) * kTile + row;
    const float sl2 = p.scale_log2;

    // Q moves to tensor memory once: Q.K^T then fetches only K from shared memory (with both operands in
    // shared memory a 128 x 128 x 16 MMA needs all of its bandwidth).  This thread's 64 elements are one row
    // of one slab; chunk c of the row lies at chunk c ^ (row % 8).
    mbar_wait(bar(Q_FULL), 0, p.status, MUX_DEV_WAIT_TIMEOUT);
    {
      uint32_t qv[32];
      const uint32_t qrow = sQ + (uint32_t)half * kSlabBytes + (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8)
        lds128(qrow + (uint32_t)((c8 ^ (row & 7)) << 4), qv[c8 * 4], qv[c8 * 4 + 1], qv[c8 * 4 + 2], qv[c8 * 4 + 3]);
      __syncwarp();
      tmem_st32u(lane_base + 384 + (uint32_t)(half * 32), qv);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(QT_FULL));
    }

    float m_run = -INFINITY, l_run = 0.f;
    float s[kHalf];
    for (int j = 0; j < n; ++j) {
      const int b = j & 1;
      mbar_wait(bar(S_FULL + j % kStages), (uint32_t)(j / kStages) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
      __syncwarp();  // the TMEM loads below are warp-collective
      tc_fence_after();
      const uint32_t tS = lane_base + (uint32_t)(b * 128 + col0);
      tmem_ld32<0>(tS, s);
      tmem_ld32<32>(tS + 32, s);
      tmem_wait_ld();

      if (j == qt) {  // diagonal tile: key c of the tile is visible to row r iff c <= r
#pragma unroll
        for (int c = 0; c < kHalf; ++c)
          if (col0 + c > row) s[c] = -INFINITY;
      }
      float mx4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) mx4[i] = s[i];
#pragma unroll
      for (int c = 4; c < kHalf; c += 4)
#pragma unroll
        for (int i = 0; i < 4; ++i) mx4[i] = fmaxf(mx4[i], s[c + i]);
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      xmax[b * 2 * kTile] = mx;
      named_bar_sync(1 + quarter, 64);
      mx = fmaxf(mx, xmax_other[b * 2 * kTile]) * sl2;
      // Lazy rescaling: the reference point of the exponentials moves only when the row maximum grew by more
      // than 2^8; until then weights up to 256 are exact enough in 16 bits and O needs no correction.
      const bool grow = mx > m_run + kRescaleStep;
      float alpha = 1.f;
      if (grow) {
        alpha = exp2f(m_run - mx);
        m_run = mx;
      }
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < kHalf; c += 4)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          s[c + i] = exp2f(fmaf(s[c + i], sl2, -m_run));
          sum4[i] += s[c + i];
        }
      l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));

      // O takes a correction only when some row of the warp moved its reference point (both halves of a row
      // decide alike); it is free for that once P.V of the previous tile has completed.  The wait is skipped
      // otherwise.
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        mbar_wait(bar(PV_DONE + (j - 1) % kStages), (uint32_t)((j - 1) / kStages) & 1u, p.status,
                  MUX_DEV_WAIT_TIMEOUT);
        __syncwarp();
        tc_fence_after();
        float o[32];
#pragma unroll 1
        for (int c2 = 0; c2 < 2; ++c2) {
          tmem_ld32<0>(tO + c2 * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= alpha;
          tmem_st32(tO + c2 * 32, o);
        }
      }
      // P replaces the logits of this tile in tensor memory: two 16-bit weights per column, this thread's 64
      // keys in 32 columns (the hi parts; the lo parts of the split go 64 columns further).  The other half of
      // the row has finished reading its logits: it passed the exchange barrier above after its loads.
      {
        const uint32_t tP = lane_base + (uint32_t)(b * 128 + half * 32);
        uint32_t hi[32];
        if (SPLIT) {
          uint32_t lo[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) split_pair<T>(s[2 * i], s[2 * i + 1], hi[i], lo[i]);
          tmem_st32u(tP, hi);
          tmem_st32u(tP + 64, lo);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) hi[i] = pack_pair<T>(s[2 * i], s[2 * i + 1]);
          tmem_st32u(tP, hi);
        }
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();  // every lane's stores have completed; lane 0 publishes them for the warp
      if (lane == 0) mbar_arrive(bar(P_FULL));
    }

    // the two halves of a row add their partial sums (slots of parity n & 1: last written for tile n - 2)
    xmax[(n & 1) * 2 * kTile] = l_run;
    named_bar_sync(1 + quarter, 64);
    l_run += xmax_other[(n & 1) * 2 * kTile];
    mbar_wait(bar(PV_DONE + (n - 1) % kStages), (uint32_t)((n - 1) / kStages) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
    __syncwarp();
    tc_fence_after();
    const float inv = 1.f / l_run;
    const bool valid = qt * kTile + row < len;
    T* orow = static_cast<T*>(p.out) + (int64_t)(start + qt * kTile + row) * p.out_seq_stride +
              (int64_t)head * p.out_head_stride + col0;
#pragma unroll 1
    for (int c2 = 0; c2 < 2; ++c2) {
      float o[32];
      tmem_ld32<0>(tO + c2 * 32, o);
      tmem_wait_ld();
      if (valid) {
#pragma unroll
        for (int v8 = 0; v8 < 4; ++v8) {
          uint4 w;
          w.x = pack_pair<T>(o[v8 * 8 + 0] * inv, o[v8 * 8 + 1] * inv);
          w.y = pack_pair<T>(o[v8 * 8 + 2] * inv, o[v8 * 8 + 3] * inv);
          w.z = pack_pair<T>(o[v8 * 8 + 4] * inv, o[v8 * 8 + 5] * inv);
          w.w = pack_pair<T>(o[v8 * 8 + 6] * inv, o[v8 * 8 + 7] * inv);
          *reinterpret_cast<uint4*>(orow + c2 * 32 + v8 * 8) = w;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// ---- host side -------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, resolved through the runtime (the library does not link libcuda).
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

// View [tokens][heads][128] (strides in elements) as a 3-D tensor (d, head, token) fetched in boxes of
// 64 d-elements x 1 head x 128 tokens with the 128-byte swizzle; rows past the end read as zeros.
static int make_map(EncodeTiledFn enc, CUtensorMap* map, const void* ptr, int dtype, int64_t tokens, int64_t heads,
                    int64_t seq_stride, int64_t head_stride) {
  const cuuint64_t dims[3] = {128, (cuuint64_t)heads, (cuuint64_t)tokens};
  const cuuint64_t strides[2] = {(cuuint64_t)head_stride * 2, (cuuint64_t)seq_stride * 2};
  const cuuint32_t box[3] = {64, 1, (cuuint32_t)kTile};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(map, dtype == MUX_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                         3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MUX_OK : record_cuda_error(cudaErrorInvalidValue);
}

static bool stride_ok(int64_t seq_stride, int64_t head_stride) {
  return seq_stride > 0 && head_stride > 0 && seq_stride % 8 == 0 && head_stride % 8 == 0;
}

template <typename T, bool SPLIT>
static int launch(const mux_prefill_args_t* a, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                  const Params& prm, cudaStream_t stream) {
  constexpr int kDevs = 64;
  static int granted[kDevs] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return record_cuda_error(e);
  if (dev < 0 || dev >= kDevs) return record_cuda_error(cudaErrorInvalidDevice);
  auto kern = prefill_attn_kernel<T, SPLIT>;
  constexpr int smem = smem_bytes<SPLIT>();
  if (granted[dev] < smem) {
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess)
      return record_cuda_error(e);
    granted[dev] = smem;
  }
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((a->max_prompt_len + kTile - 1) / kTile), (unsigned)a->num_q_heads,
                     (unsigned)a->num_seqs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = pdl;
  cfg.numAttrs = 1;
  if ((e = cudaLaunchKernelEx(&cfg, kern, mq, mk, mv, prm)) != cudaSuccess) return record_cuda_error(e);
  return MUX_OK;
}

static int run(const mux_prefill_args_t* a, cudaStream_t stream) {
  if (a == nullptr) return MUX_ERR_NULL_POINTER;
  if (a->dtype != MUX_DTYPE_F16 && a->dtype != MUX_DTYPE_BF16) return MUX_ERR_BAD_DTYPE;
  if (a->head_size != 128) return MUX_ERR_BAD_HEAD_SIZE;
  if (a->num_seqs < 0 || a->total_tokens < 0 || a->max_prompt_len < 0 || a->num_q_heads <= 0 ||
      a->num_kv_heads <= 0 || !(a->scale > 0.f) || a->num_seqs > 65535 || a->num_q_heads > 65535)
    return MUX_ERR_BAD_SHAPE;
  if (a->num_q_heads % a->num_kv_heads != 0) return MUX_ERR_BAD_GROUP;
  if (a->num_seqs == 0 || a->total_tokens == 0 || a->max_prompt_len == 0) return MUX_OK;
  if (!a->out || !a->q || !a->k || !a->v || !a->cu_seqlens) return MUX_ERR_NULL_POINTER;
  if (!aligned16(a->out) || !aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v)) return MUX_ERR_MISALIGNED;
  if (!stride_ok(a->out_seq_stride, a->out_head_stride) || !stride_ok(a->q_seq_stride, a->q_head_stride) ||
      !stride_ok(a->k_seq_stride, a->k_head_stride) || !stride_ok(a->v_seq_stride, a->v_head_stride))
    return MUX_ERR_MISALIGNED;
  unsigned* status = device_status_ptr();
  if (status == nullptr) return MUX_ERR_CUDA;
  EncodeTiledFn enc = nullptr;
  int st = encode_fn(&enc);
  if (st != MUX_OK) return st;
  alignas(64) CUtensorMap mq, mk, mv;
  if ((st = make_map(enc, &mq, a->q, a->dtype, a->total_tokens, a->num_q_heads, a->q_seq_stride, a->q_head_stride)) ||
      (st = make_map(enc, &mk, a->k, a->dtype, a->total_tokens, a->num_kv_heads, a->k_seq_stride, a->k_head_stride)) ||
      (st = make_map(enc, &mv, a->v, a->dtype, a->total_tokens, a->num_kv_heads, a->v_seq_stride, a->v_head_stride)))
    return st;
  Params prm;
  prm.out = a->out;
  prm.out_seq_stride = a->out_seq_stride;
  prm.out_head_stride = a->out_head_stride;
  prm.cu_seqlens = a->cu_seqlens;
  prm.total_tokens = a->total_tokens;
  prm.max_prompt_len = a->max_prompt_len;
  prm.group = a->num_q_heads / a->num_kv_heads;
  prm.scale_log2 = a->scale * 1.4426950408889634f;
  prm.status = status;
  if (a->dtype == MUX_DTYPE_F16) return launch<__half, false>(a, mq, mk, mv, prm, stream);
  return launch<__nv_bfloat16, true>(a, mq, mk, mv, prm, stream);
}

}  // namespace prefill
}  // namespace mux

extern "C" int mux_prefill_attention(const mux_prefill_args_t* args, void* cuda_stream) {
  return mux::prefill::run(args, static_cast<cudaStream_t>(cuda_stream));
}
