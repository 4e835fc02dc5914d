// Prompt-phase (prefill) attention: causal self-attention of every prompt of a batch over its
// own tokens, the step PagedAttentionWithRoPE runs for the prompt rows of a batch before their
// K/V are written to the pool (muxserve/flexserver/models/llama.py:160-161 with
// input_metadata.prompt_lens from muxserve/flexserver/llm_runtime.py:298-330).
//
// This is the one GEMM-shaped kernel of the library, so it runs on the 5th-generation tensor
// cores: one CTA owns 128 query rows of one (prompt, q head) and walks the keys/values in steps
// of 64 tokens up to the diagonal; two CTAs share an SM.
//   warp 4 / 5 (one lane)  TMA producers of Q + K steps / of V steps (cp.async.bulk.tensor, 128-byte
//                          swizzle, 2-stage rings, completion on mbarriers)
//   warp 6 (one lane)      issues tcgen05.mma S = Q.K^T (both operands in shared memory) into one of
//                          two TMEM buffers
//   warp 7 (one lane)      issues tcgen05.mma O += P.V (P in tensor memory, V in shared memory)
//   warps 0-3              one thread per query row: tcgen05.ld of the S row, scale, causal mask,
//                          online softmax (lazy rescaling of O), P written back to tensor memory in
//                          place of the logits, final O / l to global memory
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

constexpr int kTile = 128;                   // query rows per CTA
constexpr int kStep = 64;                    // key/value tokens per step
constexpr int kQSlabBytes = kTile * 128;     // 128 rows x 64 elements: one 128-byte-swizzled slab of Q
constexpr int kQBytes = 2 * kQSlabBytes;     // head size 128 = two slabs
constexpr int kSlabBytes = kStep * 128;      // one slab of a K or V step: 64 rows x 64 elements
constexpr int kStepBytes = 2 * kSlabBytes;   // 16 KiB
constexpr int kStages = 2;
constexpr int kSoftmaxWarps = 4;
constexpr int kKWarp = 4, kVWarp = 5, kQkWarp = 6, kPvWarp = 7;
constexpr int kThreads = 256;
constexpr uint32_t kTmemCols = 256;          // S0 | S1 (64 fp32 columns each) | O (128): two CTAs share an SM's 512
constexpr float kRescaleStep = 8.f;          // O is rescaled only when the running max grows by 2^8

enum Bar {
  Q_FULL = 0,
  P_FULL = 1,                 // + step & 1
  K_FULL = 3,                 // + stage (step & 1)
  V_FULL = K_FULL + kStages,
  S_FULL = V_FULL + kStages,  // Q.K^T of the step has completed: logits readable, K stage free
  PV_DONE = S_FULL + kStages, // P.V of the step has completed: V stage free, O up to date
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
  // optional cache write of the K/V rows (kc == nullptr: none)
  void* kc;
  void* vc;
  const long long* slots;
  long long s_ts, s_hs, num_blocks;
  int block_size;
  int bs_shift;                             // log2(block_size): 8, 16 or 32 tokens, so slot -> (block, offset) is a shift
  const int* bt;                            // block lists instead of slots (slots == nullptr)
  long long bt_ss, bt_hs;
  int max_blocks;
  const int* units;                         // optional work list: (prompt, q head | query tile << 16) per CTA
  int num_seqs, num_q_heads;
};

constexpr int smem_bytes() { return kQBytes + 2 * kStages * kStepBytes + 2048; }  // tiles + barriers + 128 slots

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
__host__ __device__ constexpr uint32_t instr_desc(uint32_t a_fmt, uint32_t b_fmt, uint32_t b_mn_major, uint32_t n) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (b_mn_major << 16) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
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

__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr)
               : "memory");
}
__device__ __forceinline__ void named_bar_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
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

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// ---- prompt cache write from the staged steps ------------------------------------------------
// The CTA of query tile qt holds the K and V steps 2 qt and 2 qt + 1 (its own rows' tokens) in shared memory at
// the end of its walk; the q head that comes first in its group copies them to the pool: the two producer warps,
// idle by then, do it while the softmax and the MMAs of those last steps run.

// Slot of the token in row r of step j for this kv head, or -1 (row past the prompt, padding slot, slot outside
// the pool: reported and skipped).
__device__ __forceinline__ long long step_slot(const Params& p, int seq, int start, int len, int kvh, int j, int r) {
  const int pos = j * kStep + r;
  if (pos >= len) return -1;
  long long slot;
  if (p.slots != nullptr) {
    slot = p.slots[(long long)(start + pos) * p.s_ts + (long long)kvh * p.s_hs];
  } else {  // from the block list of (prompt, kv head)
    const int b = pos >> p.bs_shift;
    if (b >= p.max_blocks) {
      atomicOr(p.status, MUX_DEV_BAD_CONTEXT);
      return -1;
    }
    const long long id = p.bt[(long long)seq * p.bt_ss + (long long)kvh * p.bt_hs + b];
    slot = id < 0 ? -1 : id * p.block_size + (pos - b * p.block_size);
  }
  if (slot < 0) return -1;
  if ((slot >> p.bs_shift) >= p.num_blocks) {
    atomicOr(p.status, MUX_DEV_BAD_SLOT);
    return -1;
  }
  return slot;
}

// K step (64 tokens x 128 d, two 128-byte-swizzled slabs) -> key pool [block][d/8][token][8]: lane = row, one
// 16-byte piece per d chunk; consecutive tokens of a block are neighbouring pieces.  `slots`: the step's 64
// slots in shared memory (fetched at the start of the CTA: the [token][layer][head] array puts consecutive
// tokens kilobytes apart, and a fetch at the point of use would stall the copy for a DRAM round trip each time).
template <typename T>
__device__ __forceinline__ void copy_k_step(const Params& p, uint32_t tile, const long long* slots, int lane) {
  const int BS = p.block_size;
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    const int r = half * 32 + lane;
    const long long slot = slots[r];
    if (slot < 0) continue;
    const long long blk = slot >> p.bs_shift;
    T* dst = static_cast<T*>(p.kc) + blk * (128 * BS) + (slot - blk * BS) * 8;
    const uint32_t src = tile + (uint32_t)r * 128u;
    // all of a slab's loads first, then its stores: a store directly behind its load makes every piece wait out
    // a shared-memory round trip (the loads are ordered asm statements; one at a time they took ~75 cycles each)
#pragma unroll
    for (int slab = 0; slab < 2; ++slab) {
      uint4 w[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) w[c] = lds128(src + (uint32_t)slab * kSlabBytes + (uint32_t)((c ^ (r & 7)) << 4));
#pragma unroll
      for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(dst + (slab * 8 + c) * (BS * 8)) = w[c];
    }
  }
}

// V step -> value pool [block][d][token], groups g0 .. g1 - 1 of eight tokens each.  Eight tokens whose slots are
// consecutive and start on a multiple of 8 (every full group of a prompt) are transposed by ldmatrix.trans:
// per 8 x 8 piece a lane gets two neighbouring tokens of one d, i.e. 4 bytes of that d's row in the block, and
// four lanes complete its 16 bytes.  Other rows go element by element.
template <typename T>
__device__ __forceinline__ void copy_v_groups(const Params& p, uint32_t tile, const long long* slots, int lane, int g0,
                                              int g1) {
  const int BS = p.block_size;
  const long long slot_a = slots[lane];        // rows 0..31
  const long long slot_b = slots[32 + lane];   // rows 32..63
  unsigned short* vc = reinterpret_cast<unsigned short*>(p.vc);
#pragma unroll 1
  for (int g = g0; g < g1; ++g) {  // rows 8 g .. 8 g + 7
    const long long mine = g < 4 ? slot_a : slot_b;
    const int l0 = (g & 3) * 8;
    const long long base = __shfl_sync(0xffffffffu, mine, l0);
    const bool in_group = (lane >> 3) == (g & 3);
    const unsigned good = __ballot_sync(0xffffffffu, in_group && mine >= 0 && mine == base + (lane & 7));
    const bool run = base >= 0 && (base & 7) == 0 && ((good >> l0) & 0xffu) == 0xffu;
    const int r0 = g * 8;
    if (run) {
      const long long blk = base >> p.bs_shift;
      // this lane's destination inside a piece: d = lane / 4 of the piece, tokens 2 (lane % 4), + 1
      unsigned short* dst = vc + blk * (128 * BS) + (base - blk * BS) + (long long)(lane >> 2) * BS + 2 * (lane & 3);
      const int r = r0 + (lane & 7);  // the row whose 16-byte piece this lane names to ldmatrix
      const uint32_t rowaddr = tile + (uint32_t)r * 128u;
      uint32_t m[4][4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {  // pieces (d chunks) 4 q4 .. 4 q4 + 3, one per lane octet; loads first (see K)
        const int c = 4 * q4 + (lane >> 3);
        ldmatrix_x4_trans(m[q4], rowaddr + (uint32_t)(c >> 3) * kSlabBytes + (uint32_t)(((c & 7) ^ (r & 7)) << 4));
      }
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4)
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint32_t*>(dst + (long long)(8 * (4 * q4 + i)) * BS) = m[q4][i];
    } else {
#pragma unroll 1
      for (int i = 0; i < 8; ++i) {
        const long long slot = __shfl_sync(0xffffffffu, mine, l0 + i);
        if (slot < 0) continue;  // the same for every lane
        const int r = r0 + i;
        const long long blk = slot >> p.bs_shift;
        unsigned short* dst = vc + blk * (128 * BS) + (slot - blk * BS);
#pragma unroll 1
        for (int pass = 0; pass < 4; ++pass) {
          const int d = pass * 32 + lane;
          unsigned short x;
          asm volatile("ld.shared.u16 %0, [%1];"
                       : "=h"(x)
                       : "r"(tile + (uint32_t)(d >> 6) * kSlabBytes + (uint32_t)r * 128u +
                             (uint32_t)((((d & 63) >> 3) ^ (r & 7)) << 4) + (uint32_t)(d & 7) * 2u)
                       : "memory");
          dst[(long long)d * BS] = x;
        }
      }
    }
  }
}

constexpr int kVGroupsOfVWarp = 4;  // of the 8 groups of a step; the K warp, which also copies K but starts earlier, takes the rest

// ---- the kernel ------------------------------------------------------------------------------
//
// Two CTAs share an SM (98 KiB of shared memory and 256 tensor-memory columns each), so that one CTA's
// prologue, epilogue and serial softmax -> MMA hand-offs run under the other's work.
// Tensor memory (256 columns x 128 lanes, lane = query row):
//   [0,64) and [64,128)  logits S of step j in buffer j & 1; the softmax threads overwrite them with the 16-bit
//                        weights P (32 columns hi [+ 32 columns lo]), the A operand of P.V
//   [128,256)            O accumulator
// Barriers (index = step & 1 unless noted):
//   K_FULL / V_FULL  TMA bytes of the step's K / V have landed
//   S_FULL           Q.K^T of the step has completed: logits readable, K stage free
//   P_FULL           all 4 softmax warps have written P of the step (they loaded its S before).  Two of them: a
//                    warp may be one step ahead of the slowest one (the logits of step j + 1 are ready early), and
//                    its arrival for step j + 1 must not complete the phase of step j
//   PV_DONE          P.V of the step has completed: V stage free, O holds steps 0..j

template <typename T, bool SPLIT>
__global__ void __launch_bounds__(kThreads, 2)
prefill_attn_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
                    const __grid_constant__ CUtensorMap tmv, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];  // the swizzle pattern repeats every 1024 bytes
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  int seq = blockIdx.z, head = blockIdx.y;
  int qt = (int)gridDim.x - 1 - (int)blockIdx.x;  // the tiles with the most work start first
  if (p.units != nullptr) {  // the host listed the real (prompt, q head, query tile) triples
    seq = p.units[2 * blockIdx.x];
    const int hq = p.units[2 * blockIdx.x + 1];
    head = hq & 0xffff;
    qt = (int)((unsigned)hq >> 16);
    if (seq < 0) return;  // padding
    if (seq >= p.num_seqs || head >= p.num_q_heads) {
      if (threadIdx.x == 0) atomicOr(p.status, MUX_DEV_BAD_CONTEXT);
      return;
    }
  }

  if (tid == kKWarp * 32) {  // the copy descriptors do not depend on the previous kernel: fetch them early
    prefetch_tensormap(&tmq);
    prefetch_tensormap(&tmk);
  } else if (tid == kVWarp * 32) {
    prefetch_tensormap(&tmv);
  }
  griddep_wait();
  const int start = p.cu_seqlens[seq];
  const int len = p.cu_seqlens[seq + 1] - start;
  if (start < 0 || len < 0 || len > p.max_prompt_len || start + len > p.total_tokens) {
    if (tid == 0) atomicOr(p.status, MUX_DEV_BAD_CONTEXT);  // nothing of this prompt is read or written
    return;
  }
  if (qt * kTile >= len) return;
  // key/value steps of 64 tokens up to the end of the diagonal tile (or of the prompt)
  const int kv_end = min(len, (qt + 1) * kTile);
  const int n = (kv_end + kStep - 1) / kStep;
  const int first_masked = 2 * qt;  // steps from here on reach past some row's own position

  const uint32_t raw = smem_u32(smem_raw);
  if (raw & 1023u) {  // the tiles' swizzle needs the declared alignment; never seen violated, never worked around
    if (tid == 0) atomicOr(p.status, MUX_DEV_INTERNAL);
    return;
  }
  const uint32_t sQ = raw;
  const uint32_t sK = sQ + kQBytes;
  const uint32_t sV = sK + kStages * kStepBytes;
  const uint32_t sBar = sV + kStages * kStepBytes;
  auto bar = [&](int i) { return sBar + 8u * (uint32_t)i; };
  const uint32_t sSlot = sBar + 8u * NUM_BARS;
  volatile uint32_t* slot = reinterpret_cast<volatile uint32_t*>(smem_raw + (sSlot - raw));

  // Each producer lane arms its own barriers and sends its first copies at once (the first kStages steps
  // need no free-stage signal); everybody else meets them at the CTA barrier below.
  const int kvh = head / p.group;
  const bool write_pool = p.kc != nullptr && head % p.group == 0;
  const int first = min(n, kStages);
  if (tid == kKWarp * 32) {
    mbar_init(bar(Q_FULL), 1);
    for (int i = 0; i < kStages; ++i) mbar_init(bar(K_FULL + i), 1);
    mbar_init_fence();
    const int q0 = start + qt * kTile;
    mbar_arrive_expect_tx(bar(Q_FULL), kQBytes);
    tma_load_3d(sQ, &tmq, 0, head, q0, bar(Q_FULL));
    tma_load_3d(sQ + kQSlabBytes, &tmq, 64, head, q0, bar(Q_FULL));
    for (int j = 0; j < first; ++j) {
      mbar_arrive_expect_tx(bar(K_FULL + j), kStepBytes);
      tma_load_3d(sK + j * kStepBytes, &tmk, 0, kvh, start + j * kStep, bar(K_FULL + j));
      tma_load_3d(sK + j * kStepBytes + kSlabBytes, &tmk, 64, kvh, start + j * kStep, bar(K_FULL + j));
    }
  } else if (tid == kVWarp * 32) {
    for (int i = 0; i < kStages; ++i) mbar_init(bar(V_FULL + i), 1);
    mbar_init_fence();
    for (int j = 0; j < first; ++j) {
      mbar_arrive_expect_tx(bar(V_FULL + j), kStepBytes);
      tma_load_3d(sV + j * kStepBytes, &tmv, 0, kvh, start + j * kStep, bar(V_FULL + j));
      tma_load_3d(sV + j * kStepBytes + kSlabBytes, &tmv, 64, kvh, start + j * kStep, bar(V_FULL + j));
    }
  } else if (tid == 0) {
    mbar_init(bar(P_FULL), kSoftmaxWarps);
    mbar_init(bar(P_FULL + 1), kSoftmaxWarps);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(PV_DONE + i), 1);
    }
    mbar_init_fence();
  }
  __syncthreads();  // all barriers are live; tensor memory is allocated while the first copies fly
  griddep_launch_dependents();
  uint32_t tmem = 0;
  if (warp != kKWarp && warp != kVWarp) {  // the users of tensor memory meet again after the allocation
    if (warp == kQkWarp) tmem_alloc(sSlot, kTmemCols);
    tc_fence_before();
    named_bar_sync(1, kThreads - 64);
    tc_fence_after();
    tmem = *slot;
  }

  // The slots of this tile's 128 tokens ([2 steps][64 rows]) are fetched by the softmax threads, one each, while they
  // wait for the first logits; each producer warp meets them at a named barrier of its own before its first copy.  (Fetched
  // by the producer warps' idle lanes, ahead of or beside lane 0's loop, the DRAM round trips held lane 0 up.)
  long long* sslots = reinterpret_cast<long long*>(smem_raw + (sBar + 256 - raw));
  if (warp == kKWarp) {
    // ------------------------------------------------------------------ TMA producer: the later K steps
    if (lane == 0) {
      for (int j = first; j < n; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        const uint32_t dst = sK + st * kStepBytes;
        mbar_wait_sleepy(bar(S_FULL + st), ph ^ 1u, p.status, MUX_DEV_WAIT_TIMEOUT);  // Q.K^T of step j - 2
        mbar_arrive_expect_tx(bar(K_FULL + st), kStepBytes);
        tma_load_3d(dst, &tmk, 0, kvh, start + j * kStep, bar(K_FULL + st));
        tma_load_3d(dst + kSlabBytes, &tmk, 64, kvh, start + j * kStep, bar(K_FULL + st));
      }
    }
    __syncwarp();
    if (write_pool) named_bar_sync(4, 32 + kSoftmaxWarps * 32);  // the slots are in shared memory (K warp's barrier)
    // The last steps: no copy of this CTA may still be in flight when it ends (matters only after a failed
    // wait), and the steps of this tile's own tokens (2 qt and 2 qt + 1, never overwritten) go to the pool.
    for (int j = (n > kStages ? n - kStages : 0); j < n; ++j) {
      mbar_wait_sleepy(bar(K_FULL + (j & 1)), (uint32_t)(j >> 1) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
      __syncwarp();
      if (write_pool && j >= first_masked) {
        copy_k_step<T>(p, sK + (j & 1) * kStepBytes, sslots + (j - first_masked) * kStep, lane);
        // this warp is done with its copies of K long before the V warp, whose last copy waits for P.V of step
        // n - 3: it takes its share of the step's V as soon as that has landed
        mbar_wait_sleepy(bar(V_FULL + (j & 1)), (uint32_t)(j >> 1) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
        __syncwarp();
        copy_v_groups<T>(p, sV + (j & 1) * kStepBytes, sslots + (j - first_masked) * kStep, lane, kVGroupsOfVWarp, 8);
      }
    }
  } else if (warp == kVWarp) {
    // ------------------------------------------------------------------ TMA producer: the later V steps
    if (lane == 0) {
      for (int j = first; j < n; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        const uint32_t dst = sV + st * kStepBytes;
        mbar_wait_sleepy(bar(PV_DONE + st), ph ^ 1u, p.status, MUX_DEV_WAIT_TIMEOUT);  // P.V of step j - 2
        mbar_arrive_expect_tx(bar(V_FULL + st), kStepBytes);
        tma_load_3d(dst, &tmv, 0, kvh, start + j * kStep, bar(V_FULL + st));
        tma_load_3d(dst + kSlabBytes, &tmv, 64, kvh, start + j * kStep, bar(V_FULL + st));
      }
    }
    __syncwarp();
    if (write_pool) named_bar_sync(5, 32 + kSoftmaxWarps * 32);  // the slots are in shared memory (V warp's barrier)
    for (int j = (n > kStages ? n - kStages : 0); j < n; ++j) {
      mbar_wait_sleepy(bar(V_FULL + (j & 1)), (uint32_t)(j >> 1) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
      __syncwarp();
      if (write_pool && j >= first_masked) {
        copy_v_groups<T>(p, sV + (j & 1) * kStepBytes, sslots + (j - first_masked) * kStep, lane, 0, kVGroupsOfVWarp);
      }
    }
  } else if (warp == kQkWarp) {
    // ------------------------------------------------------------------ issuer of S = Q K^T
    // Two issuing threads, so that neither the other's waits nor the time its MMAs queue behind the other
    // CTA's delay an issue.  Across threads nothing is ordered implicitly: the logits buffer of step j is
    // free once P.V of step j - 2, which read P from it, has completed.
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc_qk = instr_desc(fmt, fmt, 0, kStep);  // S[128 x 64], both operands K-major (d contiguous)
      // K-major slab: rows 128 B apart, 8-row groups 1024 B apart; a 16-element k-step is 32 B inside the
      // swizzled row, the second 64-element slab one slab further.
      const uint64_t dQ = smem_desc(sQ, 16, 1024);
      mbar_wait_sleepy(bar(Q_FULL), 0, p.status, MUX_DEV_WAIT_TIMEOUT);
      for (int j = 0; j < n; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        mbar_wait_sleepy(bar(K_FULL + st), ph, p.status, MUX_DEV_WAIT_TIMEOUT);
        mbar_wait_sleepy(bar(PV_DONE + st), ph ^ 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
        tc_fence_after();
        const uint64_t dK = smem_desc(sK + st * kStepBytes, 16, 1024);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_f16_ss(tmem + st * kStep, dQ + (uint64_t)((ks >> 2) * (kQSlabBytes >> 4) + (ks & 3) * 2),
                      dK + (uint64_t)((ks >> 2) * (kSlabBytes >> 4) + (ks & 3) * 2), idesc_qk, ks > 0 ? 1u : 0u);
        umma_commit(bar(S_FULL + st));
      }
    }
  } else if (warp == kPvWarp) {
    // ------------------------------------------------------------------ issuer of O += P V
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      // O[128 x 128] = P V: V is MN-major (d contiguous, tokens = K).  A and B must have ONE format: fp16 weights
      // over bf16 values (a_fmt 0, b_fmt 1) raise "illegal instruction" on B200, hence the hi/lo split for bf16.
      constexpr uint32_t idesc_pv = instr_desc(fmt, fmt, 1, 128);
      const uint32_t tO = tmem + 128;
      for (int j = 0; j < n; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        mbar_wait_sleepy(bar(V_FULL + st), ph, p.status, MUX_DEV_WAIT_TIMEOUT);
        mbar_wait_sleepy(bar(P_FULL + st), ph, p.status, MUX_DEV_WAIT_TIMEOUT);
        tc_fence_after();
        // MN-major slab of V: 64 d-elements contiguous (128 B), 8-token groups 1024 B apart (stride offset),
        // the other 64 d-elements one slab further (leading offset); a k-step is 16 tokens = 2048 B.
        const uint64_t dV = smem_desc(sV + st * kStepBytes, kSlabBytes, 1024);
        const uint32_t tP = tmem + st * kStep;  // A = P: 8 columns of 16-bit pairs per k-step
#pragma unroll
        for (int ks = 0; ks < kStep / 16; ++ks)
          umma_f16_ts(tO, tP + ks * 8, dV + (uint64_t)(ks * (2048 >> 4)), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        if (SPLIT) {
#pragma unroll
          for (int ks = 0; ks < kStep / 16; ++ks)
            umma_f16_ts(tO, tP + 32 + ks * 8, dV + (uint64_t)(ks * (2048 >> 4)), idesc_pv, 1u);
        }
        umma_commit(bar(PV_DONE + st));
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax: one thread per query row
    const int row = tid;  // = TMEM lane; warp w reads lanes 32 w ...
    if (write_pool) {
      sslots[row] = step_slot(p, seq, start, len, kvh, first_masked + (row >> 6), row & (kStep - 1));
      named_bar_arrive(4, 32 + kSoftmaxWarps * 32);  // one barrier per producer warp: neither waits for the other
      named_bar_arrive(5, 32 + kSoftmaxWarps * 32);
    }
    const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
    const uint32_t tO = lane_base + 128;
    const float sl2 = p.scale_log2;
    float m_run = -INFINITY, l_run = 0.f;
    float s[kStep];
    for (int j = 0; j < n; ++j) {
      const int b = j & 1;
      mbar_wait(bar(S_FULL + b), (uint32_t)(j >> 1) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
      __syncwarp();  // the TMEM loads below are warp-collective
      tc_fence_after();
      const uint32_t tS = lane_base + (uint32_t)(b * kStep);
      tmem_ld32<0>(tS, s);
      tmem_ld32<32>(tS + 32, s);
      tmem_wait_ld();

      if (j >= first_masked) {  // key c of the step is visible to row r iff 64 j + c <= 128 qt + r
        const int limit = row - (j - first_masked) * kStep;
#pragma unroll
        for (int c = 0; c < kStep; ++c)
          if (c > limit) s[c] = -INFINITY;
      }
      float mx4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) mx4[i] = s[i];
#pragma unroll
      for (int c = 4; c < kStep - 4; c += 8)   // three-input maximum: half the instructions of a two-input chain
#pragma unroll
        for (int i = 0; i < 4; ++i) mx4[i] = fmax3(mx4[i], s[c + i], s[c + 4 + i]);
#pragma unroll
      for (int i = 0; i < 4; ++i) mx4[i] = fmaxf(mx4[i], s[kStep - 4 + i]);
      const float mx = fmaxf(fmax3(mx4[0], mx4[1], mx4[2]), mx4[3]) * sl2;
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
      for (int c = 0; c < kStep; c += 4)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          s[c + i] = exp2f(fmaf(s[c + i], sl2, -m_run));
          sum4[i] += s[c + i];
        }
      l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));

      // O takes a correction only when some row of the warp moved its reference point; it is free for that
      // once P.V of the previous step has completed.  The wait is skipped otherwise.
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        mbar_wait(bar(PV_DONE + ((j - 1) & 1)), (uint32_t)((j - 1) >> 1) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
        __syncwarp();
        tc_fence_after();
        float o[32];
#pragma unroll 1
        for (int c4 = 0; c4 < 4; ++c4) {
          tmem_ld32<0>(tO + c4 * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= alpha;
          tmem_st32(tO + c4 * 32, o);
        }
      }
      // P replaces the logits of this step in tensor memory: two 16-bit weights per column (the hi parts; the
      // lo parts of the split go 32 columns further).
      {
        uint32_t hi[32];
        if (SPLIT) {
          uint32_t lo[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) split_pair<T>(s[2 * i], s[2 * i + 1], hi[i], lo[i]);
          tmem_st32u(tS, hi);
          tmem_st32u(tS + 32, lo);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) hi[i] = pack_pair<T>(s[2 * i], s[2 * i + 1]);
          tmem_st32u(tS, hi);
        }
        tmem_wait_st();
      }
      tc_fence_before();
      __syncwarp();  // every lane's stores have completed; lane 0 publishes them for the warp
      if (lane == 0) mbar_arrive(bar(P_FULL + b));
    }

    mbar_wait(bar(PV_DONE + ((n - 1) & 1)), (uint32_t)((n - 1) >> 1) & 1u, p.status, MUX_DEV_WAIT_TIMEOUT);
    __syncwarp();
    tc_fence_after();
    const float inv = 1.f / l_run;
    // O / l goes through shared memory (Q's tile: every MMA that read it has completed) so that global memory
    // is written two whole rows per instruction instead of 32 scattered 16-byte pieces.  Row r keeps its 16
    // pieces at piece ^ (r % 8): writes (lane = row) and reads (16 lanes = one row) both hit 8 bank groups.
    const uint32_t srow = sQ + (uint32_t)row * 256u;
#pragma unroll 1
    for (int c4 = 0; c4 < 4; ++c4) {
      float o[32];
      tmem_ld32<0>(tO + c4 * 32, o);
      tmem_wait_ld();
#pragma unroll
      for (int v8 = 0; v8 < 4; ++v8)
        sts128(srow + (uint32_t)(((c4 * 4 + v8) ^ (row & 7)) << 4),
               pack_pair<T>(o[v8 * 8 + 0] * inv, o[v8 * 8 + 1] * inv), pack_pair<T>(o[v8 * 8 + 2] * inv, o[v8 * 8 + 3] * inv),
               pack_pair<T>(o[v8 * 8 + 4] * inv, o[v8 * 8 + 5] * inv), pack_pair<T>(o[v8 * 8 + 6] * inv, o[v8 * 8 + 7] * inv));
    }
    __syncwarp();  // a warp writes out only the 32 rows it staged itself
    {
      const int piece = lane & 15;
      T* obase = static_cast<T*>(p.out) + (int64_t)(start + qt * kTile) * p.out_seq_stride +
                 (int64_t)head * p.out_head_stride + piece * 8;
      const int rows_valid = len - qt * kTile;  // rows of this tile inside the prompt
#pragma unroll 4
      for (int i = 0; i < 16; ++i) {
        const int r = warp * 32 + 2 * i + (lane >> 4);
        if (r < rows_valid) {
          const uint4 w = lds128(sQ + (uint32_t)r * 256u + (uint32_t)((piece ^ (r & 7)) << 4));
          *reinterpret_cast<uint4*>(obase + (int64_t)r * p.out_seq_stride) = w;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kQkWarp) {
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
                    int64_t seq_stride, int64_t head_stride, int box_rows) {
  const cuuint64_t dims[3] = {128, (cuuint64_t)heads, (cuuint64_t)tokens};
  const cuuint64_t strides[2] = {(cuuint64_t)head_stride * 2, (cuuint64_t)seq_stride * 2};
  const cuuint32_t box[3] = {64, 1, (cuuint32_t)box_rows};
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
  constexpr int smem = smem_bytes();
  if (granted[dev] < smem) {
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess)
      return record_cuda_error(e);
    granted[dev] = smem;
  }
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = a->num_units > 0 ? dim3((unsigned)a->num_units)
                                 : dim3((unsigned)((a->max_prompt_len + kTile - 1) / kTile), (unsigned)a->num_q_heads,
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
  if (a->key_cache != nullptr) {
    if (a->block_size != 8 && a->block_size != 16 && a->block_size != 32) return MUX_ERR_BAD_BLOCK_SIZE;
    if (!a->value_cache || (!a->slot_mapping && !a->block_tables)) return MUX_ERR_NULL_POINTER;
    if (!a->slot_mapping && a->max_blocks_per_seq <= 0) return MUX_ERR_BAD_SHAPE;
    if (a->num_blocks <= 0) return MUX_ERR_BAD_SHAPE;
    if (!aligned16(a->key_cache) || !aligned16(a->value_cache)) return MUX_ERR_MISALIGNED;
  }
  if (a->num_units < 0 || (a->num_units > 0 && a->units == nullptr)) return a->num_units < 0 ? MUX_ERR_BAD_SHAPE : MUX_ERR_NULL_POINTER;
  unsigned* status = device_status_ptr();
  if (status == nullptr) return MUX_ERR_CUDA;
  EncodeTiledFn enc = nullptr;
  int st = encode_fn(&enc);
  if (st != MUX_OK) return st;
  alignas(64) CUtensorMap mq, mk, mv;
  if ((st = make_map(enc, &mq, a->q, a->dtype, a->total_tokens, a->num_q_heads, a->q_seq_stride, a->q_head_stride, kTile)) ||
      (st = make_map(enc, &mk, a->k, a->dtype, a->total_tokens, a->num_kv_heads, a->k_seq_stride, a->k_head_stride, kStep)) ||
      (st = make_map(enc, &mv, a->v, a->dtype, a->total_tokens, a->num_kv_heads, a->v_seq_stride, a->v_head_stride, kStep)))
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
  prm.kc = a->key_cache;
  prm.vc = a->value_cache;
  prm.slots = reinterpret_cast<const long long*>(a->slot_mapping);
  prm.s_ts = a->slot_token_stride;
  prm.s_hs = a->slot_head_stride;
  prm.num_blocks = a->num_blocks;
  prm.block_size = a->block_size;
  prm.bs_shift = a->block_size == 8 ? 3 : a->block_size == 16 ? 4 : 5;
  prm.bt = a->block_tables;
  prm.bt_ss = a->bt_seq_stride;
  prm.bt_hs = a->bt_head_stride;
  prm.max_blocks = a->max_blocks_per_seq;
  prm.units = a->num_units > 0 ? a->units : nullptr;
  prm.num_seqs = a->num_seqs;
  prm.num_q_heads = a->num_q_heads;
  if (a->dtype == MUX_DTYPE_F16) return launch<__half, false>(a, mq, mk, mv, prm, stream);
  return launch<__nv_bfloat16, true>(a, mq, mk, mv, prm, stream);
}

}  // namespace prefill
}  // namespace mux

extern "C" int mux_prefill_attention(const mux_prefill_args_t* args, void* cuda_stream) {
  return mux::prefill::run(args, static_cast<cudaStream_t>(cuda_stream));
}
