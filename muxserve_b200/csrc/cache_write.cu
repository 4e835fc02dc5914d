// reshape_and_cache: scatter new tokens' K/V rows into the head-granular pool.
//
// Few tokens (decode): one warp per (token, kv head) row.  The K row (128 elements)
// lands as 16 16-byte pieces, one per 8-wide d chunk, block_size*16 bytes apart; the
// V row lands as 128 single elements block_size*2 bytes apart.  Many tokens (prompt
// phase, multi-token decode): cache_write_runs_kernel below.
#include <cstdint>

#include "internal.h"
#include "ptx.cuh"

namespace mux {

struct CacheWriteParams {
  const void* k;
  const void* v;
  void* kc;
  void* vc;
  const long long* slots;
  long long k_ts, k_hs, v_ts, v_hs, s_ts, s_hs;
  long long num_blocks;
  unsigned* status;
  int num_tokens, num_heads;
};

constexpr int kCwWarps = 4;

template <typename T, int BS>
__global__ void __launch_bounds__(kCwWarps * 32)
cache_write_kernel(const __grid_constant__ CacheWriteParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * kCwWarps + warp;
  griddep_wait();               // inputs may come from the previous kernel of the stream
  griddep_launch_dependents();  // the next kernel may start being scheduled
  if (row >= (long long)p.num_tokens * p.num_heads) return;
  const int t = (int)(row / p.num_heads);
  const int h = (int)(row - (long long)t * p.num_heads);
  // the row's data and its slot are independent loads: issue all of them before the first use
  const T* krow = static_cast<const T*>(p.k) + t * p.k_ts + h * p.k_hs;
  const T* vrow = static_cast<const T*>(p.v) + t * p.v_ts + h * p.v_hs;
  const uint2 vval = *reinterpret_cast<const uint2*>(vrow + 4 * lane);
  uint4 kval = make_uint4(0u, 0u, 0u, 0u);
  if (lane < 16) kval = *reinterpret_cast<const uint4*>(krow + 8 * lane);
  const long long slot = p.slots[t * p.s_ts + h * p.s_hs];
  if (slot < 0) return;  // padding row
  const long long b = slot / BS;
  const int o = (int)(slot - b * BS);
  if (b >= p.num_blocks) {
    if (lane == 0) atomicOr(p.status, MUX_DEV_BAD_SLOT);
    return;
  }
  T* kblk = static_cast<T*>(p.kc) + b * (128 * BS);
  T* vblk = static_cast<T*>(p.vc) + b * (128 * BS);
  // V (all lanes): lane owns d = 4*lane .. 4*lane+3
  {
    unsigned short* dst = reinterpret_cast<unsigned short*>(vblk) + (4 * lane) * BS + o;
    dst[0] = (unsigned short)(vval.x & 0xffffu);
    dst[BS] = (unsigned short)(vval.x >> 16);
    dst[2 * BS] = (unsigned short)(vval.y & 0xffffu);
    dst[3 * BS] = (unsigned short)(vval.y >> 16);
  }
  // K: lanes 0..15 own one 8-wide chunk each
  if (lane < 16) *reinterpret_cast<uint4*>(kblk + lane * (BS * 8) + o * 8) = kval;
}

// Many tokens per sequence (prompt phase, multi-token decode): consecutive rows of one head fall into
// consecutive slots of one block, so their V elements, which the pool keeps token-minor, form contiguous
// runs.  A CTA stages kRunRows rows of one head in shared memory, finds the runs (same block, offsets
// ascending by one) and writes each run of V as whole 16-byte pieces where offset and length allow it
// (a full block of one head = 128 x block_size*2 contiguous bytes), K as 16-byte pieces with the run's rows
// in neighbouring lanes.  Any slot pattern is handled; without runs it degenerates to element stores.
constexpr int kRunRows = 32;
constexpr int kRunThreads = 128;
constexpr int kRunStride = 136;   // staged row = 128 elements + 8 of padding: 16-byte reads down a column of rows
                                  // hit eight different bank groups
constexpr int kRunMinTokens = 256;

template <typename T, int BS>
__global__ void __launch_bounds__(kRunThreads)
cache_write_runs_kernel(const __grid_constant__ CacheWriteParams p) {
  __shared__ __align__(16) T sk[kRunRows * kRunStride];
  __shared__ __align__(16) T sv[kRunRows * kRunStride];
  __shared__ long long sblk[kRunRows];  // block of the row, -1 = skip the row
  __shared__ int soff[kRunRows];
  __shared__ int srun[kRunRows];        // length of the run that starts at the row, 0 elsewhere
  const int tid = threadIdx.x;
  const int h = blockIdx.y;
  const int t0 = blockIdx.x * kRunRows;
  griddep_wait();
  griddep_launch_dependents();
  const int rows = min(kRunRows, p.num_tokens - t0);
  for (int r = tid >> 4; r < rows; r += kRunThreads / 16) {
    const int c = (tid & 15) * 8;
    const T* krow = static_cast<const T*>(p.k) + (long long)(t0 + r) * p.k_ts + h * p.k_hs;
    const T* vrow = static_cast<const T*>(p.v) + (long long)(t0 + r) * p.v_ts + h * p.v_hs;
    *reinterpret_cast<uint4*>(sk + r * kRunStride + c) = *reinterpret_cast<const uint4*>(krow + c);
    *reinterpret_cast<uint4*>(sv + r * kRunStride + c) = *reinterpret_cast<const uint4*>(vrow + c);
  }
  if (tid < kRunRows) {  // warp 0: one lane per row
    long long blk = -1;
    int off = 0;
    if (tid < rows) {
      const long long slot = p.slots[(long long)(t0 + tid) * p.s_ts + h * p.s_hs];
      if (slot >= 0) {  // negative = padding row
        blk = slot / BS;
        off = (int)(slot - blk * BS);
        if (blk >= p.num_blocks) {
          atomicOr(p.status, MUX_DEV_BAD_SLOT);
          blk = -1;
        }
      }
    }
    const long long prev_blk = __shfl_up_sync(0xffffffffu, blk, 1);
    const int prev_off = __shfl_up_sync(0xffffffffu, off, 1);
    const bool start = blk >= 0 && (tid == 0 || prev_blk != blk || prev_off + 1 != off);
    const unsigned starts = __ballot_sync(0xffffffffu, start);
    const unsigned valid = __ballot_sync(0xffffffffu, blk >= 0);
    int len = 0;
    if (start) {  // the run ends before the next start or the next skipped row
      const unsigned above = tid == 31 ? 0u : (0xffffffffu << (tid + 1));
      const unsigned stop = (starts | ~valid) & above;
      len = (stop ? __ffs(stop) - 1 : kRunRows) - tid;
    }
    sblk[tid] = blk;
    soff[tid] = off;
    srun[tid] = len;
  }
  __syncthreads();

  // K: lane = row, warp and pass = 8-wide d chunk; a run's rows are neighbouring 16-byte pieces of the block
  {
    const int r = tid & 31;
    const long long blk = sblk[r];
    if (blk >= 0) {
      T* kblk = static_cast<T*>(p.kc) + blk * (128 * BS) + soff[r] * 8;
#pragma unroll
      for (int it = 0; it < 4; ++it) {
        const int c = it * 4 + (tid >> 5);
        *reinterpret_cast<uint4*>(kblk + c * (BS * 8)) = *reinterpret_cast<const uint4*>(sk + r * kRunStride + c * 8);
      }
    }
  }
  // V: thread = d; run by run (the same runs for every thread)
  {
    const unsigned short* col = reinterpret_cast<const unsigned short*>(sv) + tid;
    for (int r = 0; r < rows;) {
      const int len = srun[r];
      if (len == 0) {  // skipped row
        ++r;
        continue;
      }
      unsigned short* dst = reinterpret_cast<unsigned short*>(p.vc) + sblk[r] * (128 * BS) + tid * BS + soff[r];
      const unsigned short* src = col + r * kRunStride;
      if (((soff[r] | len) & 7) == 0) {
        for (int i = 0; i < len; i += 8) {
          uint4 w;
          w.x = (unsigned)src[(i + 0) * kRunStride] | ((unsigned)src[(i + 1) * kRunStride] << 16);
          w.y = (unsigned)src[(i + 2) * kRunStride] | ((unsigned)src[(i + 3) * kRunStride] << 16);
          w.z = (unsigned)src[(i + 4) * kRunStride] | ((unsigned)src[(i + 5) * kRunStride] << 16);
          w.w = (unsigned)src[(i + 6) * kRunStride] | ((unsigned)src[(i + 7) * kRunStride] << 16);
          *reinterpret_cast<uint4*>(dst + i) = w;
        }
      } else {
        for (int i = 0; i < len; ++i) dst[i] = src[i * kRunStride];
      }
      r += len;
    }
  }
}

template <typename T>
static int launch_cw(const CacheWriteParams& p, int block_size, cudaStream_t stream) {
  const long long rows = (long long)p.num_tokens * p.num_heads;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((rows + kCwWarps - 1) / kCwWarps));
  cfg.blockDim = dim3(kCwWarps * 32);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  // Same shared-memory carve-out as the attention kernel that follows, so that the SMs are
  // not reconfigured between the two launches.
  static bool carve = false;
  if (!carve) {
    cudaFuncSetAttribute(cache_write_kernel<T, 8>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(cache_write_kernel<T, 16>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    cudaFuncSetAttribute(cache_write_kernel<T, 32>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    carve = true;
  }
  if (p.num_tokens >= kRunMinTokens) {
    cfg.gridDim = dim3((unsigned)((p.num_tokens + kRunRows - 1) / kRunRows), (unsigned)p.num_heads);
    cfg.blockDim = dim3(kRunThreads);
    if (block_size == 8)
      e = cudaLaunchKernelEx(&cfg, cache_write_runs_kernel<T, 8>, p);
    else if (block_size == 16)
      e = cudaLaunchKernelEx(&cfg, cache_write_runs_kernel<T, 16>, p);
    else
      e = cudaLaunchKernelEx(&cfg, cache_write_runs_kernel<T, 32>, p);
    return e == cudaSuccess ? MUX_OK : record_cuda_error(e);
  }
  if (block_size == 8)
    e = cudaLaunchKernelEx(&cfg, cache_write_kernel<T, 8>, p);
  else if (block_size == 16)
    e = cudaLaunchKernelEx(&cfg, cache_write_kernel<T, 16>, p);
  else
    e = cudaLaunchKernelEx(&cfg, cache_write_kernel<T, 32>, p);
  return e == cudaSuccess ? MUX_OK : record_cuda_error(e);
}

}  // namespace mux

extern "C" int mux_reshape_and_cache(const mux_cache_write_args_t* a, void* cuda_stream) {
  if (a == nullptr) return MUX_ERR_NULL_POINTER;
  if (a->dtype != MUX_DTYPE_F16 && a->dtype != MUX_DTYPE_BF16) return MUX_ERR_BAD_DTYPE;
  if (a->head_size != 128) return MUX_ERR_BAD_HEAD_SIZE;
  if (a->block_size != 8 && a->block_size != 16 && a->block_size != 32) return MUX_ERR_BAD_BLOCK_SIZE;
  if (a->num_tokens < 0 || a->num_kv_heads <= 0 || a->num_blocks <= 0) return MUX_ERR_BAD_SHAPE;
  if (a->num_tokens == 0) return MUX_OK;
  if (!a->k || !a->v || !a->key_cache || !a->value_cache || !a->slot_mapping)
    return MUX_ERR_NULL_POINTER;
  if (!mux::aligned16(a->k) || !mux::aligned16(a->v) || !mux::aligned16(a->key_cache) ||
      !mux::aligned16(a->value_cache))
    return MUX_ERR_MISALIGNED;
  // rows are read as 16-byte pieces: every row must start on a 16-byte boundary
  if ((a->k_token_stride & 7) || (a->k_head_stride & 7) || (a->v_token_stride & 7) ||
      (a->v_head_stride & 7))
    return MUX_ERR_MISALIGNED;
  if ((long long)a->num_tokens * a->num_kv_heads > 0x7fffffffLL * mux::kCwWarps || a->num_kv_heads > 65535)
    return MUX_ERR_BAD_SHAPE;
  unsigned* status = mux::device_status_ptr();
  if (status == nullptr) return MUX_ERR_CUDA;
  mux::CacheWriteParams p;
  p.k = a->k;
  p.v = a->v;
  p.kc = a->key_cache;
  p.vc = a->value_cache;
  p.slots = reinterpret_cast<const long long*>(a->slot_mapping);
  p.k_ts = a->k_token_stride;
  p.k_hs = a->k_head_stride;
  p.v_ts = a->v_token_stride;
  p.v_hs = a->v_head_stride;
  p.s_ts = a->slot_token_stride;
  p.s_hs = a->slot_head_stride;
  p.num_blocks = a->num_blocks;
  p.status = status;
  p.num_tokens = a->num_tokens;
  p.num_heads = a->num_kv_heads;
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  return a->dtype == MUX_DTYPE_F16 ? mux::launch_cw<__half>(p, a->block_size, s)
                                   : mux::launch_cw<__nv_bfloat16>(p, a->block_size, s);
}
