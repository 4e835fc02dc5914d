// reshape_and_cache: scatter new tokens' K/V rows into the head-granular pool.
//
// One warp per (token, kv head) row.  The K row (128 elements) lands as 16
// 16-byte pieces, one per 8-wide d chunk, block_size*16 bytes apart; the V row
// lands as 128 single elements block_size*2 bytes apart.
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
  if ((long long)a->num_tokens * a->num_kv_heads > 0x7fffffffLL * mux::kCwWarps) return MUX_ERR_BAD_SHAPE;
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
