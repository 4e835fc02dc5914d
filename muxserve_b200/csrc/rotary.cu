// Stand-alone rotary position embedding of q and k rows, in place (GPT-NeoX pairing, rotary
// dimension = head size = 128).  One warp per (token, head) row.  The fused decode step applies the
// same arithmetic inside the attention kernel; this kernel serves the two-op path and prefill.
#include "internal.h"
#include "rope.cuh"

namespace mux {

struct RotaryParams {
  void* q;
  void* k;
  const long long* positions;
  const void* cache;
  long long q_ts, q_hs, k_ts, k_hs, max_position;
  unsigned* status;
  int num_tokens, num_q_heads, num_kv_heads;
};

constexpr int kRotWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kRotWarps * 32) rotary_kernel(const __grid_constant__ RotaryParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = p.num_q_heads + p.num_kv_heads;
  const long long row = (long long)blockIdx.x * kRotWarps + warp;
  griddep_wait();
  griddep_launch_dependents();
  if (row >= (long long)p.num_tokens * heads) return;
  const int t = (int)(row / heads);
  const int h = (int)(row - (long long)t * heads);
  long long pos = p.positions[t];
  if (pos < 0 || pos >= p.max_position) {
    if (lane == 0) atomicOr(p.status, MUX_DEV_BAD_CONTEXT);
    pos = pos < 0 ? 0 : p.max_position - 1;
  }
  T* x = h < p.num_q_heads ? static_cast<T*>(p.q) + t * p.q_ts + h * p.q_hs
                           : static_cast<T*>(p.k) + t * p.k_ts + (h - p.num_q_heads) * p.k_hs;
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (lane < 16) v = *reinterpret_cast<const uint4*>(x + 8 * lane);
  v = rope_row16<T>(v, lane, static_cast<const T*>(p.cache) + pos * 128);
  if (lane < 16) *reinterpret_cast<uint4*>(x + 8 * lane) = v;
}

}  // namespace mux

extern "C" int mux_rotary_embedding(const mux_rotary_args_t* a, void* cuda_stream) {
  if (a == nullptr) return MUX_ERR_NULL_POINTER;
  if (a->dtype != MUX_DTYPE_F16 && a->dtype != MUX_DTYPE_BF16) return MUX_ERR_BAD_DTYPE;
  if (a->head_size != 128) return MUX_ERR_BAD_HEAD_SIZE;
  if (a->num_tokens < 0 || a->num_q_heads < 0 || a->num_kv_heads < 0 || a->max_position <= 0)
    return MUX_ERR_BAD_SHAPE;
  if (a->num_tokens == 0 || a->num_q_heads + a->num_kv_heads == 0) return MUX_OK;
  if (!a->positions || !a->cos_sin_cache || (a->num_q_heads > 0 && !a->q) || (a->num_kv_heads > 0 && !a->k))
    return MUX_ERR_NULL_POINTER;
  if (!mux::aligned16(a->q) || !mux::aligned16(a->k) || !mux::aligned16(a->cos_sin_cache))
    return MUX_ERR_MISALIGNED;
  if ((a->q_token_stride & 7) || (a->q_head_stride & 7) || (a->k_token_stride & 7) || (a->k_head_stride & 7))
    return MUX_ERR_MISALIGNED;
  unsigned* status = mux::device_status_ptr();
  if (status == nullptr) return MUX_ERR_CUDA;
  mux::RotaryParams p;
  p.q = a->q;
  p.k = a->k;
  p.positions = reinterpret_cast<const long long*>(a->positions);
  p.cache = a->cos_sin_cache;
  p.q_ts = a->q_token_stride;
  p.q_hs = a->q_head_stride;
  p.k_ts = a->k_token_stride;
  p.k_hs = a->k_head_stride;
  p.max_position = a->max_position;
  p.status = status;
  p.num_tokens = a->num_tokens;
  p.num_q_heads = a->num_q_heads;
  p.num_kv_heads = a->num_kv_heads;
  const long long rows = (long long)a->num_tokens * (a->num_q_heads + a->num_kv_heads);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((rows + mux::kRotWarps - 1) / mux::kRotWarps));
  cfg.blockDim = dim3(mux::kRotWarps * 32);
  cfg.stream = static_cast<cudaStream_t>(cuda_stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = a->dtype == MUX_DTYPE_F16 ? cudaLaunchKernelEx(&cfg, mux::rotary_kernel<__half>, p)
                                            : cudaLaunchKernelEx(&cfg, mux::rotary_kernel<__nv_bfloat16>, p);
  return e == cudaSuccess ? MUX_OK : mux::record_cuda_error(e);
}
