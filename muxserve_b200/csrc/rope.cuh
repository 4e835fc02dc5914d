// Rotary position embedding (GPT-NeoX pairing: element d < 64 rotates with element d + 64) on
// packed pairs of 16-bit elements.  Arithmetic in fp32, one rounding to the tensor dtype; the
// stand-alone kernel and the fused decode step share these functions, so their results are
// bit-identical.  Cache row of a position: 64 cosines followed by 64 sines, in the tensor dtype.
#pragma once
#include "ptx.cuh"

namespace mux {

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

// lo = two elements at d, d+1 (d < 64), hi = the elements at d+64, d+65; cs / sn = cos, sin at d, d+1.
//   lo' = lo*cos - hi*sin      hi' = hi*cos + lo*sin
template <typename T>
__device__ __forceinline__ void rope_words(uint32_t& lo, uint32_t& hi, uint32_t cs, uint32_t sn) {
  const float2 x = unpack2<T>(lo), y = unpack2<T>(hi), c = unpack2<T>(cs), s = unpack2<T>(sn);
  lo = pack2<T>(__fsub_rn(__fmul_rn(x.x, c.x), __fmul_rn(y.x, s.x)), __fsub_rn(__fmul_rn(x.y, c.y), __fmul_rn(y.y, s.y)));
  hi = pack2<T>(__fadd_rn(__fmul_rn(y.x, c.x), __fmul_rn(x.x, s.x)), __fadd_rn(__fmul_rn(y.y, c.y), __fmul_rn(x.y, s.y)));
}

// A 128-element row held by 16 lanes as 16-byte pieces (lane l: elements 8l .. 8l+7).  Every lane of
// `mask` must call: the whole warp (lanes >= 16 get their value back unchanged), or one half-warp
// (mask 0x0000ffff / 0xffff0000) with `lane` counted inside the half.
template <typename T>
__device__ __forceinline__ uint4 rope_row16(uint4 mine, int lane, const T* cache_row, unsigned mask = 0xffffffffu) {
  uint4 other;
  other.x = __shfl_xor_sync(mask, mine.x, 8);
  other.y = __shfl_xor_sync(mask, mine.y, 8);
  other.z = __shfl_xor_sync(mask, mine.z, 8);
  other.w = __shfl_xor_sync(mask, mine.w, 8);
  if (lane >= 16) return mine;
  const int d0 = 8 * (lane & 7);
  const uint4 cs = *reinterpret_cast<const uint4*>(cache_row + d0);
  const uint4 sn = *reinterpret_cast<const uint4*>(cache_row + 64 + d0);
  const bool low = lane < 8;  // this lane holds the d < 64 half of the pairs
  uint4 lo = low ? mine : other, hi = low ? other : mine;
  rope_words<T>(lo.x, hi.x, cs.x, sn.x);
  rope_words<T>(lo.y, hi.y, cs.y, sn.y);
  rope_words<T>(lo.z, hi.z, cs.z, sn.z);
  rope_words<T>(lo.w, hi.w, cs.w, sn.w);
  return low ? lo : hi;
}

}  // namespace mux
