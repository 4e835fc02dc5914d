// Inline-PTX building blocks for the sm_100a kernels: mbarrier pipeline,
// 1-D bulk (TMA) global->shared copies, ldmatrix and the m16n8k16 MMA.
// No cluster multicast is used anywhere in this library.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace mux {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// Makes freshly initialised barriers visible to the async (TMA) proxy.
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Orders this thread's earlier generic-proxy accesses to shared memory before later
// async-proxy (bulk copy) accesses to it.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Orders this thread's earlier generic-proxy writes to global memory before later async-proxy (bulk copy)
// reads of it.
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking test of a phase: for a thread that usually finds the phase complete (an MMA issuer behind a deep
// ring) and cannot afford the wake-up latency of a suspended wait on every pass of its loop.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  When the limit runs out the caller's status word gets
// `timeout_bit` and the wait returns as if it had succeeded, so that every
// later barrier of the CTA is still reached and the kernel ends; the result of
// that CTA is then garbage and the host learns it from the status word.  Once
// the bit is set (by any CTA) every other wait gives up after kWaitRecheck
// polls, so a protocol error costs one expiry, not one per wait.
constexpr uint32_t kWaitLimit = 1u << 20;
constexpr uint32_t kWaitRecheck = 1u << 10;

__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, unsigned* status,
                                          unsigned timeout_bit, uint32_t limit = kWaitLimit) {
  if (mbar_test_wait(bar, parity)) return;  // usually complete behind a ring: no (potentially suspending) try_wait then
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return;
    if ((i & (kWaitRecheck - 1)) == kWaitRecheck - 1 &&
        (*reinterpret_cast<volatile unsigned*>(status) & timeout_bit))
      return;
  }
  atomicOr(status, timeout_bit);
}

// The same bounded wait for threads that expect to wait long (a producer or an MMA-issuing thread of the
// prompt kernel): each poll carries a suspend-time hint, so the thread sleeps in hardware until the phase
// completes or the hint (in ns) runs out instead of spinning through the issue slots of its scheduler.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

constexpr uint32_t kSleepyHintNs = 2000;
constexpr uint32_t kSleepyLimit = 1u << 18;  // x 2 us: the same order of patience as kWaitLimit spins

__device__ __forceinline__ void mbar_wait_sleepy(uint32_t bar, uint32_t parity, unsigned* status,
                                                 unsigned timeout_bit) {
  // A suspended wait costs a few hundred cycles of wake-up even when the phase is already complete (measured:
  // 250-450 cycles on B200), and an issuing thread behind a deep ring mostly finds it complete: test first.
  if (mbar_test_wait(bar, parity)) return;
  for (uint32_t i = 0; i < kSleepyLimit; ++i) {
    if (mbar_try_wait_hint(bar, parity, kSleepyHintNs)) return;
    if ((i & 15u) == 15u && (*reinterpret_cast<volatile unsigned*>(status) & timeout_bit)) return;
  }
  atomicOr(status, timeout_bit);
}

// 1-D bulk copy global -> shared of `bytes` (multiple of 16, both sides 16-B
// aligned), completion counted on `bar`.  Non-multicast.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}

// Programmatic dependent launch: `wait` blocks until every kernel this launch
// depends on has completed and its writes are visible; `launch_dependents`
// lets the next kernel of the stream start being scheduled.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

__device__ __forceinline__ uint32_t ldg32_nc(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// D = A(16x16, row) * B(16x8, col) + D, fp32 accumulate.
template <typename T>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1);

template <>
__device__ __forceinline__ void mma_16816<__half>(float (&d)[4], const uint32_t (&a)[4],
                                                  uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4],
                                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ T from_float(float x);
template <>
__device__ __forceinline__ __half from_float<__half>(float x) {
  return __float2half_rn(x);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}

__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

// Two fp32 softmax weights -> one packed pair of their 16-bit roundings (hi) and one packed pair
// of the rounding residues (lo); hi + lo carries ~16 mantissa bits.
template <typename T>
__device__ __forceinline__ void split_pair(float a, float b, uint32_t& hi, uint32_t& lo);
template <>
__device__ __forceinline__ void split_pair<__half>(float a, float b, uint32_t& hi, uint32_t& lo) {
  const __half2 h = __floats2half2_rn(a, b);
  const float2 back = __half22float2(h);
  const __half2 l = __floats2half2_rn(a - back.x, b - back.y);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}
template <>
__device__ __forceinline__ void split_pair<__nv_bfloat16>(float a, float b, uint32_t& hi, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  const float2 back = __bfloat1622float2(h);
  const __nv_bfloat162 l = __floats2bfloat162_rn(a - back.x, b - back.y);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace mux
