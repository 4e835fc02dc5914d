// All-reduce (sum) of the tensor-parallel attention output over NVLink peer memory (sm_100a).
//
// The reference sums the row-parallel o_proj output over the TP group with an NCCL
// all-reduce (muxserve/flexserver/models/llama.py:131-137,162).  For the message sizes of
// a decode step ([batch, hidden] in 16-bit: 0.5 - 2 MiB) that collective is latency-bound,
// so this file does it in ONE kernel per rank with plain peer stores and loads:
//
//   one-shot  (small messages): every rank pushes its chunk into slot [rank] of every
//             rank's exchange buffer, raises a flag there, waits for the world's flags
//             in its own buffer and sums the world's chunks from LOCAL memory in rank
//             order (so every rank gets the same bits).
//   two-shot  (large messages): rank r owns slice r.  Every rank publishes its input in
//             its own buffer and raises flags; rank r sums slice r over the world with
//             peer loads, pushes the sum to every rank, raises a second flag; every
//             rank waits for the world's second flags and copies the sums out.
//
// Synchronisation is per CTA index: CTA b of every rank works on chunk b and only ever
// waits for CTA b of the other ranks, so no grid-wide barrier is needed and the CTAs of
// a launch need not be resident together.  Every launch has the same number of CTAs
// (those beyond the ones that move data only exchange flags), so a CTA's own call
// counter — kept in the exchange buffer, no atomics — is the launch's epoch on every
// rank.  Flags carry the epoch, data slots alternate with its parity: a rank can start
// epoch e + 2, the next user of a slot, only after every peer raised its flag of epoch
// e + 1, i.e. after every peer's kernel of epoch e has ended.  Every wait is bounded; when one runs out the kernel sets
// MUX_DEV_WAIT_TIMEOUT and goes on to its end (results are then garbage, nothing hangs).
// No multimem, no TMA, no cluster multicast: plain ld / st on peer pointers.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdint>
#include <cstring>

#include "internal.h"
#include "ptx.cuh"

namespace mux {

constexpr int kArMaxWorld = MUX_TP_MAX_WORLD;
constexpr int kArMaxCtas = 64;
constexpr int kArCtas = 32;  // CTAs of every launch
constexpr int kArThreads = 512;
constexpr unsigned kArWaitLimit = 1u << 23;  // polls of ~0.4 us: a few seconds

struct ArCtrl {
  unsigned epoch[kArMaxCtas];                // per CTA: launches completed on this rank
  unsigned ready[kArMaxWorld][kArMaxCtas];   // [source rank][cta]: source's chunk is published (epoch value)
  unsigned done[kArMaxWorld][kArMaxCtas];    // two-shot: source's reduced slice has been pushed
};
constexpr size_t kArCtrlBytes = MUX_TP_CTRL_BYTES;  // this op's block is the first 8 KiB; the fused o_proj's follows
static_assert(sizeof(ArCtrl) <= 8192, "control block");

struct ArParams {
  unsigned char* buf[kArMaxWorld];   // exchange buffers of all ranks as mapped in this process
  const void* in[kArMaxWorld];       // real launch: only [rank] is used; emulated launch: one per rank
  void* out[kArMaxWorld];
  long long slot_bytes;              // bytes of one data slot (two per buffer)
  long long nvec;                    // 16-byte vectors per message
  unsigned* status;
  int world, rank, algo, ncta;
};

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

// Threads 0..world-1 each wait for one source's flag to reach `epoch`.
__device__ __forceinline__ void wait_flags(const unsigned* flags_of_source0, int world, unsigned epoch,
                                           unsigned* status) {
  if ((int)threadIdx.x < world) {
    const unsigned* f = flags_of_source0 + (size_t)threadIdx.x * kArMaxCtas;
    unsigned i = 0;
    while ((int)(ld_flag(f) - epoch) < 0) {
      if (++i >= kArWaitLimit || ((i & 1023u) == 0 && (*reinterpret_cast<volatile unsigned*>(status) & MUX_DEV_WAIT_TIMEOUT))) {
        atomicOr(status, MUX_DEV_WAIT_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
}

template <typename T>
__device__ __forceinline__ void accumulate(float (&acc)[8], const uint4& v);
template <>
__device__ __forceinline__ void accumulate<__half>(float (&acc)[8], const uint4& v) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}
template <>
__device__ __forceinline__ void accumulate<__nv_bfloat16>(float (&acc)[8], const uint4& v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&acc)[8]);
template <>
__device__ __forceinline__ uint4 pack8<__half>(const float (&acc)[8]) {
  uint4 v;
  __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
  return v;
}
template <>
__device__ __forceinline__ uint4 pack8<__nv_bfloat16>(const float (&acc)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  return v;
}

// The whole all-reduce as seen by CTA `cta` (of `p.ncta`) of rank `rank`.
template <typename T>
__device__ void allreduce_body(const ArParams& p, int rank, int cta) {
  const int tid = threadIdx.x, world = p.world;
  ArCtrl* my = reinterpret_cast<ArCtrl*>(p.buf[rank]);
  // launched with programmatic dependent launch: the CTA may be resident before the kernel ahead has ended,
  // and that kernel may be this rank's previous all-reduce (which stores the counter read next) or the producer of `in`
  griddep_wait();
  griddep_launch_dependents();
  const unsigned epoch = *reinterpret_cast<volatile unsigned*>(&my->epoch[cta]) + 1u;
  const size_t slot_off = kArCtrlBytes + (size_t)(epoch & 1u) * (size_t)p.slot_bytes;
  const size_t msg_bytes = (size_t)p.nvec * 16;
  const uint4* in = static_cast<const uint4*>(p.in[rank]);
  uint4* out = static_cast<uint4*>(p.out[rank]);

  if (p.algo == 1) {
    // ---- one-shot: push my chunk to everybody, sum everybody's chunk locally ----
    const long long per = (p.nvec + p.ncta - 1) / p.ncta;
    const long long v0 = (long long)cta * per, v1 = min(p.nvec, v0 + per);
    for (long long v = v0 + tid; v < v1; v += kArThreads) {
      const uint4 x = in[v];
      for (int q = 0; q < world; ++q)
        *reinterpret_cast<uint4*>(p.buf[q] + slot_off + (size_t)rank * msg_bytes + (size_t)v * 16) = x;
    }
    __syncthreads();  // the releasing flag stores below are cumulative: they order every thread's pushes before the flag
    if (tid < world) st_flag(&reinterpret_cast<ArCtrl*>(p.buf[tid])->ready[rank][cta], epoch);
    wait_flags(&my->ready[0][cta], world, epoch, p.status);
    const unsigned char* mine = p.buf[rank] + slot_off;
    for (long long v = v0 + tid; v < v1; v += kArThreads) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int q = 0; q < world; ++q) accumulate<T>(acc, ld_vol(mine + (size_t)q * msg_bytes + (size_t)v * 16));
      out[v] = pack8<T>(acc);
    }
  } else {
    // ---- two-shot: publish, reduce my slice over peer loads, push the sums, collect ----
    const long long sv = (p.nvec + world - 1) / world;       // vectors per slice
    const long long per = (sv + p.ncta - 1) / p.ncta;         // vectors per (slice, cta)
    const size_t a_off = slot_off, b_off = slot_off + ((msg_bytes + 255) & ~(size_t)255);
    for (int s = 0; s < world; ++s) {
      const long long lo = s * sv + (long long)cta * per, hi = min(min(p.nvec, (s + 1) * sv), lo + per);
      for (long long v = lo + tid; v < hi; v += kArThreads)
        *reinterpret_cast<uint4*>(p.buf[rank] + a_off + (size_t)v * 16) = in[v];
    }
    __syncthreads();  // the releasing flag stores below are cumulative: they order every thread's pushes before the flag
    if (tid < world) st_flag(&reinterpret_cast<ArCtrl*>(p.buf[tid])->ready[rank][cta], epoch);
    wait_flags(&my->ready[0][cta], world, epoch, p.status);
    {
      const long long lo = rank * sv + (long long)cta * per, hi = min(min(p.nvec, (rank + 1) * sv), lo + per);
      for (long long v = lo + tid; v < hi; v += kArThreads) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint4 x[kArMaxWorld];
#pragma unroll
        for (int q = 0; q < kArMaxWorld; ++q)
          if (q < world) x[q] = ld_vol(p.buf[q] + a_off + (size_t)v * 16);
#pragma unroll
        for (int q = 0; q < kArMaxWorld; ++q)
          if (q < world) accumulate<T>(acc, x[q]);
        const uint4 r = pack8<T>(acc);
        for (int q = 0; q < world; ++q) *reinterpret_cast<uint4*>(p.buf[q] + b_off + (size_t)v * 16) = r;
      }
    }
    __syncthreads();  // the releasing flag stores below are cumulative: they order every thread's pushes before the flag
    if (tid < world) st_flag(&reinterpret_cast<ArCtrl*>(p.buf[tid])->done[rank][cta], epoch);
    wait_flags(&my->done[0][cta], world, epoch, p.status);
    for (int s = 0; s < world; ++s) {
      const long long lo = s * sv + (long long)cta * per, hi = min(min(p.nvec, (s + 1) * sv), lo + per);
      for (long long v = lo + tid; v < hi; v += kArThreads) out[v] = ld_vol(p.buf[rank] + b_off + (size_t)v * 16);
    }
  }

  __syncthreads();
  if (tid == 0) my->epoch[cta] = epoch;  // this CTA's next launch (after this kernel has ended) is epoch + 1
}

template <typename T>
__global__ void __launch_bounds__(kArThreads) tp_allreduce_kernel(const __grid_constant__ ArParams p) {
  allreduce_body<T>(p, p.rank, blockIdx.x);
}

// All ranks of a world in ONE grid on one GPU (blockIdx.y = rank): the same device code with every
// "peer" buffer on the local GPU.  Its CTAs wait on one another, so it is launched cooperatively.
template <typename T>
__global__ void __launch_bounds__(kArThreads) tp_allreduce_emulated_kernel(const __grid_constant__ ArParams p) {
  allreduce_body<T>(p, blockIdx.y, blockIdx.x);
}

static int pick_algo(int algo, int world, size_t bytes) {
  if (algo == MUX_TP_ONE_SHOT || algo == MUX_TP_TWO_SHOT) return algo;
  // one-shot sends the whole message to every peer: cheapest in latency while that traffic stays small
  return (size_t)(world - 1) * bytes <= (size_t)MUX_TP_ONE_SHOT_MAX_PUSH_BYTES ? MUX_TP_ONE_SHOT : MUX_TP_TWO_SHOT;
}

// How many of the launch's kArCtas CTAs move data (the others only exchange flags).
static int pick_ctas(int num_ctas, int algo, int world, long long nvec) {
  if (num_ctas > 0) return std::min(num_ctas, kArCtas);
  // enough CTAs to keep the links busy, at least ~4 KiB of the message per CTA
  const long long share = algo == MUX_TP_ONE_SHOT ? nvec : (nvec + world - 1) / world;
  return (int)std::max<long long>(1, std::min<long long>(kArCtas, share / 256));
}

static int fill_params(ArParams& prm, int world, void* const* buffers, long long buffer_bytes, long long count,
                       int dtype, int algo, int num_ctas) {
  if (world < 2 || world > kArMaxWorld || count < 0 || num_ctas < 0) return MUX_ERR_BAD_SHAPE;
  if (dtype != MUX_DTYPE_F16 && dtype != MUX_DTYPE_BF16) return MUX_ERR_BAD_DTYPE;
  if (algo != MUX_TP_AUTO && algo != MUX_TP_ONE_SHOT && algo != MUX_TP_TWO_SHOT) return MUX_ERR_BAD_SHAPE;
  if (count % 8 != 0) return MUX_ERR_MISALIGNED;  // whole 16-byte vectors
  if (buffers == nullptr) return MUX_ERR_NULL_POINTER;
  for (int q = 0; q < world; ++q) {
    if (buffers[q] == nullptr) return MUX_ERR_NULL_POINTER;
    if ((reinterpret_cast<uintptr_t>(buffers[q]) & 255u) != 0) return MUX_ERR_MISALIGNED;
    prm.buf[q] = static_cast<unsigned char*>(buffers[q]);
  }
  const size_t bytes = (size_t)count * 2;
  prm.algo = pick_algo(algo, world, bytes);
  prm.world = world;
  prm.nvec = count / 8;
  prm.slot_bytes = (buffer_bytes - (long long)kArCtrlBytes) / 2 / 256 * 256;
  const size_t padded = (bytes + 255) & ~(size_t)255;
  const size_t need = prm.algo == MUX_TP_ONE_SHOT ? (size_t)world * bytes : 2 * padded;
  if (prm.slot_bytes <= 0 || need > (size_t)prm.slot_bytes) return MUX_ERR_TOO_LARGE;
  prm.ncta = pick_ctas(num_ctas, prm.algo, world, prm.nvec);
  return MUX_OK;
}

}  // namespace mux

extern "C" {

size_t mux_tp_allreduce_buffer_size(int32_t world, size_t max_message_bytes) {
  if (world < 2 || world > mux::kArMaxWorld) return 0;
  const size_t padded = (max_message_bytes + 255) & ~(size_t)255;
  const size_t slot = std::max((size_t)world * padded, 2 * padded);
  return mux::kArCtrlBytes + 2 * slot;
}

int mux_tp_buffer_create(size_t bytes, void** ptr) {
  if (ptr == nullptr || bytes == 0) return MUX_ERR_NULL_POINTER;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);  // its own allocation: an IPC handle names a whole allocation
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (p != nullptr) cudaFree(p);
    return mux::record_cuda_error(e);
  }
  *ptr = p;
  return MUX_OK;
}

int mux_tp_buffer_destroy(void* ptr) {
  if (ptr == nullptr) return MUX_OK;
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? MUX_OK : mux::record_cuda_error(e);
}

int mux_tp_buffer_export(const void* ptr, unsigned char handle[MUX_TP_IPC_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == MUX_TP_IPC_HANDLE_BYTES, "IPC handle size");
  if (ptr == nullptr || handle == nullptr) return MUX_ERR_NULL_POINTER;
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(ptr));
  if (e != cudaSuccess) return mux::record_cuda_error(e);
  memcpy(handle, &h, sizeof(h));
  return MUX_OK;
}

int mux_tp_buffer_import(const unsigned char handle[MUX_TP_IPC_HANDLE_BYTES], void** ptr) {
  if (ptr == nullptr || handle == nullptr) return MUX_ERR_NULL_POINTER;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  // Mapped into the address space of the CURRENT device (the one whose kernels will touch it), with peer
  // access to the exporting GPU switched on as part of the mapping.
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return mux::record_cuda_error(e);
  cudaPointerAttributes attr;
  e = cudaPointerGetAttributes(&attr, p);
  if (e != cudaSuccess || attr.type != cudaMemoryTypeDevice) {
    cudaIpcCloseMemHandle(p);
    return mux::record_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidDevicePointer);
  }
  int dev = 0, can = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return mux::record_cuda_error(e);
  if (attr.device != dev) {  // a peer GPU's memory: this device's kernels must be allowed to reach it
    e = cudaDeviceCanAccessPeer(&can, dev, attr.device);
    if (e != cudaSuccess || !can) {
      cudaIpcCloseMemHandle(p);
      return mux::record_cuda_error(e != cudaSuccess ? e : cudaErrorPeerAccessUnsupported);
    }
    e = cudaDeviceEnablePeerAccess(attr.device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
      (void)cudaGetLastError();
    } else if (e != cudaSuccess) {
      cudaIpcCloseMemHandle(p);
      return mux::record_cuda_error(e);
    }
  }
  *ptr = p;
  return MUX_OK;
}

int mux_tp_buffer_release(void* ptr) {
  if (ptr == nullptr) return MUX_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? MUX_OK : mux::record_cuda_error(e);
}

int mux_tp_allreduce(const mux_tp_comm_t* comm, const void* in, void* out, int64_t count, int32_t dtype,
                     int32_t algo, int32_t num_ctas, void* cuda_stream) {
  if (comm == nullptr) return MUX_ERR_NULL_POINTER;
  if (comm->rank < 0 || comm->rank >= comm->world) return MUX_ERR_BAD_SHAPE;
  mux::ArParams prm = {};
  int st = mux::fill_params(prm, comm->world, comm->buffers, comm->buffer_bytes, count, dtype, algo, num_ctas);
  if (st != MUX_OK) return st;
  if (count == 0) return MUX_OK;
  if (in == nullptr || out == nullptr) return MUX_ERR_NULL_POINTER;
  if (!mux::aligned16(in) || !mux::aligned16(out)) return MUX_ERR_MISALIGNED;
  prm.rank = comm->rank;
  prm.in[comm->rank] = in;
  prm.out[comm->rank] = out;
  prm.status = mux::device_status_ptr();
  if (prm.status == nullptr) return MUX_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(mux::kArCtas);
  cfg.blockDim = dim3(mux::kArThreads);
  cfg.stream = s;
  cfg.attrs = pdl;
  cfg.numAttrs = 1;
  cudaError_t e = dtype == MUX_DTYPE_F16 ? cudaLaunchKernelEx(&cfg, mux::tp_allreduce_kernel<__half>, prm)
                                         : cudaLaunchKernelEx(&cfg, mux::tp_allreduce_kernel<__nv_bfloat16>, prm);
  return e == cudaSuccess ? MUX_OK : mux::record_cuda_error(e);
}

int mux_tp_allreduce_emulated(int32_t world, void* const* buffers, int64_t buffer_bytes, const void* const* ins,
                              void* const* outs, int64_t count, int32_t dtype, int32_t algo, int32_t num_ctas,
                              void* cuda_stream) {
  mux::ArParams prm = {};
  int st = mux::fill_params(prm, world, buffers, buffer_bytes, count, dtype, algo, num_ctas);
  if (st != MUX_OK) return st;
  if (count == 0) return MUX_OK;
  if (ins == nullptr || outs == nullptr) return MUX_ERR_NULL_POINTER;
  for (int q = 0; q < world; ++q) {
    if (ins[q] == nullptr || outs[q] == nullptr) return MUX_ERR_NULL_POINTER;
    if (!mux::aligned16(ins[q]) || !mux::aligned16(outs[q])) return MUX_ERR_MISALIGNED;
    prm.in[q] = ins[q];
    prm.out[q] = outs[q];
  }
  prm.rank = 0;
  prm.status = mux::device_status_ptr();
  if (prm.status == nullptr) return MUX_ERR_CUDA;
  // The ranks' CTAs wait on one another: a cooperative launch makes the runtime check that the whole
  // grid is resident at once (it fails the launch otherwise), which is what the waits need.
  void* kargs[] = {&prm};
  const void* fn = dtype == MUX_DTYPE_F16 ? (const void*)mux::tp_allreduce_emulated_kernel<__half>
                                          : (const void*)mux::tp_allreduce_emulated_kernel<__nv_bfloat16>;
  const dim3 grid((unsigned)mux::kArCtas, (unsigned)world);
  cudaError_t e = cudaLaunchCooperativeKernel(fn, grid, dim3(mux::kArThreads), kargs, 0,
                                              static_cast<cudaStream_t>(cuda_stream));
  return e == cudaSuccess ? MUX_OK : mux::record_cuda_error(e);
}

}  // extern "C"
