// Device status word, error strings and CUDA error bookkeeping.
#include <mutex>

#include "internal.h"
#include "ptx.cuh"

namespace {

__device__ unsigned int g_mux_device_status = 0;

constexpr int kMaxDevices = 64;
unsigned* g_status_ptr[kMaxDevices] = {};
std::mutex g_status_mutex;
thread_local int g_last_cuda_error = 0;

// One warp waits, with the library's bounded wait, on a barrier that nothing will ever complete.
__global__ void wait_selftest_kernel(unsigned* status) {
  __shared__ __align__(8) unsigned long long bar;
  const uint32_t b = mux::smem_u32(&bar);
  if (threadIdx.x == 0) {
    mux::mbar_init(b, 1);
    mux::mbar_init_fence();
  }
  __syncwarp();
  mux::mbar_wait(b, 0, status, MUX_DEV_WAIT_TIMEOUT, 1u << 16);  // same wait, a 16th of the poll limit
}

}  // namespace

namespace mux {

int record_cuda_error(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return MUX_ERR_CUDA;
}

unsigned* device_status_ptr() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    record_cuda_error(e == cudaSuccess ? cudaErrorInvalidDevice : e);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (g_status_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_mux_device_status);
    if (e != cudaSuccess) {
      record_cuda_error(e);
      return nullptr;
    }
    g_status_ptr[dev] = static_cast<unsigned*>(p);
  }
  return g_status_ptr[dev];
}

}  // namespace mux

extern "C" {

const char* mux_strerror(int status) {
  switch (status) {
    case MUX_OK: return "ok";
    case MUX_ERR_NULL_POINTER: return "a required pointer is NULL";
    case MUX_ERR_BAD_DTYPE: return "dtype must be MUX_DTYPE_F16 or MUX_DTYPE_BF16";
    case MUX_ERR_BAD_HEAD_SIZE: return "head_size must be 128";
    case MUX_ERR_BAD_BLOCK_SIZE: return "block_size must be 8, 16 or 32";
    case MUX_ERR_MISALIGNED: return "pointer or stride is not 16-byte aligned";
    case MUX_ERR_BAD_SHAPE: return "negative or inconsistent size";
    case MUX_ERR_BAD_GROUP: return "query heads per kv head must be a positive integer (at most 8 in the mixed form)";
    case MUX_ERR_WORKSPACE_TOO_SMALL: return "workspace is NULL or smaller than mux_*_workspace_size";
    case MUX_ERR_CUDA: return "a CUDA runtime call failed (see mux_last_cuda_error)";
    case MUX_ERR_BAD_HANDLE: return "handle is NULL";
    case MUX_ERR_BUFFER_TOO_SMALL: return "output buffer too small";
    case MUX_ERR_UNKNOWN_REQUEST: return "request id is not known to the scheduler";
    case MUX_ERR_TOO_LARGE: return "size exceeds a fixed capacity of this entry point";
    default: return "unknown status";
  }
}

int mux_last_cuda_error(void) { return g_last_cuda_error; }

int mux_abi_version(void) { return 16; }

int mux_selftest_wait_timeout(void* cuda_stream) {
  unsigned* p = mux::device_status_ptr();
  if (p == nullptr) return MUX_ERR_CUDA;
  wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? MUX_OK : mux::record_cuda_error(e);
}

int mux_device_status(void* cuda_stream) {
  unsigned* p = mux::device_status_ptr();
  if (p == nullptr) return MUX_ERR_CUDA;
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  unsigned host = 0;
  cudaError_t e = cudaMemcpyAsync(&host, p, sizeof(host), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaMemsetAsync(p, 0, sizeof(host), s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return mux::record_cuda_error(e);
  return static_cast<int>(host);
}

}  // extern "C"
