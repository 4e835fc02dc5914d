// Incremental maintenance of a block table that lives on the device: newly granted blocks are
// scattered into it instead of re-uploading the whole table every step.
#include "internal.h"
#include "ptx.cuh"

namespace mux {

struct AppendParams {
  int* tables;
  long long ls, rs, hs;
  const int* upd_row;
  const int* upd_block;
  const int* upd_ids;
  unsigned* status;
  int L, R, H, max_blocks, n;
};

__global__ void __launch_bounds__(256) block_table_append_kernel(const __grid_constant__ AppendParams p) {
  griddep_wait();
  griddep_launch_dependents();
  const int i = blockIdx.x;
  const int row = p.upd_row[i], blk = p.upd_block[i];
  if (row < 0 || row >= p.R || blk < 0 || blk >= p.max_blocks) {  // reported, never written
    if (threadIdx.x == 0) atomicOr(p.status, MUX_DEV_BAD_SLOT);
    return;
  }
  const int LH = p.L * p.H;
  for (int j = threadIdx.x; j < LH; j += blockDim.x) {
    const int l = j / p.H, h = j - l * p.H;
    p.tables[l * p.ls + row * p.rs + h * p.hs + blk] = p.upd_ids[(long long)i * LH + j];
  }
}

}  // namespace mux

extern "C" int mux_block_table_append(int32_t* tables, int64_t layer_stride, int64_t row_stride, int64_t head_stride,
                                      int32_t num_layers, int32_t num_rows, int32_t num_kv_heads, int32_t max_blocks,
                                      const int32_t* upd_row, const int32_t* upd_block, const int32_t* upd_ids,
                                      int32_t num_updates, void* cuda_stream) {
  if (num_updates < 0 || num_layers <= 0 || num_rows <= 0 || num_kv_heads <= 0 || max_blocks <= 0 ||
      layer_stride < 0 || row_stride < 0 || head_stride < 0)
    return MUX_ERR_BAD_SHAPE;
  if (num_updates == 0) return MUX_OK;
  if (!tables || !upd_row || !upd_block || !upd_ids) return MUX_ERR_NULL_POINTER;
  unsigned* status = mux::device_status_ptr();
  if (status == nullptr) return MUX_ERR_CUDA;
  mux::AppendParams p;
  p.tables = tables;
  p.ls = layer_stride;
  p.rs = row_stride;
  p.hs = head_stride;
  p.upd_row = upd_row;
  p.upd_block = upd_block;
  p.upd_ids = upd_ids;
  p.status = status;
  p.L = num_layers;
  p.R = num_rows;
  p.H = num_kv_heads;
  p.max_blocks = max_blocks;
  p.n = num_updates;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)num_updates);
  cfg.blockDim = dim3(256);
  cfg.stream = static_cast<cudaStream_t>(cuda_stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, mux::block_table_append_kernel, p);
  return e == cudaSuccess ? MUX_OK : mux::record_cuda_error(e);
}
