"""Geometry of the FlexStore unified KV pool.

Restates the shape arithmetic of ``FlexStoreManager``
(muxserve/flexstore/manager.py:444-498): one key tensor and one value tensor per
GPU with no layer and no head dimension; a block is ``block_size`` tokens of one
head of one layer of one model.
"""
from __future__ import annotations

from typing import Tuple

import torch

HEAD_SIZE = 128  # muxserve/flexstore/manager.py:336-337


def get_key_block_shape(block_size: int, element_size: int = 2, head_size: int = HEAD_SIZE) -> Tuple[int, int, int]:
    x = 16 // element_size
    return (head_size // x, block_size, x)


def get_value_block_shape(block_size: int, head_size: int = HEAD_SIZE) -> Tuple[int, int]:
    return (head_size, block_size)


def block_bytes(block_size: int, element_size: int = 2, head_size: int = HEAD_SIZE) -> int:
    """Bytes of one block's key part plus value part."""
    return 2 * head_size * block_size * element_size


def get_num_gpu_blocks(total_gpu_memory: int, gpu_memory_utilization: float, block_size: int,
                       head_size: int = HEAD_SIZE) -> int:
    """manager.py:444-454: usable bytes // block bytes, rounded down to a multiple of 128."""
    available = round(gpu_memory_utilization * total_gpu_memory) - 1
    block_mem = 2 * (head_size * block_size + head_size * block_size)
    return (available // block_mem // 128) * 128


def allocate_gpu_cache(num_blocks: int, block_size: int, dtype: torch.dtype = torch.float16,
                       device="cuda") -> Tuple[torch.Tensor, torch.Tensor]:
    """Uninitialised (key pool, value pool) as manager.py:470-498 allocates them."""
    es = torch.empty((), dtype=dtype).element_size()
    k = torch.empty((num_blocks, *get_key_block_shape(block_size, es)), dtype=dtype, device=device)
    v = torch.empty((num_blocks, *get_value_block_shape(block_size)), dtype=dtype, device=device)
    return k, v


def get_tensor_metadata(tensor: torch.Tensor) -> dict:
    """Everything another process on the same GPU needs to map ``tensor`` through CUDA IPC — the dictionary the
    FlexStore service sends to its model workers for pool and weight tensors
    (muxserve/flexstore/manager.py:893-911, same keys).  The exporting process must keep ``tensor`` alive."""
    if not tensor.is_cuda:
        raise RuntimeError("only CUDA tensors can be exported through CUDA IPC")
    storage = tensor._typed_storage()
    (device, handle, size_bytes, offset_bytes, ref_counter_handle, ref_counter_offset, event_handle,
     event_sync_required) = storage._share_cuda_()
    return {
        "tensor_size": tensor.size(),
        "tensor_stride": tensor.stride(),
        "tensor_offset": tensor.storage_offset(),
        "storage_cls": type(storage),
        "dtype": tensor.dtype,
        "storage_device": device,
        "storage_handle": handle,
        "storage_size_bytes": size_bytes,
        "storage_offset_bytes": offset_bytes,
        "requires_grad": tensor.requires_grad,
        "ref_counter_handle": ref_counter_handle,
        "ref_counter_offset": ref_counter_offset,
        "event_handle": event_handle,
        "event_sync_required": event_sync_required,
    }


def rebuild_tensor(metadata: dict) -> torch.Tensor:
    """The importing side: a tensor over the exporter's memory (what the worker does with each received dictionary,
    muxserve/flexserver/model_loader.py:44-49)."""
    from torch.multiprocessing.reductions import rebuild_cuda_tensor
    return rebuild_cuda_tensor(torch.Tensor, **metadata)
