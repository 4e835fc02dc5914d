"""Tensor-parallel all-reduce of the attention path's output over NVLink peer memory.

The reference sums the row-parallel ``o_proj`` output over the TP group with NCCL
(muxserve/flexserver/models/llama.py:131-137,162).  ``TPAllReduce`` sets up the exchange buffers
that ``mux_tp_allreduce`` needs — one per rank, exported to the other ranks through CUDA IPC (as FlexStore
exports its pool to the model workers, muxserve/flexstore/manager.py:893-911) — and calls the kernel.  ``torch.distributed`` is only the plumbing that carries the IPC handles; the data path is the
library's own kernel.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist

from . import _lib
from ._lib import check, lib

_DTYPES = {torch.float16: _lib.MUX_DTYPE_F16, torch.bfloat16: _lib.MUX_DTYPE_BF16}


def buffer_size(world: int, max_message_bytes: int) -> int:
    n = lib().mux_tp_allreduce_buffer_size(world, max_message_bytes)
    if n == 0:
        raise ValueError(f"world size {world} is outside 2..8")
    return n


class TPAllReduce:
    """One communicator per TP group and device.  All ranks must call ``all_reduce`` with the same shapes, in the
    same order, on one stream each."""

    def __init__(self, max_message_bytes: int, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised (it carries the IPC handles)")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device)
        self.max_message_bytes = int(max_message_bytes)
        nbytes = buffer_size(self.world, self.max_message_bytes)
        L = lib()
        self._local = C.c_void_p()
        self._imported = []
        with torch.cuda.device(self.device):
            check(L.mux_tp_buffer_create(nbytes, C.byref(self._local)), "tp_buffer_create")
            handle = C.create_string_buffer(64)
            check(L.mux_tp_buffer_export(self._local, handle), "tp_buffer_export")
            handles: List[bytes] = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            ptrs = []
            for r, raw in enumerate(handles):
                if r == self.rank:
                    ptrs.append(self._local.value)
                    continue
                p = C.c_void_p()
                check(L.mux_tp_buffer_import(raw, C.byref(p)), "tp_buffer_import")
                self._imported.append(p)
                ptrs.append(p.value)
        self.slot_bytes = (nbytes - 8192) // 2      # what one message's exchange area may take (one-shot: world x message)
        self.comm = _lib.TpComm(world=self.world, rank=self.rank, buffer_bytes=nbytes)
        for r, p in enumerate(ptrs):
            self.comm.buffers[r] = p
        dist.barrier(group=group)      # every buffer is zeroed and mapped before anybody's first call

    def close(self) -> None:
        """Unmaps the peers' buffers and frees the local one (after every rank's last call: synchronise first)."""
        L = lib()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for p in self._imported:
                L.mux_tp_buffer_release(p)
            self._imported = []
            if dist.is_initialized():
                dist.barrier(group=self.group)      # nobody still maps this rank's buffer
            if self._local:
                L.mux_tp_buffer_destroy(self._local)
                self._local = C.c_void_p()

    def all_reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None, algo: int = _lib.MUX_TP_AUTO,
                   num_ctas: int = 0) -> torch.Tensor:
        """Sum of ``x`` over the ranks into ``out`` (default: in place), on the current stream."""
        out = x if out is None else out
        if x.dtype not in _DTYPES or out.dtype != x.dtype:
            raise TypeError("all_reduce takes float16 or bfloat16 tensors of one dtype")
        if not x.is_contiguous() or not out.is_contiguous() or out.numel() != x.numel():
            raise ValueError("x and out must be contiguous tensors of one size")
        if x.device != self.device or out.device != self.device:
            raise RuntimeError(f"tensors must live on {self.device}")
        check(lib().mux_tp_allreduce(C.byref(self.comm), x.data_ptr(), out.data_ptr(), x.numel(), _DTYPES[x.dtype],
                                     algo, num_ctas, torch.cuda.current_stream().cuda_stream), "tp_allreduce")
        return out


def all_reduce_emulated(inputs: List[torch.Tensor], max_message_bytes: Optional[int] = None,
                        algo: int = _lib.MUX_TP_AUTO, num_ctas: int = 0, buffers: Optional[List[torch.Tensor]] = None):
    """The kernel's protocol for ``len(inputs)`` ranks on ONE GPU (one cooperative launch): returns
    (outputs per rank, exchange buffers).  Pass the returned buffers back in to continue a sequence of calls."""
    world = len(inputs)
    dev = inputs[0].device
    nbytes = buffer_size(world, max_message_bytes or inputs[0].numel() * inputs[0].element_size())
    if buffers is None:
        buffers = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    outs = [torch.empty_like(x) for x in inputs]
    arr = lambda ts: (C.c_void_p * world)(*[t.data_ptr() for t in ts])
    check(lib().mux_tp_allreduce_emulated(world, arr(buffers), buffers[0].numel(), arr(inputs), arr(outs),
                                          inputs[0].numel(), _DTYPES[inputs[0].dtype], algo, num_ctas,
                                          torch.cuda.current_stream().cuda_stream), "tp_allreduce_emulated")
    return outs, buffers
