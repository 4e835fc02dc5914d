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
        self.slot_bytes = (nbytes - 32768) // 2     # what one message's exchange area may take (one-shot: world x message)
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


def _oproj_args(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, algo: int = _lib.MUX_TP_AUTO,
                early_w: bool = False) -> "_lib.OprojArgs":
    if a.dim() != 2 or w.dim() != 2 or out.dim() != 2:
        raise ValueError("a [m, k], w [n, k] and out [m, n] must be 2-D")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or tuple(out.shape) != (m, n):
        raise ValueError(f"shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if a.dtype not in _DTYPES or w.dtype != a.dtype or out.dtype != a.dtype:
        raise TypeError("a, w and out must be float16 or bfloat16 tensors of one dtype")
    for name, t in (("a", a), ("w", w), ("out", out)):
        if not t.is_cuda or t.stride(1) != 1:
            raise ValueError(f"{name} must be a CUDA tensor with a dense last dimension")
    return _lib.OprojArgs(a=a.data_ptr(), a_row_stride=a.stride(0), w=w.data_ptr(), w_row_stride=w.stride(0),
                          out=out.data_ptr(), out_row_stride=out.stride(0), m=m, n=n, k=k, dtype=_DTYPES[a.dtype],
                          algo=algo, flags=_lib.MUX_OPROJ_EARLY_W if early_w else 0)


def oproj(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, early_w: bool = False) -> torch.Tensor:
    """``out = a @ w.T`` on the tcgen05 GEMM of the fused kernel, without any exchange (one rank).  ``early_w``:
    ``w`` is not written by the kernels directly ahead in the stream, so its first tiles may stream while they drain."""
    args = _oproj_args(a, w, out, early_w=early_w)
    check(lib().mux_tp_oproj_allreduce(None, C.byref(args), torch.cuda.current_stream().cuda_stream), "tp_oproj")
    return out


class TPOProj(TPAllReduce):
    """The row-parallel output projection of a TP rank fused with the all-reduce of its result
    (muxserve/flexserver/models/llama.py:131-137,162).  One instance per hidden size: its communicator is used for
    nothing else, and every rank calls ``forward`` in the same order."""

    def __init__(self, max_tokens: int, hidden: int, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        super().__init__(max_tokens * hidden * 2, device, group)
        self.hidden = hidden

    def forward(self, a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, algo: int = _lib.MUX_TP_AUTO,
                early_w: bool = False) -> torch.Tensor:
        """``out[t, n] = sum over ranks of round(a_rank[t, :] @ w_rank[n, :])``; ``a`` [tokens, local q heads * 128],
        ``w`` [hidden, local q heads * 128] (this rank's columns of the o_proj weight), ``out`` [tokens, hidden]."""
        if w.shape[0] != self.hidden:
            raise ValueError(f"this communicator was made for hidden size {self.hidden}")
        args = _oproj_args(a, w, out, algo, early_w)
        check(lib().mux_tp_oproj_allreduce(C.byref(self.comm), C.byref(args), torch.cuda.current_stream().cuda_stream),
              "tp_oproj_allreduce")
        return out


def oproj_allreduce_emulated(a_list: List[torch.Tensor], w_list: List[torch.Tensor], buffers=None,
                             algo: int = _lib.MUX_TP_AUTO):
    """The fused kernel for ``len(a_list)`` ranks on ONE GPU (one cooperative launch); returns (outs, buffers)."""
    world = len(a_list)
    m, n = a_list[0].shape[0], w_list[0].shape[0]
    dev = a_list[0].device
    nbytes = buffer_size(world, m * n * 2)
    if buffers is None:
        buffers = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    outs = [torch.empty((m, n), dtype=a_list[0].dtype, device=dev) for _ in range(world)]
    args = (_lib.OprojArgs * world)(*[_oproj_args(a, w, o, algo) for a, w, o in zip(a_list, w_list, outs)])
    bufs = (C.c_void_p * world)(*[b.data_ptr() for b in buffers])
    scratch = torch.empty(2 * world * 128, dtype=torch.uint8, device=dev)
    check(lib().mux_tp_oproj_allreduce_emulated(world, bufs, nbytes, args, scratch.data_ptr(),
                                                torch.cuda.current_stream().cuda_stream), "tp_oproj_allreduce_emulated")
    torch.cuda.synchronize()          # `scratch` holds the launch's copy descriptors
    return outs, buffers
