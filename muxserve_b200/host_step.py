"""One decode step of the attention path driven from HOST buffers.

The reference uploads a step's index tensors from the CPU every step
(``slot_mapping``, ``block_tables``, ``context_lens``:
muxserve/flexserver/llm_runtime.py:300-327) and synchronises at its end (:274).
``HostDecodeStep.run`` does the same for all inputs of the path: per layer it
uploads q / k / v and that layer's block tables from pinned host memory on a
copy stream, runs ``reshape_and_cache`` + ``paged_attention`` on the caller's
stream and downloads the layer's output on a third stream, so that transfers of
neighbouring layers overlap the kernels.  With one new token per sequence the two ops run
as the fused ``decode_attention`` launch (``slot_mapping`` is still uploaded, as the reference
does, but the kernel derives the slots from the block tables).
"""
from __future__ import annotations

import torch

from . import ops
from .workloads import HEAD_SIZE, ModelShape


class HostDecodeStep:
    def __init__(self, shape: ModelShape, block_size: int, dtype: torch.dtype, key_cache: torch.Tensor,
                 value_cache: torch.Tensor, max_blocks_per_seq: int, new_tokens: int = 1, depth: int = 4,
                 partition_size: int = 0, num_stages: int = 0, fused: bool = True, units_capacity: int = 0):
        dev = key_cache.device
        self.shape, self.block_size, self.dtype = shape, block_size, dtype
        self.kc, self.vc = key_cache, value_cache
        self.depth = depth
        self.partition_size, self.num_stages = partition_size, num_stages
        self.fused = fused and new_tokens == 1   # one launch per layer when one token per sequence is appended
        S, T = shape.batch, shape.batch * new_tokens
        self.q = torch.empty((depth, S, shape.num_q_heads, HEAD_SIZE), dtype=dtype, device=dev)
        self.out = torch.empty_like(self.q)
        self.k = torch.empty((depth, T, shape.num_kv_heads, HEAD_SIZE), dtype=dtype, device=dev)
        self.v = torch.empty_like(self.k)
        self.bt = torch.empty((depth, S, shape.num_kv_heads, max_blocks_per_seq), dtype=torch.int32, device=dev)
        self.slots = torch.empty((T, shape.num_layers, shape.num_kv_heads), dtype=torch.int64, device=dev)
        self.ctx = torch.empty((S,), dtype=torch.int32, device=dev)
        # optional work list (ops.work_units of the host's context lengths, padded with -1 to a fixed length)
        self.units = torch.empty((units_capacity,), dtype=torch.int32, device=dev) if units_capacity > 0 else None
        self.copy_stream = torch.cuda.Stream(device=dev)
        self.out_stream = torch.cuda.Stream(device=dev)
        self.ready = [torch.cuda.Event() for _ in range(depth)]
        self.done = [torch.cuda.Event() for _ in range(depth)]
        self.free = [torch.cuda.Event() for _ in range(depth)]
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.launches = 0

    def run(self, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor, block_tables_host: torch.Tensor,
            slot_mapping_host: torch.Tensor, context_lens_host: torch.Tensor, out_host: torch.Tensor,
            max_context_len: int, units_host: torch.Tensor = None) -> None:
        """All ``*_host`` tensors are pinned CPU tensors: q/out [L, S, Hq, D], k/v [L, T, H, D],
        block_tables [L, S, H, max_blocks] int32, slot_mapping [T, L, H] int64, context_lens [S] int32.
        Returns when everything is enqueued; the caller's stream is ordered after the last download."""
        compute = torch.cuda.current_stream()
        cs, os_ = self.copy_stream, self.out_stream
        L = self.shape.num_layers
        cs.wait_stream(compute)          # a step's inputs exist only once the previous step is done
        h2d = d2h = 0
        with torch.cuda.stream(cs):
            self.ctx.copy_(context_lens_host, non_blocking=True)
            self.slots.copy_(slot_mapping_host, non_blocking=True)
            h2d += self.ctx.numel() * 4 + self.slots.numel() * 8
            if units_host is not None:
                self.units.copy_(units_host, non_blocking=True)
                h2d += self.units.numel() * 4
        for l in range(L):
            b = l % self.depth
            if l >= self.depth:
                cs.wait_event(self.free[b])
            with torch.cuda.stream(cs):
                self.q[b].copy_(q_host[l], non_blocking=True)
                self.k[b].copy_(k_host[l], non_blocking=True)
                self.v[b].copy_(v_host[l], non_blocking=True)
                self.bt[b].copy_(block_tables_host[l], non_blocking=True)
                self.ready[b].record(cs)
            h2d += (self.q[b].numel() + 2 * self.k[b].numel()) * self.q.element_size() + self.bt[b].numel() * 4
            compute.wait_event(self.ready[b])
            if self.fused:
                ops.decode_attention(self.out[b], self.q[b], self.k[b], self.v[b], self.kc, self.vc, None,
                                     HEAD_SIZE ** -0.5, self.bt[b], self.ctx, self.block_size, max_context_len,
                                     partition_size=self.partition_size, num_stages=self.num_stages,
                                     units=self.units if units_host is not None else None)
            else:
                ops.reshape_and_cache(self.k[b], self.v[b], self.kc, self.vc, self.slots[:, l, :])
                ops.paged_attention(self.out[b], self.q[b], self.kc, self.vc, None, HEAD_SIZE ** -0.5, self.bt[b],
                                    self.ctx, self.block_size, max_context_len,
                                    partition_size=self.partition_size, num_stages=self.num_stages)
            self.done[b].record(compute)
            os_.wait_event(self.done[b])
            with torch.cuda.stream(os_):
                out_host[l].copy_(self.out[b], non_blocking=True)
                self.free[b].record(os_)
            d2h += self.out[b].numel() * self.out.element_size()
        compute.wait_stream(os_)
        self.h2d_bytes, self.d2h_bytes = h2d, d2h
