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

Two extensions serve the other callers of the step:
* ``device_tables`` — block tables that are already on the device for the whole step (the
  reference's ``[L, S, H, max_blocks]`` tensor after its upload + permute, or the persistent table of
  ``device_tables.DeviceBlockTables`` together with ``seq_rows``): the per-layer table upload is skipped;
* ``out_views`` / ``post`` — tensor-parallel ranks write their heads' output into a slice of a
  ``[S, hidden]`` buffer and ``post(slot)`` (the output all-reduce) returns what is downloaded.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from . import ops
from .workloads import HEAD_SIZE, ModelShape


class HostDecodeStep:
    def __init__(self, shape: ModelShape, block_size: int, dtype: torch.dtype, key_cache: torch.Tensor,
                 value_cache: torch.Tensor, max_blocks_per_seq: int, new_tokens: int = 1, depth: int = 4,
                 partition_size: int = 0, num_stages: int = 0, fused: bool = True, units_capacity: int = 0,
                 out_views: Optional[List[torch.Tensor]] = None,
                 post: Optional[Callable[[int], torch.Tensor]] = None, early_kv: bool = False):
        dev = key_cache.device
        self.shape, self.block_size, self.dtype = shape, block_size, dtype
        self.kc, self.vc = key_cache, value_cache
        self.depth = depth
        self.partition_size, self.num_stages = partition_size, num_stages
        self.early_kv = early_kv
        self.new_tokens = new_tokens
        self.fused = fused and new_tokens <= ops.MAX_FUSED_NEW_TOKENS   # one launch per layer
        S, T = shape.batch, shape.batch * new_tokens
        self.q = torch.empty((depth, S, shape.num_q_heads, HEAD_SIZE), dtype=dtype, device=dev)
        if out_views is not None and len(out_views) != depth:
            raise ValueError("out_views needs one tensor per pipeline slot")
        self.out = out_views if out_views is not None else list(torch.empty_like(self.q))
        self.post = post
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

    def run(self, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor,
            block_tables_host: Optional[torch.Tensor], slot_mapping_host: Optional[torch.Tensor],
            context_lens_host: torch.Tensor, out_host: torch.Tensor, max_context_len: int,
            units_host: torch.Tensor = None, device_tables: Optional[torch.Tensor] = None,
            seq_rows: Optional[torch.Tensor] = None) -> None:
        """All ``*_host`` tensors are pinned CPU tensors: q [L, S, Hq, D], k/v [L, T, H, D],
        block_tables [L, S, H, max_blocks] int32 (or ``None`` with ``device_tables``), slot_mapping [T, L, H] int64
        (``None``: not uploaded), context_lens [S] int32, out [L, ...] (what ``post`` returns, else [S, Hq, D]).
        Returns when everything is enqueued; the caller's stream is ordered after the last download."""
        compute = torch.cuda.current_stream()
        cs, os_ = self.copy_stream, self.out_stream
        L = self.shape.num_layers
        cs.wait_stream(compute)          # a step's inputs exist only once the previous step is done
        h2d = d2h = 0
        with torch.cuda.stream(cs):
            self.ctx.copy_(context_lens_host, non_blocking=True)
            h2d += self.ctx.numel() * 4
            if slot_mapping_host is not None:
                self.slots.copy_(slot_mapping_host, non_blocking=True)
                h2d += self.slots.numel() * 8
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
                if device_tables is None:
                    self.bt[b].copy_(block_tables_host[l], non_blocking=True)
                    h2d += self.bt[b].numel() * 4
                self.ready[b].record(cs)
            h2d += (self.q[b].numel() + 2 * self.k[b].numel()) * self.q.element_size()
            compute.wait_event(self.ready[b])
            bt = self.bt[b] if device_tables is None else device_tables[l]
            if self.fused:
                ops.decode_attention(self.out[b], self.q[b], self.k[b], self.v[b], self.kc, self.vc, None,
                                     HEAD_SIZE ** -0.5, bt, self.ctx, self.block_size, max_context_len,
                                     partition_size=self.partition_size, num_stages=self.num_stages,
                                     units=self.units if units_host is not None else None, seq_rows=seq_rows,
                                     early_kv=self.early_kv and device_tables is None)
            else:
                ops.reshape_and_cache(self.k[b], self.v[b], self.kc, self.vc, self.slots[:, l, :])
                ops.paged_attention(self.out[b], self.q[b], self.kc, self.vc, None, HEAD_SIZE ** -0.5, bt,
                                    self.ctx, self.block_size, max_context_len,
                                    partition_size=self.partition_size, num_stages=self.num_stages, seq_rows=seq_rows)
            result = self.out[b] if self.post is None else self.post(b)
            self.done[b].record(compute)
            os_.wait_event(self.done[b])
            with torch.cuda.stream(os_):
                out_host[l].copy_(result, non_blocking=True)
                self.free[b].record(os_)
            d2h += result.numel() * result.element_size()
        compute.wait_stream(os_)
        self.h2d_bytes, self.d2h_bytes = h2d, d2h
