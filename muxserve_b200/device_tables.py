"""Block tables that stay on the device and are updated incrementally.

The reference rebuilds the [tokens, max_blocks, L, H] table on the host every step, uploads it
(33.5 MB for 64 LLaMA-7B sequences of up to 2048 tokens) and permutes it on the device
(csrc/batch_scheduler.cpp:156-169, muxserve/flexserver/llm_runtime.py:322-327).  A decode step
changes the table only where a sequence crosses a block boundary, so here every request owns a
row of a persistent device table [L, rows, H, max_blocks]; the blocks the allocator grants are
staged on the host and scattered into the table by one small kernel per step, and the attention
ops reach a sequence's lists through ``seq_rows``.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import numpy as np
import torch

from ._lib import check, lib


class DeviceBlockTables:
    """``num_kv_heads`` are the heads THIS process attends over.  On a tensor-parallel rank they are a slice
    ``[kv_head_start, kv_head_start + num_kv_heads)`` of the model's ``total_kv_heads``: the allocator grants ids for
    all heads of a logical block (one allocator serves every rank, muxserve/flexstore/manager.py:397-398) and every
    rank keeps its own heads' columns of the same small grant (``parallel.broadcast_grant`` carries it) instead of
    receiving the whole rebuilt table (muxserve/flexserver/llm_runtime.py:389-400)."""

    def __init__(self, num_layers: int, num_kv_heads: int, max_rows: int, max_blocks: int, device="cuda",
                 total_kv_heads: int = None, kv_head_start: int = 0):
        self.L, self.H, self.R, self.max_blocks = num_layers, num_kv_heads, max_rows, max_blocks
        self.H_total = num_kv_heads if total_kv_heads is None else int(total_kv_heads)
        self.h0 = int(kv_head_start)
        if self.h0 < 0 or self.h0 + self.H > self.H_total:
            raise ValueError("the local kv heads must be a slice of the model's")
        self.tables = torch.zeros((num_layers, max_rows, num_kv_heads, max_blocks), dtype=torch.int32, device=device)
        self.row_of: Dict[int, int] = {}
        self.blocks_of: Dict[int, int] = {}          # physical blocks already in the table, per request
        self._free: List[int] = list(range(max_rows - 1, -1, -1))
        self._rows: List[int] = []
        self._blks: List[int] = []
        self._ids: List[np.ndarray] = []
        self.uploaded_bytes = 0

    def assign(self, req_id: int) -> int:
        """Gives the request a row (idempotent)."""
        if req_id not in self.row_of:
            if not self._free:
                raise RuntimeError("DeviceBlockTables: no free row")
            self.row_of[req_id] = self._free.pop()
            self.blocks_of[req_id] = 0
        return self.row_of[req_id]

    def release(self, req_ids: Sequence[int]) -> None:
        """Frees the rows of finished or preempted requests (their stale entries are never read:
        a row is rewritten from block 0 when it is assigned again)."""
        for r in req_ids:
            row = self.row_of.pop(int(r), None)
            if row is not None:
                self._free.append(row)
                self.blocks_of.pop(int(r), None)

    def stage_grant(self, batch_block_request, block_info) -> None:
        """Stages the blocks the allocator just granted: ``batch_block_request`` rows
        ``[request id, blocks, has_blocks]`` and ``block_info`` ``[preempt_idx, ids...]`` exactly as
        ``BatchScheduler.get_batch_info`` consumes them (csrc/batch_scheduler.cpp:51-97): every
        granted logical block is L*H ids in [layer][head] order."""
        req = np.asarray(batch_block_request, dtype=np.int64).reshape(-1, 3)
        info = np.asarray(block_info, dtype=np.int32)
        keep, off, LH = int(info[0]), 1, self.L * self.H_total
        for i in range(min(keep, len(req))):
            rid, n = int(req[i, 0]), int(req[i, 1])
            if n <= 0:
                continue
            row = self.assign(rid)
            first = self.blocks_of[rid]
            if first + n > self.max_blocks:
                raise RuntimeError(f"request {rid} outgrows the table ({first + n} > {self.max_blocks} blocks)")
            for j in range(n):
                self._rows.append(row)
                self._blks.append(first + j)
            ids = info[off:off + n * LH].reshape(n, self.L, self.H_total)[:, :, self.h0:self.h0 + self.H]
            self._ids.append(np.ascontiguousarray(ids).reshape(n, self.L * self.H))
            off += n * LH
            self.blocks_of[rid] = first + n
        for i in range(max(keep, 0), len(req)):           # preempted by the allocator
            self.release([int(req[i, 0])])

    def flush(self) -> int:
        """Uploads the staged grants (a few KB) and scatters them into the table; returns the update count."""
        n = len(self._rows)
        if n == 0:
            return 0
        dev = self.tables.device
        rows = torch.tensor(self._rows, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        blks = torch.tensor(self._blks, dtype=torch.int32).pin_memory().to(dev, non_blocking=True)
        ids = torch.from_numpy(np.concatenate(self._ids, axis=0)).pin_memory().to(dev, non_blocking=True)
        self.uploaded_bytes += 8 * n + ids.numel() * 4
        t = self.tables
        check(lib().mux_block_table_append(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2), self.L, self.R, self.H,
                                           self.max_blocks, rows.data_ptr(), blks.data_ptr(), ids.data_ptr(), n,
                                           torch.cuda.current_stream().cuda_stream), "block_table_append")
        self._rows, self._blks, self._ids = [], [], []
        self._keepalive = (rows, blks, ids)               # until the next flush; the kernel is asynchronous
        return n

    def rows_for(self, req_ids: Sequence[int]) -> torch.Tensor:
        """int32 device tensor: the table row of every sequence of the batch, in batch order."""
        host = torch.tensor([self.row_of[int(r)] for r in req_ids], dtype=torch.int32)
        self.uploaded_bytes += host.numel() * 4
        return host.pin_memory().to(self.tables.device, non_blocking=True)
