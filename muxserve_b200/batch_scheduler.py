"""``BatchScheduler`` — per-model step builder (host C++ behind the C ABI).

Same methods and results as the pybind class ``muxserve.batch_scheduler.BatchScheduler``
(csrc/batch_scheduler.cpp:201-211) as driven by ``LLMRuntime.prepare_inputs``
(muxserve/flexserver/llm_runtime.py:277-339).  ``get_batch`` fills caller-provided
CPU tensors exactly like the reference; block-table padding is written as 0.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence

import numpy as np
import torch

from ._lib import check, i32p, i64p, lib


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32).reshape(-1))


def _np_view(t: torch.Tensor, dtype: torch.dtype, name: str) -> np.ndarray:
    if t.device.type != "cpu" or t.dtype != dtype or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous CPU tensor of {dtype}")
    return t.numpy().reshape(-1)


class BatchScheduler:
    def __init__(self, num_layers: int, num_heads: int, max_seq_len: int, block_size: int):
        self._lib = lib()
        self._h = self._lib.mux_batch_scheduler_create(int(num_layers), int(num_heads), int(max_seq_len),
                                                       int(block_size))
        if not self._h:
            raise ValueError("BatchScheduler: sizes must be positive")
        self.num_layers, self.num_heads = int(num_layers), int(num_heads)
        self.max_seq_len, self.block_size = int(max_seq_len), int(block_size)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.mux_batch_scheduler_destroy(h)

    def add_request(self, prompt, req_id: int, max_tokens: int) -> None:
        p = _i32(prompt)
        check(self._lib.mux_batch_scheduler_add_request(self._h, i32p(p), p.size, int(req_id), int(max_tokens)),
              "BatchScheduler.add_request")

    def try_batch(self, batch_request_ids: Sequence[int], batch_last_output_tokens: Sequence[int]) -> np.ndarray:
        """Rows ``[request id, blocks needed, has_blocks]`` + total (batch_scheduler.cpp:22-48).

        A non-empty token list makes this a decode step: every request's new
        token is appended to its logical state before the allocator is asked.
        """
        ids = _i32(batch_request_ids)
        last = _i32(batch_last_output_tokens)
        out = np.empty(3 * ids.size + 1, dtype=np.int32)
        check(self._lib.mux_batch_scheduler_try_batch(self._h, i32p(ids), ids.size, i32p(last), last.size,
                                                      i32p(out)), "BatchScheduler.try_batch")
        return out

    def get_batch_info(self, batch_block_request, block_info) -> List[int]:
        """Stores granted block ids and returns ``[numTokens, numContexts, maxContextLen,
        maxBlocksPerSeq, L, H, prompt lens...]`` (batch_scheduler.cpp:51-97)."""
        req, info = _i32(batch_block_request), _i32(block_info)
        n = req.size // 3
        out = np.empty(6 + n, dtype=np.int32)
        out_len = C.c_int32(0)
        check(self._lib.mux_batch_scheduler_get_batch_info(self._h, i32p(req), n, i32p(info), info.size,
                                                           i32p(out), out.size, C.byref(out_len)),
              "BatchScheduler.get_batch_info")
        return out[:out_len.value].tolist()

    def _fill(self, fn, where, batch_info, block_info, token_tensor, token_position_tensor, context_len_tensor,
              block_table_tensor, slot_mapping_tensor) -> None:
        req, info = _i32(batch_info), _i32(block_info)
        tok = _np_view(token_tensor, torch.int32, "token tensor")
        pos = _np_view(token_position_tensor, torch.int32, "position tensor")
        ctx = _np_view(context_len_tensor, torch.int32, "context_len tensor")
        bt = _np_view(block_table_tensor, torch.int32, "block_table tensor")
        sm = _np_view(slot_mapping_tensor, torch.int64, "slot_mapping tensor")
        if tok.size != pos.size:
            raise ValueError("token and position tensors differ in length")
        check(fn(self._h, i32p(req), req.size // 3, i32p(info), info.size, i32p(tok), i32p(pos), tok.size,
                 i32p(ctx), ctx.size, i32p(bt), bt.size, i64p(sm), sm.size), where)

    def get_batch(self, batch_info, block_info, token_tensor, token_position_tensor, context_len_tensor,
                  block_table_tensor, slot_mapping_tensor) -> None:
        """Fills the step's CPU tensors (batch_scheduler.cpp:99-193): block tables as
        [tokens, max_blocks, L, H], slot mapping as [tokens, L, H]."""
        self._fill(self._lib.mux_batch_scheduler_get_batch, "BatchScheduler.get_batch", batch_info, block_info,
                   token_tensor, token_position_tensor, context_len_tensor, block_table_tensor,
                   slot_mapping_tensor)

    def get_batch_decode_layered(self, batch_info, block_info, token_tensor, token_position_tensor,
                                 context_len_tensor, block_table_tensor, slot_mapping_tensor) -> None:
        """``get_batch`` for a decode step with block tables already in kernel order
        [L, seqs, H, max_blocks] (the reference permutes on the device, llm_runtime.py:327)."""
        self._fill(self._lib.mux_batch_scheduler_get_batch_decode_layered, "BatchScheduler.get_batch_decode_layered",
                   batch_info, block_info, token_tensor, token_position_tensor, context_len_tensor,
                   block_table_tensor, slot_mapping_tensor)

    def release_requests(self, request_ids: Sequence[int]) -> None:
        ids = _i32(request_ids)
        check(self._lib.mux_batch_scheduler_release_requests(self._h, i32p(ids), ids.size),
              "BatchScheduler.release_requests")

    def _vec(self, fn) -> List[int]:
        n = fn(self._h, None, 0)
        out = np.empty(max(n, 1), dtype=np.int32)
        fn(self._h, i32p(out), out.size)
        return out[:n].tolist()

    def get_preempt_requests(self) -> List[int]:
        return self._vec(self._lib.mux_batch_scheduler_preempt_requests)

    def get_prompt_info(self) -> List[int]:
        """Prompt lengths of the last batch followed by its max context length."""
        return self._vec(self._lib.mux_batch_scheduler_prompt_info)

    def get_batch_reqs(self) -> List[List[int]]:
        flat = self._vec(self._lib.mux_batch_scheduler_batch_reqs)
        return [flat[i:i + 2] for i in range(0, len(flat), 2)]

    # ---- introspection (not in the reference) ----
    def request_state(self, req_id: int) -> dict:
        out = np.empty(5, dtype=np.int32)
        check(self._lib.mux_batch_scheduler_request_state(self._h, int(req_id), i32p(out)),
              "BatchScheduler.request_state")
        keys = ("context_len", "num_physical_blocks", "logical_block_idx", "logical_block_offset", "num_outputs")
        return dict(zip(keys, out.tolist()))
