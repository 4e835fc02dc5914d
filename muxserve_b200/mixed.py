"""Descriptors for ONE attention launch over the decode batches of several colocated models.

MuxServe runs every model in its own processes (muxserve/muxsched/scheduler.py:167-208) over one
shared pool; block ids are globally unique because a single allocator serves all models
(muxserve/flexstore/manager.py:397-398).  That makes a fused launch possible: an *item* is one
(sequence, kv head) of some model, and the kernel needs per item only its context length, its first
row in a packed q / out matrix, its group size (q heads per kv head), its softmax scale and its block
list.  Models are ordered by layer count, deepest first, so that the models that still have layer
``l`` always form a prefix of the item arrays and of the packed rows.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import numpy as np
import torch


@dataclass
class ModelBatch:
    """Decode batch of one model on this GPU (local head counts)."""
    name: str
    num_layers: int
    num_q_heads: int
    num_kv_heads: int
    scale: float
    context_lens: torch.Tensor      # int32 [S] (CPU or device)
    block_tables: torch.Tensor      # int32 [L, S, H, max_blocks] on the device

    @property
    def group(self) -> int:
        return self.num_q_heads // self.num_kv_heads

    @property
    def num_seqs(self) -> int:
        return int(self.context_lens.numel())


@dataclass
class MixedPlan:
    order: List[int]                 # indices into the caller's list, deepest model first
    item_context_len: torch.Tensor   # int32 [items] device
    item_q_row: torch.Tensor         # int32 [items]
    item_group: torch.Tensor         # int32 [items]
    item_scale: torch.Tensor         # float32 [items]
    block_tables: torch.Tensor       # int32 [L_max, items, max_blocks]; rows of models without layer l unused
    row_offset: List[int]            # first packed q row of each model (in `order`), plus the total
    item_offset: List[int]           # first item of each model (in `order`), plus the total
    layers: List[int]                # layer count of each model (in `order`)
    max_group: int
    max_context_len: int
    item_context_len_host: np.ndarray = None   # the same lengths on the host (work lists, launch heuristics)
    tp: int = 1                      # rows laid out for `tp` tensor-parallel ranks (see build_mixed_plan)
    tp_rank: int = 0

    def active(self, layer: int):
        """(number of items, number of packed rows) that take part in `layer`."""
        k = sum(1 for n in self.layers if n > layer)
        return self.item_offset[k], self.row_offset[k]

    def units(self, layer: int, partition_size: int = 512) -> torch.Tensor:
        """Work list of `layer` for ``ops.paged_attention_mixed(..., units=, partition_size=)``: one int32
        ``item | partition << 24`` per real (item, partition) pair, full partitions first, so that the launch has
        no CTA that only finds out it has nothing to do and the longest pieces of work start first."""
        n_items, _ = self.active(layer)
        key = (n_items, partition_size)
        cache = self.__dict__.setdefault("_units", {})
        if key not in cache:
            from .ops import work_units
            cache[key] = work_units(self.item_context_len_host[:n_items], partition_size,
                                    self.item_context_len.device)
        return cache[key]


def build_mixed_plan(batches: Sequence[ModelBatch], device, tp: int = 1, tp_rank: int = 0) -> MixedPlan:
    """``tp`` > 1: the batches hold the LOCAL heads of tensor-parallel rank ``tp_rank``; the packed q / out matrix is
    then laid out as every model's full ``[S, tp * local q heads, D]`` with this rank's heads at their global
    position, so that the sum of the ranks' ``out`` matrices (the TP all-reduce) is the models' whole output and
    rows of other ranks' heads stay untouched (zero)."""
    order = sorted(range(len(batches)), key=lambda i: -batches[i].num_layers)
    ctx_all, row_all, grp_all, scl_all = [], [], [], []
    row_offset, item_offset, layers = [0], [0], []
    max_blocks = max(b.block_tables.shape[-1] for b in batches)
    L_max = max(b.num_layers for b in batches)
    for i in order:
        b = batches[i]
        S, H, G = b.num_seqs, b.num_kv_heads, b.group
        if b.num_q_heads % b.num_kv_heads or G > 8:
            raise ValueError(f"{b.name}: q heads per kv head must be an integer <= 8 for the fused launch")
        ctx = b.context_lens.cpu().numpy().astype(np.int32)
        s_idx, h_idx = np.meshgrid(np.arange(S), np.arange(H), indexing="ij")
        ctx_all.append(np.repeat(ctx, H))
        row_all.append((row_offset[-1] + s_idx * (b.num_q_heads * tp) + tp_rank * b.num_q_heads + h_idx * G)
                       .reshape(-1).astype(np.int32))
        grp_all.append(np.full(S * H, G, dtype=np.int32))
        scl_all.append(np.full(S * H, b.scale, dtype=np.float32))
        row_offset.append(row_offset[-1] + S * b.num_q_heads * tp)
        item_offset.append(item_offset[-1] + S * H)
        layers.append(b.num_layers)
    n_items = item_offset[-1]
    tables = torch.zeros((L_max, n_items, max_blocks), dtype=torch.int32, device=device)
    for k, i in enumerate(order):
        b = batches[i]
        bt = b.block_tables.to(device).clamp_min(0)
        L, S, H, mb = bt.shape
        tables[:L, item_offset[k]:item_offset[k + 1], :mb] = bt.reshape(L, S * H, mb)
    cat = lambda xs, dt: torch.from_numpy(np.concatenate(xs)).to(dt).to(device)
    return MixedPlan(order=order, item_context_len=cat(ctx_all, torch.int32), item_q_row=cat(row_all, torch.int32),
                     item_group=cat(grp_all, torch.int32), item_scale=cat(scl_all, torch.float32),
                     block_tables=tables, row_offset=row_offset, item_offset=item_offset, layers=layers,
                     max_group=max(b.group for b in batches),
                     max_context_len=int(max(int(b.context_lens.max()) for b in batches)),
                     item_context_len_host=np.concatenate(ctx_all).astype(np.int64), tp=tp, tp_rank=tp_rank)


def plan_from_schedulers(models, device, max_blocks: int, tp: int = 1, tp_rank: int = 0) -> MixedPlan:
    """The same plan built by the host library straight from the models' step builders
    (``mux_batch_scheduler_get_batch_mixed``): ``models`` is a list of ``(BatchScheduler, request ids of its decode
    batch, local q heads, softmax scale)``; call after every scheduler's ``get_batch_info`` of the step.
    ``plan.order`` indexes that list, deepest model first."""
    import ctypes as C

    from . import _lib
    n = len(models)
    arr = (_lib.MixedModel * n)()
    keep = []
    for m, (sched, req_ids, num_q_heads, scale) in enumerate(models):
        ids = np.ascontiguousarray(np.asarray(req_ids, dtype=np.int32))
        keep.append(ids)
        arr[m] = _lib.MixedModel(sched._h, _lib.i32p(ids), ids.size, int(num_q_heads), float(scale))
    spans = (_lib.MixedSpan * n)()
    totals = np.zeros(5, dtype=np.int32)
    L = _lib.lib()
    _lib.check(L.mux_batch_scheduler_get_batch_mixed(arr, n, tp, tp_rank, max_blocks, None, None, None, None, None, 0,
                                                     spans, _lib.i32p(totals)), "get_batch_mixed (sizes)")
    items, rows, layers_max, max_group = (int(x) for x in totals[:4])
    ctx = np.empty(items, dtype=np.int32)
    row = np.empty(items, dtype=np.int32)
    grp = np.empty(items, dtype=np.int32)
    scl = np.empty(items, dtype=np.float32)
    tables = np.empty((layers_max, items, max_blocks), dtype=np.int32)
    _lib.check(L.mux_batch_scheduler_get_batch_mixed(arr, n, tp, tp_rank, max_blocks, _lib.i32p(ctx), _lib.i32p(row),
                                                     _lib.i32p(grp), scl.ctypes.data_as(C.POINTER(C.c_float)),
                                                     _lib.i32p(tables), tables.size, spans, _lib.i32p(totals)),
               "get_batch_mixed")
    up = lambda a: torch.from_numpy(a).to(device)
    return MixedPlan(order=[spans[k].model for k in range(n)], item_context_len=up(ctx), item_q_row=up(row),
                     item_group=up(grp), item_scale=up(scl), block_tables=up(tables),
                     row_offset=[spans[k].first_row for k in range(n)] + [rows],
                     item_offset=[spans[k].first_item for k in range(n)] + [items],
                     layers=[spans[k].num_layers for k in range(n)], max_group=max_group,
                     max_context_len=int(totals[4]), item_context_len_host=ctx.astype(np.int64), tp=tp, tp_rank=tp_rank)


def pack_rows(plan: MixedPlan, per_model: Sequence[torch.Tensor]) -> torch.Tensor:
    """Places per-model [S, Hq, D] tensors (caller's order) into the packed [rows, D] matrix (rows of other
    tensor-parallel ranks' heads are zero)."""
    if plan.tp == 1:
        return torch.cat([per_model[i].reshape(-1, per_model[i].shape[-1]) for i in plan.order], dim=0)
    D = per_model[0].shape[-1]
    out = torch.zeros((plan.row_offset[-1], D), dtype=per_model[0].dtype, device=per_model[0].device)
    for k, i in enumerate(plan.order):
        S, Hq, _ = per_model[i].shape
        view = out[plan.row_offset[k]:plan.row_offset[k + 1]].view(S, Hq * plan.tp, D)
        view[:, plan.tp_rank * Hq:(plan.tp_rank + 1) * Hq] = per_model[i]
    return out


def pack_items(plan: MixedPlan, per_model: Sequence[torch.Tensor]) -> torch.Tensor:
    """Concatenates per-model [S, H, D] tensors (one row per (sequence, kv head), e.g. the new K / V rows) into the
    [items, D] matrix in item order."""
    return torch.cat([per_model[i].reshape(-1, per_model[i].shape[-1]) for i in plan.order], dim=0)


def unpack_rows(plan: MixedPlan, packed: torch.Tensor, batches: Sequence[ModelBatch]) -> List[torch.Tensor]:
    """Views of the packed matrix per model (this rank's heads), in the caller's order."""
    out = [None] * len(batches)
    for k, i in enumerate(plan.order):
        b = batches[i]
        view = packed[plan.row_offset[k]:plan.row_offset[k + 1]].view(b.num_seqs, b.num_q_heads * plan.tp, packed.shape[-1])
        out[i] = view[:, plan.tp_rank * b.num_q_heads:(plan.tp_rank + 1) * b.num_q_heads]
    return out
