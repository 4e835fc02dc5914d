"""Tensor-parallel sharding of the attention path by kv head (host-side helpers).

MuxServe shards heads Megatron-style (muxserve/flexserver/models/llama.py:100-117): rank r owns
kv heads [r*H/tp, (r+1)*H/tp) and their q heads; when there are fewer kv heads than ranks the kv
heads are replicated (:109-114).  Block ids are identical on every rank (one allocator, equal
pools: muxserve/flexstore/manager.py:397-398,479-493) and each rank stores only its own heads'
blocks, so attention and the cache write need no cross-GPU traffic; the only collective is the
all-reduce of the row-parallel output projection (llama.py:131-137,162).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class HeadShard:
    tp: int
    rank: int
    q_start: int
    q_count: int
    kv_start: int
    kv_count: int
    kv_replicas: int   # ranks that hold a copy of each kv head (1 unless tp > total kv heads)


def shard_heads(total_q_heads: int, total_kv_heads: int, tp: int, rank: int) -> HeadShard:
    if total_q_heads % tp:
        raise ValueError(f"{total_q_heads} q heads do not divide over tp={tp}")
    qn = total_q_heads // tp
    if total_kv_heads >= tp:
        if total_kv_heads % tp:
            raise ValueError(f"{total_kv_heads} kv heads do not divide over tp={tp}")
        kn = total_kv_heads // tp
        return HeadShard(tp, rank, rank * qn, qn, rank * kn, kn, 1)
    if tp % total_kv_heads:
        raise ValueError(f"tp={tp} is not a multiple of {total_kv_heads} kv heads")
    rep = tp // total_kv_heads
    return HeadShard(tp, rank, rank * qn, qn, rank // rep, 1, rep)


def shard_qkv(shard: HeadShard, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
    """Views of the full [N, heads, D] tensors that belong to this rank."""
    return (q[:, shard.q_start:shard.q_start + shard.q_count],
            k[:, shard.kv_start:shard.kv_start + shard.kv_count],
            v[:, shard.kv_start:shard.kv_start + shard.kv_count])


def shard_index_tensors(shard: HeadShard, block_tables: torch.Tensor, slot_mapping: torch.Tensor):
    """block_tables [L, S, H, blk] and slot_mapping [T, L, H] restricted to this rank's kv heads.

    The reference broadcasts the full tensors to every rank (llm_runtime.py:389-400) and each rank's
    scheduler was built with the local head count, so the local view is what its kernels see."""
    sl = slice(shard.kv_start, shard.kv_start + shard.kv_count)
    return block_tables[:, :, sl, :], slot_mapping[:, :, sl]


def broadcast_grant(batch_block_request, block_info, src: int = 0, group: Optional[dist.ProcessGroup] = None,
                    device="cpu"):
    """Carries one step's allocator answer — the rows ``[request id, blocks, has_blocks]`` and ``[preempt_idx,
    ids...]``, a few KB — from the rank that runs the scheduler to every rank of the TP group.  The reference
    broadcasts the rebuilt ``slot_mapping`` / ``context_lens`` / ``block_tables`` tensors instead
    (muxserve/flexserver/llm_runtime.py:389-400: 33 MB per step for 64 LLaMA-7B sequences); here every rank applies
    the grant to its own ``DeviceBlockTables`` (its heads' columns).  ``device``: where the group's backend wants
    its tensors ("cpu" for gloo, the rank's GPU for nccl).  Returns the two int32 numpy arrays on every rank."""
    import numpy as np
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return np.asarray(batch_block_request, dtype=np.int32).reshape(-1), np.asarray(block_info, dtype=np.int32).reshape(-1)
    mine = dist.get_rank(group) == src
    head = torch.zeros(2, dtype=torch.int64, device=device)
    if mine:
        req = torch.as_tensor(np.asarray(batch_block_request, dtype=np.int32).reshape(-1))
        info = torch.as_tensor(np.asarray(block_info, dtype=np.int32).reshape(-1))
        head = torch.tensor([req.numel(), info.numel()], dtype=torch.int64, device=device)
    dist.broadcast(head, src=src, group=group)
    n_req, n_info = (int(x) for x in head.tolist())
    payload = torch.empty(n_req + n_info, dtype=torch.int32, device=device)
    if mine:
        payload.copy_(torch.cat([req, info]))
    dist.broadcast(payload, src=src, group=group)
    host = payload.cpu().numpy()
    return host[:n_req].copy(), host[n_req:].copy()


def all_reduce_output(partial: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Sum of the ranks' partial [tokens, hidden] outputs, in place (the TP all-reduce after o_proj)."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


def max_over_ranks(value: float, device=None, group: Optional[dist.ProcessGroup] = None) -> float:
    """Largest value over the ranks (how multi-GPU step times are reported)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
