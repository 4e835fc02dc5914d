"""fp32 gather-based restatement of decode paged attention.  TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED: the op's source is in the un-vendored MuxServe-vLLM fork and the
reference has no test or golden vector for it.  Call site:
muxserve/flexserver/models/llama.py:160-161; pool layout:
muxserve/flexstore/manager.py:456-468; per-layer block tables [S, H, max_blocks]:
muxserve/flexserver/llm_runtime.py:327.

For sequence s, q head hq with kv head h = head_mapping[hq]:
    K_j = key_pool  [bt[s,h,j // B]][:, j % B, :]  flattened over (d/x, x)   j < ctx_s
    V_j = value_pool[bt[s,h,j // B]][:, j % B]
    out[s,hq] = softmax_j(scale * q[s,hq] . K_j) . V_j          (fp32 throughout)
"""
from __future__ import annotations

from typing import Optional

import torch


def gather_kv(key_cache: torch.Tensor, value_cache: torch.Tensor, block_ids: torch.Tensor, ctx: int):
    """De-interleaves the named blocks into K, V of shape [ctx, D] (fp32)."""
    nb, dx, B, x = key_cache.shape
    ids = block_ids.long()
    k = key_cache[ids]                       # [n, D/x, B, x]
    k = k.permute(0, 2, 1, 3).reshape(-1, dx * x)[:ctx]
    v = value_cache[ids]                     # [n, D, B]
    v = v.permute(0, 2, 1).reshape(-1, value_cache.shape[1])[:ctx]
    return k.float(), v.float()


def paged_attention_ref(q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                        head_mapping: Optional[torch.Tensor], scale: float, block_tables: torch.Tensor,
                        context_lens: torch.Tensor, block_size: int) -> torch.Tensor:
    """q [S, Hq, D]; block_tables [S, H, max_blocks] (or [S, max_blocks]); returns fp32 [S, Hq, D]."""
    S, Hq, D = q.shape
    if block_tables.dim() == 2:
        block_tables = block_tables.unsqueeze(1)
    if head_mapping is None:
        Hkv = block_tables.shape[1] if block_tables.shape[1] > 1 else Hq
        G = Hq // Hkv
        head_mapping = torch.arange(Hq) // G
    out = torch.zeros(S, Hq, D, dtype=torch.float32)
    qf = q.float()
    for s in range(S):
        ctx = int(context_lens[s])
        if ctx <= 0:
            continue
        nblk = (ctx + block_size - 1) // block_size
        cache = {}
        for hq in range(Hq):
            h = int(head_mapping[hq])
            hb = h if block_tables.shape[1] > 1 else 0
            if hb not in cache:
                cache[hb] = gather_kv(key_cache, value_cache, block_tables[s, hb, :nblk], ctx)
            k, v = cache[hb]
            logits = (k @ qf[s, hq]) * scale
            p = torch.softmax(logits, dim=0)
            out[s, hq] = p @ v
    return out


def paged_attention_items_ref(q_rows: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                              block_tables: torch.Tensor, item_context_len, item_q_row, item_group, item_scale,
                              block_size: int) -> torch.Tensor:
    """Mixed-model form: item i = rows item_q_row[i]..+item_group[i] of q_rows [R, D] over block_tables[i]."""
    out = torch.zeros(q_rows.shape, dtype=torch.float32)
    qf = q_rows.float()
    for i in range(block_tables.shape[0]):
        ctx = int(item_context_len[i])
        if ctx <= 0:
            continue
        nblk = (ctx + block_size - 1) // block_size
        k, v = gather_kv(key_cache, value_cache, block_tables[i, :nblk], ctx)
        r0, g = int(item_q_row[i]), int(item_group[i])
        logits = (qf[r0:r0 + g] @ k.T) * float(item_scale[i])
        out[r0:r0 + g] = torch.softmax(logits, dim=1) @ v
    return out


def paged_attention_ref_batched(q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, scale: float,
                                block_tables: torch.Tensor, context_lens: torch.Tensor, block_size: int) -> torch.Tensor:
    """Same arithmetic for contiguous head groups, one batched gather per sequence (the timed CPU baseline)."""
    S, Hq, D = q.shape
    H = block_tables.shape[1]
    G = Hq // H
    out = torch.empty(S, Hq, D, dtype=torch.float32)
    dx, x = key_cache.shape[1], key_cache.shape[3]
    for s in range(S):
        ctx = int(context_lens[s])
        nblk = (ctx + block_size - 1) // block_size
        ids = block_tables[s, :, :nblk].long()                       # [H, n]
        k = key_cache[ids].permute(0, 1, 3, 2, 4).reshape(H, nblk * block_size, dx * x)[:, :ctx].float()
        v = value_cache[ids].permute(0, 1, 3, 2).reshape(H, nblk * block_size, D)[:, :ctx].float()
        qs = q[s].float().view(H, G, D)
        p = torch.softmax(torch.bmm(qs, k.transpose(1, 2)) * scale, dim=-1)
        out[s] = torch.bmm(p, v).view(Hq, D)
    return out
