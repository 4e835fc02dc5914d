"""Scatter-copy restatement of reshape_and_cache.  TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED (op source in the un-vendored MuxServe-vLLM fork; no reference test).
Layout from muxserve/flexstore/manager.py:456-468, slot formula from
csrc/batch_scheduler.h:42-67:
    b = slot // B, o = slot % B
    key_pool[b, d // x, o, d % x] = k[t, h, d];  value_pool[b, d, o] = v[t, h, d]
"""
from __future__ import annotations

import torch


def reshape_and_cache_ref(k: torch.Tensor, v: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                          slot_mapping: torch.Tensor) -> None:
    """k, v [T, H, D]; slot_mapping int64 [T, H]; pools are modified in place (CPU tensors)."""
    T, H, D = k.shape
    nb, dx, B, x = key_cache.shape
    slots = slot_mapping.reshape(-1)
    keep = slots >= 0
    slots = slots[keep]
    b = slots // B
    o = slots % B
    kk = k.reshape(T * H, dx, x)[keep]
    vv = v.reshape(T * H, D)[keep]
    key_cache[b, :, o, :] = kk
    value_cache[b, :, o] = vv
