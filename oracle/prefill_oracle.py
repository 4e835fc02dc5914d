"""CPU oracle for prompt-phase attention (test infrastructure only; never imported by the product path).

PARITY UNPINNED: the prompt branch of ``PagedAttentionWithRoPE`` lives in the un-vendored MuxServe-vLLM
fork (call site ``muxserve/flexserver/models/llama.py:160-161``, prompt lengths from
``muxserve/flexserver/llm_runtime.py:298-330``); the reference holds no source, test or golden vector
for it.  This restates its published semantics: every prompt attends causally to its own tokens
(block-diagonal causal mask over the concatenated rows), softmax in fp32, q head h reading kv head
h // (Hq // H).
"""
from __future__ import annotations

from typing import Sequence

import torch


def prefill_attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, prompt_lens: Sequence[int],
                          scale: float) -> torch.Tensor:
    """q [T, Hq, D], k/v [T, H, D] (any float dtype) -> fp32 [T, Hq, D]."""
    T, Hq, D = q.shape
    H = k.shape[1]
    group = Hq // H
    out = torch.zeros((T, Hq, D), dtype=torch.float32)
    qf, kf, vf = q.float().cpu(), k.float().cpu(), v.float().cpu()
    start = 0
    for n in prompt_lens:
        n = int(n)
        if n == 0:
            continue
        qs = qf[start:start + n].permute(1, 0, 2)                                   # [Hq, n, D]
        ks = kf[start:start + n].permute(1, 0, 2).repeat_interleave(group, dim=0)   # [Hq, n, D]
        vs = vf[start:start + n].permute(1, 0, 2).repeat_interleave(group, dim=0)
        logits = torch.matmul(qs, ks.transpose(1, 2)) * scale
        mask = torch.ones((n, n), dtype=torch.bool).tril()
        logits = logits.masked_fill(~mask, float("-inf"))
        w = torch.softmax(logits, dim=-1)
        out[start:start + n] = torch.matmul(w, vs).permute(1, 0, 2)
        start += n
    return out
