"""fp32 restatement of rotary position embedding (GPT-NeoX pairing).  TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED: the op lives in the un-vendored MuxServe-vLLM fork (PagedAttentionWithRoPE,
constructed at muxserve/flexserver/models/llama.py:138-147 with rotary_dim = head size, base =
rope_theta); the reference holds no test or golden vector for it.  Published algorithm (RoFormer /
GPT-NeoX): inv_freq_i = base^(-2i/D); for position p and i < D/2:
    x'[i]       = x[i] * cos(p * inv_freq_i) - x[i + D/2] * sin(p * inv_freq_i)
    x'[i + D/2] = x[i + D/2] * cos(...)      + x[i] * sin(...)
"""
from __future__ import annotations

import torch


def make_cos_sin_cache(max_position: int, base: float = 10000.0, dim: int = 128) -> torch.Tensor:
    """[max_position, dim] fp32: dim/2 cosines then dim/2 sines."""
    inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    freqs = torch.outer(torch.arange(max_position, dtype=torch.float32), inv_freq)
    return torch.cat([freqs.cos(), freqs.sin()], dim=-1)


def rotary_ref(x: torch.Tensor, positions: torch.Tensor, cache: torch.Tensor) -> torch.Tensor:
    """x [T, heads, D] (any dtype) -> rotated fp32; cache [max_position, D] in the dtype the kernel reads."""
    T, _, D = x.shape
    cs = cache[positions.long()].float()
    cos, sin = cs[:, None, :D // 2], cs[:, None, D // 2:]
    xf = x.float()
    x1, x2 = xf[..., :D // 2], xf[..., D // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)
