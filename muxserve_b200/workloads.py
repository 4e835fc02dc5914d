"""Seeded synthetic decode workloads with the shapes of the benchmark configurations.

The reference measures on ShareGPT / LMSYS traces that are not redistributable;
these generators stand in for them: query / key / value entries ~ N(0, 1),
context lengths from the stated distribution, and every (layer, sequence, kv
head) block list scattered without replacement over the pool, as a long-running
FlexStore pool would be.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from . import flexstore

HEAD_SIZE = flexstore.HEAD_SIZE


@dataclass
class ModelShape:
    name: str
    num_layers: int
    num_q_heads: int   # local (per tensor-parallel rank)
    num_kv_heads: int  # local
    batch: int

    @property
    def group(self) -> int:
        return self.num_q_heads // self.num_kv_heads


@dataclass
class DecodeCase:
    """One decode step of one model on one GPU (all layers)."""
    shape: ModelShape
    block_size: int
    dtype: torch.dtype
    scale: float
    context_lens: torch.Tensor   # int32 [S], includes the token written this step
    block_tables: torch.Tensor   # int32 [L, S, H, max_blocks]; entries past a list's end are -1
    slot_mapping: torch.Tensor   # int64 [T, L, H]
    q: torch.Tensor              # [L_q, S, Hq, D]   (L_q = distinct per-layer inputs kept)
    k: torch.Tensor              # [L_q, T, H, D]
    v: torch.Tensor              # [L_q, T, H, D]
    new_tokens: int = 1
    max_context_len: int = 0
    seed: int = 0
    extra: dict = field(default_factory=dict)


def uniform_context_lens(n: int, lo: int, hi: int, gen: torch.Generator) -> torch.Tensor:
    return torch.randint(lo, hi + 1, (n,), generator=gen, dtype=torch.int64).to(torch.int32)


def lognormal_context_lens(n: int, median: float, sigma: float, lo: int, hi: int,
                           gen: torch.Generator) -> torch.Tensor:
    z = torch.randn(n, generator=gen, dtype=torch.float64)
    x = torch.exp(math.log(median) + sigma * z).round().clamp(lo, hi)
    return x.to(torch.int32)


def fill_pool_(key_cache: torch.Tensor, value_cache: torch.Tensor, seed: int, chunk_elems: int = 1 << 28) -> None:
    """In-place N(0,1) fill of both pool tensors, chunked so no large temporary is made."""
    gen = torch.Generator(device=key_cache.device)
    gen.manual_seed(seed)
    for t in (key_cache, value_cache):
        flat = t.view(-1)
        for a in range(0, flat.numel(), chunk_elems):
            flat[a:a + chunk_elems].normal_(generator=gen)


def scatter_block_tables(context_lens: torch.Tensor, num_layers: int, num_kv_heads: int, block_size: int,
                         block_ids: torch.Tensor, first: int = 0):
    """Deals ids from ``block_ids[first:]`` to every (layer, seq, head) list; returns (tables, next unused index).

    ``tables`` is int32 [L, S, H, max_blocks] on the device of ``block_ids``; unused entries are -1.
    """
    S = context_lens.numel()
    nblk = (context_lens.to(torch.int64) + block_size - 1) // block_size
    max_blocks = int(nblk.max()) if S else 0
    tables = torch.full((num_layers, S, num_kv_heads, max_blocks), -1, dtype=torch.int32, device=block_ids.device)
    off = first
    for s in range(S):
        n = int(nblk[s])
        cnt = num_layers * num_kv_heads * n
        if off + cnt > block_ids.numel():
            raise ValueError("pool too small for this workload")
        tables[:, s, :, :n] = block_ids[off:off + cnt].view(num_layers, num_kv_heads, n).to(torch.int32)
        off += cnt
    return tables, off


def blocks_needed(context_lens: torch.Tensor, num_layers: int, num_kv_heads: int, block_size: int) -> int:
    nblk = (context_lens.to(torch.int64) + block_size - 1) // block_size
    return int(nblk.sum()) * num_layers * num_kv_heads


def last_token_slots(block_tables: torch.Tensor, context_lens: torch.Tensor, block_size: int,
                     new_tokens: int = 1) -> torch.Tensor:
    """Slots of the last ``new_tokens`` positions of every sequence: int64 [S*new_tokens, L, H]
    (token-major within a sequence), slot = block id * block_size + offset (csrc/batch_scheduler.h:58-67)."""
    L, S, H, _ = block_tables.shape
    ctx = context_lens.to(block_tables.device).to(torch.int64)
    out = torch.empty((S, new_tokens, L, H), dtype=torch.int64, device=block_tables.device)
    for j in range(new_tokens):
        pos = ctx - new_tokens + j                                   # [S]
        blk = (pos // block_size).view(1, S, 1, 1).expand(L, S, H, 1)
        ids = torch.gather(block_tables.to(torch.int64), 3, blk).squeeze(3)   # [L, S, H]
        out[:, j] = (ids * block_size + (pos % block_size).view(1, S, 1)).permute(1, 0, 2)
    return out.view(S * new_tokens, L, H)


def prompt_slots(block_tables: torch.Tensor, prompt_lens: torch.Tensor, block_size: int) -> torch.Tensor:
    """Slots of EVERY token of every prompt: int64 [sum(prompt_lens), L, H], prompts back to back — what the
    reference hands to the prompt-phase cache write (getPromptSlots, csrc/batch_scheduler.h:42-56)."""
    L, S, H, _ = block_tables.shape
    dev = block_tables.device
    lens = prompt_lens.to(torch.int64).cpu()
    out = torch.empty((int(lens.sum()), L, H), dtype=torch.int64, device=dev)
    row = 0
    for s in range(S):
        n = int(lens[s])
        pos = torch.arange(n, device=dev)
        ids = block_tables[:, s, :, :(n + block_size - 1) // block_size].to(torch.int64)   # [L, H, nblk]
        blk = ids[:, :, pos // block_size]                                                   # [L, H, n]
        out[row:row + n] = (blk * block_size + (pos % block_size)).permute(2, 0, 1)
        row += n
    return out


def prefill_flops(prompt_lens: Sequence[int], num_q_heads: int) -> int:
    """Useful FLOPs of one causal prompt attention launch: 4 * 128 per (query, visible key) pair and q head."""
    return 4 * HEAD_SIZE * num_q_heads * int(sum(int(n) * (int(n) + 1) // 2 for n in prompt_lens))


def make_decode_case(shape: ModelShape, context_lens: torch.Tensor, *, block_size: int, num_blocks: int,
                     dtype: torch.dtype, device, seed: int, block_ids: Optional[torch.Tensor] = None,
                     first_block: int = 0, input_layers: Optional[int] = None, new_tokens: int = 1,
                     scale: Optional[float] = None) -> DecodeCase:
    """Builds block tables, slots and N(0,1) q/k/v for one decode step.

    ``block_ids``: a permutation of the pool shared by colocated models (so that
    their lists interleave and never overlap); by default a fresh seeded one.
    ``input_layers``: how many distinct per-layer q/k/v inputs to keep (they are
    cycled over the layers; the KV blocks are always distinct per layer).
    """
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    if block_ids is None:
        block_ids = torch.randperm(num_blocks, generator=gen).to(device)
    tables, nxt = scatter_block_tables(context_lens, shape.num_layers, shape.num_kv_heads, block_size,
                                       block_ids, first_block)
    slots = last_token_slots(tables, context_lens, block_size, new_tokens)
    Lq = shape.num_layers if input_layers is None else max(1, min(input_layers, shape.num_layers))
    S, T = shape.batch, shape.batch * new_tokens
    q = torch.randn((Lq, S, shape.num_q_heads, HEAD_SIZE), generator=gen, dtype=torch.float32).to(dtype).to(device)
    k = torch.randn((Lq, T, shape.num_kv_heads, HEAD_SIZE), generator=gen, dtype=torch.float32).to(dtype).to(device)
    v = torch.randn((Lq, T, shape.num_kv_heads, HEAD_SIZE), generator=gen, dtype=torch.float32).to(dtype).to(device)
    return DecodeCase(shape=shape, block_size=block_size, dtype=dtype,
                      scale=scale if scale is not None else HEAD_SIZE ** -0.5,
                      context_lens=context_lens.to(device), block_tables=tables, slot_mapping=slots,
                      q=q, k=k, v=v, new_tokens=new_tokens, max_context_len=int(context_lens.max()),
                      seed=seed, extra=dict(next_block=nxt))


def attention_bytes(context_lens: Sequence[int], num_q_heads: int, num_kv_heads: int, block_size: int,
                    elem: int = 2) -> int:
    """Algorithmic bytes of one paged_attention launch: K+V of every (seq, kv head) once,
    q read + out write, block ids, context lengths."""
    total = 0
    for c in context_lens:
        c = int(c)
        total += num_kv_heads * c * 2 * HEAD_SIZE * elem
        total += 2 * num_q_heads * HEAD_SIZE * elem
        total += 4 * num_kv_heads * ((c + block_size - 1) // block_size)
        total += 4
    return total


def cache_write_bytes(num_tokens: int, num_kv_heads: int, elem: int = 2) -> int:
    """Algorithmic bytes of one reshape_and_cache launch: k, v read + written, one int64 slot per row."""
    return 4 * num_tokens * num_kv_heads * HEAD_SIZE * elem + 8 * num_tokens * num_kv_heads


def attention_flops(context_lens: Sequence[int], num_q_heads: int) -> int:
    return 4 * HEAD_SIZE * num_q_heads * int(sum(int(c) for c in context_lens))
