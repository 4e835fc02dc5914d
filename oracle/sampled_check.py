"""Oracle check of a few sampled sequences of a full-size decode launch.  TEST INFRASTRUCTURE ONLY.

The fp32 gather oracle (``attention_oracle``; parity unpinned, see its header) takes minutes on a
whole benchmark launch but well under a second on three or four sequences.  This helper copies just
the KV blocks those sequences name from the device pool into a compact CPU pool, runs the oracle on
them and compares all their heads' output rows; the appended K/V rows are compared bit for bit with
the slots ``csrc/batch_scheduler.h:58-67`` names for them (block id * block_size + offset).
Used by the GPU tests at benchmark sizes and by ``bench.py`` AFTER its timed regions, as the checker.
"""
from __future__ import annotations

from typing import Sequence

import torch

from .attention_oracle import paged_attention_ref_batched

ATOL, RTOL = 2e-3, 1e-2      # |out - ref| <= ATOL + RTOL * |ref|, fp16 and bf16


def pick_sequences(context_lens: Sequence[int], count: int = 3, seed: int = 0):
    """Shortest, longest and seeded random others."""
    n = len(context_lens)
    order = sorted(range(n), key=lambda i: int(context_lens[i]))
    picks = [order[0], order[-1]]
    gen = torch.Generator().manual_seed(seed)
    for i in torch.randperm(n, generator=gen).tolist():
        if len(picks) >= min(count, n):
            break
        if i not in picks:
            picks.append(i)
    return sorted(set(picks))


def check_decode_rows(out: torch.Tensor, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                      key_cache: torch.Tensor, value_cache: torch.Tensor, block_tables: torch.Tensor,
                      context_lens: torch.Tensor, scale: float, block_size: int, seqs: Sequence[int],
                      new_tokens: int = 1) -> dict:
    """``out``/``q`` [S, Hq, D], ``k_new``/``v_new`` [S * new_tokens, H, D] (None: no append to check),
    ``block_tables`` [S, H, max_blocks] and ``context_lens`` [S] of ONE layer, pool tensors on the device.
    Returns ``{rows, max_abs_err, ok, pool_bit_exact}``."""
    seqs = [int(s) for s in seqs]
    H = block_tables.shape[1]
    ctx = context_lens[seqs].cpu().to(torch.int64)
    nblk = (ctx + block_size - 1) // block_size
    max_nb = int(nblk.max())
    bt = block_tables[seqs][:, :, :max_nb].to(torch.int64)                   # [n, H, max_nb] device
    valid = (torch.arange(max_nb).view(1, 1, -1) < nblk.view(-1, 1, 1)).expand(len(seqs), H, max_nb)
    ids = bt.cpu()[valid]                                                    # pool ids, in (seq, head, block) order
    compact = torch.zeros((len(seqs), H, max_nb), dtype=torch.int32)
    compact[valid] = torch.arange(ids.numel(), dtype=torch.int32)
    dev_ids = ids.to(key_cache.device)
    kc = key_cache[dev_ids].cpu()
    vc = value_cache[dev_ids].cpu()
    ref = paged_attention_ref_batched(q[seqs].cpu(), kc, vc, scale, compact, ctx.to(torch.int32), block_size)
    got = out[seqs].float().cpu()
    err = (got - ref).abs()
    ok = bool((err <= ATOL + RTOL * ref.abs()).all()) and not bool(torch.isnan(got).any())
    pool_ok = None
    if k_new is not None:
        pool_ok = True
        T = new_tokens
        for i, s in enumerate(seqs):
            for j in range(T):
                pos = int(ctx[i]) - T + j
                blocks = compact[i, :, pos // block_size].long()                 # [H] compact ids
                off = pos % block_size
                krow = kc[blocks][:, :, off, :].reshape(H, -1)
                vrow = vc[blocks][:, :, off]
                want_k = k_new[s * T + j].cpu().reshape(H, -1)
                want_v = v_new[s * T + j].cpu().reshape(H, -1)
                same = torch.equal(krow.view(torch.int16), want_k.view(torch.int16)) and \
                    torch.equal(vrow.view(torch.int16), want_v.view(torch.int16))
                pool_ok = pool_ok and same
    return {"rows": len(seqs) * q.shape[1], "sequences": seqs, "max_abs_err": float(err.max()), "ok": ok,
            "pool_bit_exact": pool_ok, "tolerance": f"{ATOL} + {RTOL} * |ref|"}
