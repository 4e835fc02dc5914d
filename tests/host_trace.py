"""Drives an allocator + step builder pair through a seeded serving trace.

Works with any implementation that has the reference's method names: the compiled
reference, the Python restatement in ``oracle/host_oracle.py`` and this
repository's C++ (``muxserve_b200.memory_manager`` / ``batch_scheduler``).  The
loop follows ``LLMRuntime.prepare_inputs`` (muxserve/flexserver/llm_runtime.py:277-339).
Every record holds only defined values: block-table entries past a request's
blocks (uninitialised in the reference) are masked to -1.
"""
from __future__ import annotations

import numpy as np
import torch


def _prepare(kv, sched, ids, last, L, H, B):
    info = np.asarray(sched.try_batch(list(ids), list(last)), dtype=np.int32)
    total, req = int(info[-1]), info[:-1]
    if total > 0:
        block_info = np.asarray(kv.allocate_batch(req, L, H), dtype=np.int32)
    else:
        block_info = np.array([len(ids)], dtype=np.int32)
    binfo = list(sched.get_batch_info(req, block_info))
    ntok, nctx, maxctx, maxblk = binfo[0], binfo[1], binfo[2], binfo[3]
    padded = (ntok + 7) // 8 * 8
    slot = torch.empty((ntok, L, H), dtype=torch.int64)
    if maxctx > 0:
        bt = torch.empty((ntok, maxblk, L, H), dtype=torch.int32)
    else:
        bt = torch.empty((0, maxblk, 0, 0), dtype=torch.int32)
    tokens = torch.empty((padded,), dtype=torch.int32)
    positions = torch.empty((padded,), dtype=torch.int32)
    ctx = torch.empty((nctx,), dtype=torch.int32)
    sched.get_batch(req, block_info, tokens, positions, ctx, bt, slot)
    bt = bt.clone()
    if maxctx > 0:
        for i in range(nctx):
            nblk = (int(ctx[i]) + B - 1) // B
            bt[i, nblk:] = -1
    rec = dict(
        try_batch=info.tolist(), block_info=block_info.tolist(),
        new_blocks=int(kv.get_new_blocks_allocated()), batch_info=[int(x) for x in binfo],
        tokens=tokens.tolist(), positions=positions.tolist(), context_lens=ctx.tolist(),
        slot_mapping=slot.reshape(-1).tolist(), block_tables=bt.reshape(-1).tolist(),
        preempted=[int(x) for x in sched.get_preempt_requests()],
        prompt_info=[int(x) for x in sched.get_prompt_info()],
        batch_reqs=[[int(a), int(b)] for a, b in sched.get_batch_reqs()],
    )
    return rec


def run_engine_trace(KV, BS, *, seed, num_blocks, L, H, B, max_seq_len, n_requests, steps,
                     max_prompt=24, max_new=12, free_prob=0.15):
    """Returns the list of per-step records of a seeded trace (identical inputs for every implementation)."""
    rng = np.random.RandomState(seed)
    kv, sched = KV(num_blocks), BS(L, H, max_seq_len, B)
    prompts = {}
    waiting = []
    for i in range(n_requests):
        rid = 1000 + i
        plen = int(rng.randint(1, max_prompt + 1))
        prompts[rid] = (rng.randint(0, 32000, size=plen).astype(np.int32), int(rng.randint(1, max_new + 1)))
        waiting.append(rid)
    running, generated = [], {}
    records = []
    for _ in range(steps):
        if not waiting and not running:
            break
        if waiting and (not running or rng.rand() < 0.35):
            k = int(rng.randint(1, min(4, len(waiting)) + 1))
            ids, waiting = waiting[:k], waiting[k:]
            for rid in ids:
                sched.add_request(prompts[rid][0], rid, prompts[rid][1])
                generated[rid] = 0
            last = []
        else:
            ids = list(running)
            rng.shuffle(ids)
            last = rng.randint(0, 32000, size=len(ids)).tolist()
        rec = _prepare(kv, sched, ids, last, L, H, B)
        rec["ids"] = [int(x) for x in ids]
        rec["decode"] = bool(last)
        records.append(rec)
        pre = set(rec["preempted"])
        served = [r for r in ids if r not in pre]
        for rid in ids:
            if rid in pre:
                if rid in running:
                    running.remove(rid)
                waiting.append(rid)            # re-queued from scratch, as the engine does
        for rid in served:
            if rid not in running:
                running.append(rid)
            generated[rid] += 1
        done = [r for r in running if generated[r] >= prompts[r][1] or rng.rand() < free_prob]
        if done:
            sched.release_requests(done)
            freed = int(kv.free_batch(done + [999999]))     # an unknown id is ignored
            records.append(dict(freed=freed, done=[int(x) for x in done]))
            running = [r for r in running if r not in done]
    return records


def run_alloc_trace(KV, *, seed, num_blocks, L, H, n_requests, steps, max_logical=4, free_frac=0.45):
    """Allocator alone: random allocate_batch (prefill / decode rows, over-subscription) and free_batch calls."""
    rng = np.random.RandomState(seed)
    kv = KV(num_blocks)
    known, out = [], []
    next_id = 1
    for _ in range(steps):
        r = rng.rand()
        if r < 1.0 - free_frac or not known:
            rows = []
            for _ in range(int(rng.randint(1, 5))):
                if known and rng.rand() < 0.5:
                    rows += [int(known[rng.randint(len(known))]), int(rng.randint(0, 2)), 1]
                elif next_id <= n_requests:
                    rows += [next_id, int(rng.randint(1, max_logical + 1)), 0]
                    next_id += 1
            if not rows:
                continue
            ids = rows[0::3]
            if len(set(ids)) != len(ids):
                continue
            res = np.asarray(kv.allocate_batch(np.array(rows, dtype=np.int32), L, H)).tolist()
            p = res[0]
            for j, rid in enumerate(ids):
                if j < p and rid not in known:
                    known.append(rid)
                if j >= p and rid in known:
                    known.remove(rid)
            out.append(dict(op="alloc", rows=rows, result=res, new=int(kv.get_new_blocks_allocated())))
        else:
            k = int(rng.randint(1, min(3, len(known)) + 1))
            ids = [int(x) for x in rng.choice(known, size=k, replace=False)]
            freed = int(kv.free_batch(ids))
            known = [x for x in known if x not in ids]
            out.append(dict(op="free", ids=ids, freed=freed))
    return out
