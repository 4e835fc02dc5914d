"""Tensor-parallel plumbing on CPU ranks (gloo, world_size 2): sharding by kv head needs no exchange
inside attention, and the all-reduce of the row-parallel projection reproduces the single-rank result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from muxserve_b200 import parallel


def test_shard_heads_layouts():
    s = parallel.shard_heads(64, 8, 4, 3)
    assert (s.q_start, s.q_count, s.kv_start, s.kv_count, s.kv_replicas) == (48, 16, 6, 2, 1)
    s = parallel.shard_heads(64, 8, 8, 5)
    assert (s.q_start, s.q_count, s.kv_start, s.kv_count) == (40, 8, 5, 1)
    s = parallel.shard_heads(32, 2, 8, 5)              # fewer kv heads than ranks: replicated (llama.py:109-114)
    assert (s.q_start, s.q_count, s.kv_start, s.kv_count, s.kv_replicas) == (20, 4, 1, 1, 4)
    with pytest.raises(ValueError):
        parallel.shard_heads(52, 52, 8, 0)             # LLaMA-30B does not divide over 8 ranks


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from muxserve_b200 import workloads
        from oracle.attention_oracle import paged_attention_ref
        gen = torch.Generator().manual_seed(11)                      # identical inputs on every rank
        Hq, H, S, L, B, nb, hidden = 8, 4, 5, 2, 16, 512, 64
        ctx = workloads.uniform_context_lens(S, 1, 90, gen)
        case = workloads.make_decode_case(workloads.ModelShape("tp", L, Hq, H, S), ctx, block_size=B, num_blocks=nb,
                                          dtype=torch.float32, device="cpu", seed=5)
        kc = torch.randn(nb, 32, B, 4, generator=gen)                # fp32 pool: x = 16 bytes / 4
        vc = torch.randn(nb, 128, B, generator=gen)
        w_o = torch.randn(Hq * 128, hidden, generator=gen) / 32
        shard = parallel.shard_heads(Hq, H, world, rank)
        bt, slots = parallel.shard_index_tensors(shard, case.block_tables, case.slot_mapping)
        assert bt.shape[2] == H // world and slots.shape[2] == H // world
        layer = 1
        q, k, v = parallel.shard_qkv(shard, case.q[layer], case.k[layer], case.v[layer])
        local = paged_attention_ref(q, kc, vc, None, case.scale, bt[layer], ctx, B)          # no communication
        rows = slice(shard.q_start * 128, (shard.q_start + shard.q_count) * 128)
        partial = local.reshape(S, -1) @ w_o[rows]
        total = parallel.all_reduce_output(partial.clone())
        full = paged_attention_ref(case.q[layer], kc, vc, None, case.scale, case.block_tables[layer], ctx, B)
        expect = full.reshape(S, -1) @ w_o
        slow = parallel.max_over_ranks(float(rank + 1))
        q_out.put((rank, bool(torch.allclose(total, expect, atol=1e-4, rtol=1e-4)),
                   bool(torch.equal(local, full[:, shard.q_start:shard.q_start + shard.q_count])), slow))
    finally:
        dist.destroy_process_group()


def test_tp2_gloo_allreduce_matches_single_rank():
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q_out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, True, True, 2.0), (1, True, True, 2.0)]


def _grant_worker(rank, world, port, q_out):
    """Rank 0 runs the allocator and the step builder for ALL heads; every rank receives the few-KB grant and keeps
    its own heads' columns in its persistent table, which must equal its slice of the rebuilt full table."""
    import numpy as np
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from muxserve_b200.batch_scheduler import BatchScheduler
        from muxserve_b200.device_tables import DeviceBlockTables
        from muxserve_b200.memory_manager import KVStorage
        L, H, B, max_seq = 3, 4, 16, 128
        shard = parallel.shard_heads(H, H, world, rank)
        dbt = DeviceBlockTables(L, shard.kv_count, max_rows=4, max_blocks=max_seq // B, device="cpu",
                                total_kv_heads=H, kv_head_start=shard.kv_start)
        ids = [7, 8, 9]
        if rank == 0:
            kv, sched = KVStorage(1024), BatchScheduler(L, H, max_seq, B)
            for r, n in zip(ids, [5, 16, 31]):
                sched.add_request(np.arange(n, dtype=np.int32), r, 64)
        ok, sent = True, 0
        for step in range(24):
            req = info = None
            if rank == 0:
                req = sched.try_batch(ids, [] if step == 0 else [step] * len(ids))
                info = kv.allocate_batch(req[:-1], L, H) if req[-1] > 0 else np.array([len(ids)], dtype=np.int32)
                req = req[:-1]
            req, info = parallel.broadcast_grant(req, info, src=0)
            sent += req.nbytes + info.nbytes
            dbt.stage_grant(req, info)
            for row, blk, block_ids in zip(dbt._rows, dbt._blks, np.concatenate(dbt._ids) if dbt._ids else []):
                dbt.tables[:, row, :, blk] = torch.from_numpy(block_ids.reshape(L, shard.kv_count))   # what flush scatters
            dbt._rows, dbt._blks, dbt._ids = [], [], []
            full = None
            if rank == 0:
                ntok, nctx, maxctx, maxblk = sched.get_batch_info(req, info)[:4]
                if step > 0:
                    S = len(ids)
                    tok, pos, ctx = torch.empty(8, dtype=torch.int32), torch.empty(8, dtype=torch.int32), torch.empty(S, dtype=torch.int32)
                    full = torch.zeros((L, S, H, max_seq // B), dtype=torch.int32)
                    view = torch.empty((L, S, H, maxblk), dtype=torch.int32)
                    sched.get_batch_decode_layered(req, info, tok, pos, ctx, view, torch.empty((S, L, H), dtype=torch.int64))
                    full[..., :maxblk] = view
            box = [full]
            dist.broadcast_object_list(box, src=0)                  # the check's reference only
            if box[0] is not None:
                rows = torch.tensor([dbt.row_of[r] for r in ids])
                mine = dbt.tables[:, rows]
                want = box[0][:, :, shard.kv_start:shard.kv_start + shard.kv_count]
                nb = [dbt.blocks_of[r] for r in ids]
                for s, n in enumerate(nb):
                    ok = ok and torch.equal(mine[:, s, :, :n], want[:, s, :, :n])
        q_out.put((rank, bool(ok), sent < 24 * 3 * L * H * (max_seq // B) * 4))
    finally:
        dist.destroy_process_group()


def test_tp2_grant_broadcast_keeps_each_ranks_heads():
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_grant_worker, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q_out.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert results == [(0, True, True), (1, True, True)]
