"""A small serving loop on the GPU: allocator -> step builder -> persistent device block tables
(incremental updates) -> prefill cache write -> fused decode steps, checked every step against the
full table the step builder produces and against the path that uploads it."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_serving_loop_with_incremental_device_tables(built_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from muxserve_b200 import ops
    from muxserve_b200.batch_scheduler import BatchScheduler
    from muxserve_b200.device_tables import DeviceBlockTables
    from muxserve_b200.memory_manager import KVStorage
    L, H, G, B, nblocks, max_seq = 2, 3, 2, 16, 2048, 256
    dtype = torch.float16
    gen = torch.Generator().manual_seed(3)
    kv, sched = KVStorage(nblocks), BatchScheduler(L, H, max_seq, B)
    dbt = DeviceBlockTables(L, H, max_rows=6, max_blocks=max_seq // B)
    kc = torch.randn(nblocks, 16, B, 8, generator=gen).to(dtype).cuda()
    vc = torch.randn(nblocks, 128, B, generator=gen).to(dtype).cuda()
    kc_ref, vc_ref = kc.clone(), vc.clone()
    rnd = lambda *shape: torch.randn(*shape, generator=gen).to(dtype).cuda()

    def prefill(ids, lens):
        for rid, n in zip(ids, lens):
            sched.add_request(np.arange(n, dtype=np.int32), rid, 64)
        info = sched.try_batch(ids, [])
        blocks = kv.allocate_batch(info[:-1], L, H)
        assert blocks[0] == len(ids)
        dbt.stage_grant(info[:-1], blocks)
        ntok = sched.get_batch_info(info[:-1], blocks)[0]
        pad = (ntok + 7) // 8 * 8
        tok, pos = torch.empty(pad, dtype=torch.int32), torch.empty(pad, dtype=torch.int32)
        slots = torch.empty((ntok, L, H), dtype=torch.int64)
        sched.get_batch(info[:-1], blocks, tok, pos, torch.empty(0, dtype=torch.int32),
                        torch.empty((0, 0, 0, 0), dtype=torch.int32), slots)
        slots = slots.cuda()
        for layer in range(L):                       # prompt K/V of every layer: the prefill-side cache write
            k, v = rnd(ntok, H, 128), rnd(ntok, H, 128)
            for pool_k, pool_v in ((kc, vc), (kc_ref, vc_ref)):
                ops.reshape_and_cache(k, v, pool_k, pool_v, slots[:, layer, :])

    running = [11, 12, 13, 14]
    prefill(running, [5, 16, 31, 40])
    for step in range(40):
        if step == 12:                               # one request finishes, a new one takes its row
            sched.release_requests([12])
            assert kv.free_batch([12]) > 0
            dbt.release([12])
            running.remove(12)
            prefill([21], [17])
            running.append(21)
        info = sched.try_batch(running, [step] * len(running))
        blocks = kv.allocate_batch(info[:-1], L, H) if info[-1] > 0 else np.array([len(running)], dtype=np.int32)
        dbt.stage_grant(info[:-1], blocks)
        ntok, nctx, maxctx, maxblk = sched.get_batch_info(info[:-1], blocks)[:4]
        S = len(running)
        tok, pos = torch.empty(8, dtype=torch.int32), torch.empty(8, dtype=torch.int32)
        ctx = torch.empty(S, dtype=torch.int32)
        full = torch.empty((L, S, H, maxblk), dtype=torch.int32)
        slots = torch.empty((S, L, H), dtype=torch.int64)
        sched.get_batch_decode_layered(info[:-1], blocks, tok, pos, ctx, full, slots)
        dbt.flush()
        rows = dbt.rows_for(running)
        # the incrementally maintained table equals the rebuilt one wherever it is defined
        dev = dbt.tables[:, rows.long()].cpu()
        for s in range(S):
            nb = (int(ctx[s]) + B - 1) // B
            assert torch.equal(dev[:, s, :, :nb], full[:, s, :, :nb]), (step, s)
        ctx_d, full_d = ctx.cuda(), full.cuda()
        for layer in range(L):
            q, k, v = rnd(S, H * G, 128), rnd(S, H, 128), rnd(S, H, 128)
            a, b = torch.empty_like(q), torch.empty_like(q)
            ops.decode_attention(a, q, k, v, kc, vc, None, 0.09, dbt.tables[layer], ctx_d, B, maxctx, seq_rows=rows)
            ops.decode_attention(b, q, k, v, kc_ref, vc_ref, None, 0.09, full_d[layer], ctx_d, B, maxctx)
            assert torch.equal(a, b), (step, layer)
    assert torch.equal(kc, kc_ref) and torch.equal(vc, vc_ref)
    assert kv.check_invariants() and ops.device_status() == 0
    # 40 steps moved a few KB of updates instead of 40 full tables
    assert dbt.uploaded_bytes < 40 * 4 * L * 4 * H * (max_seq // B) / 4
