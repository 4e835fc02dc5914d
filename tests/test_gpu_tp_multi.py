"""The peer-memory all-reduce and the KV-head sharding on REAL ranks: one process per GPU (needs >= 2 GPUs; skipped
otherwise), NVLS off and no multimem anywhere.  Checks: the kernel's sums equal fp32 sums in rank order exactly,
for both algorithms, over a run of calls of different sizes; sharded attention + all-reduce equals the unsharded
launch bit for bit; NCCL's all-reduce agrees within tp roundings."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, results):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from muxserve_b200 import flexstore, ops, parallel, workloads
    from muxserve_b200.tp_comm import TPAllReduce
    comm = TPAllReduce(2 << 20, dev)
    ok = True
    for dt in (torch.bfloat16, torch.float16):
        for count, algo, ctas in ((8, 1, 0), (64 * 4096, 1, 0), (128 * 8192, 2, 0), (1000 * 8, 2, 5), (64 * 4096, 0, 0),
                                  (128 * 8192, 0, 0), (24, 2, 0)):
            g = torch.Generator().manual_seed(1000 * rank + count)
            x = torch.randn((count,), generator=g).to(dt).to(dev)
            parts = [torch.empty_like(x) for _ in range(world)]
            dist.all_gather(parts, x)
            acc = torch.zeros((count,), dtype=torch.float32, device=dev)
            for p_ in parts:
                acc += p_.float()
            y = torch.empty_like(x)
            for _ in range(3):
                comm.all_reduce(x, y, algo=algo, num_ctas=ctas)
            torch.cuda.synchronize()
            ok = ok and torch.equal(y, acc.to(dt))
            z = x.clone()
            dist.all_reduce(z)
            eps = 2.0 ** (-8 if dt == torch.bfloat16 else -11)
            ok = ok and float((z.float() - acc).abs().max()) <= world * eps * float(acc.abs().max()) + 1e-6
    # a model sharded by kv head: same pool and batch on every rank
    S, Hq, H, nb, B = 10, 16, 8, 4096, 16
    gen = torch.Generator().manual_seed(77)
    ctx = workloads.uniform_context_lens(S, 1, 900, gen)
    case = workloads.make_decode_case(workloads.ModelShape("t", 1, Hq, H, S), ctx, block_size=B, num_blocks=nb,
                                      dtype=torch.bfloat16, device=dev, seed=5)
    kc, vc = flexstore.allocate_gpu_cache(nb, B, torch.bfloat16, dev)
    workloads.fill_pool_(kc, vc, 6)
    kc2, vc2 = kc.clone(), vc.clone()
    whole = torch.empty((S, Hq, 128), dtype=torch.bfloat16, device=dev)
    ops.decode_attention(whole, case.q[0], case.k[0], case.v[0], kc, vc, None, case.scale, case.block_tables[0],
                         case.context_lens, B, case.max_context_len, partition_size=128)
    sh = parallel.shard_heads(Hq, H, world, rank)
    q, k, v = parallel.shard_qkv(sh, case.q[0], case.k[0], case.v[0])
    bt, _ = parallel.shard_index_tensors(sh, case.block_tables, case.slot_mapping)
    partial = torch.zeros((S, Hq * 128), dtype=torch.bfloat16, device=dev)
    mine = partial.view(S, Hq, 128)[:, sh.q_start:sh.q_start + sh.q_count]
    ops.decode_attention(mine, q, k, v, kc2, vc2, None, case.scale, bt[0], case.context_lens, B, case.max_context_len,
                         partition_size=128)
    total = torch.empty_like(partial)
    comm.all_reduce(partial, total)
    torch.cuda.synchronize()
    ok = ok and torch.equal(total.view(S, Hq, 128), whole)
    # o_proj fused with the all-reduce: equals the rank-order sum of the ranks' rounded partial products
    from muxserve_b200 import tp_comm
    m, n, k = 96, 1024, 256
    op = tp_comm.TPOProj(m, n, dev)
    for dt in (torch.bfloat16, torch.float16):
        g = torch.Generator().manual_seed(50 + rank)
        a = torch.randn((m, k), generator=g).to(dt).to(dev)
        w = (torch.randn((n, k), generator=g) / 16).to(dt).to(dev)
        out, part = torch.empty((m, n), dtype=dt, device=dev), torch.empty((m, n), dtype=dt, device=dev)
        tp_comm.oproj(a, w, part)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        acc = torch.zeros((m, n), dtype=torch.float32, device=dev)
        for p_ in parts:
            acc += p_.float()
        for algo in (0, 1, 2, 1):
            out.zero_()
            op.forward(a, w, out, algo=algo)
            torch.cuda.synchronize()
            ok = ok and torch.equal(out, acc.to(dt))
    ok = ok and ops.device_status() == 0
    results.put((rank, bool(ok)))
    op.close()
    comm.close()
    dist.barrier()
    dist.destroy_process_group()


def test_peer_allreduce_and_head_sharding_on_real_ranks(built_lib):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    world = min(torch.cuda.device_count(), 8)
    while world & (world - 1):           # 8 kv heads must divide over the ranks
        world -= 1
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(results.get(timeout=150) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
    assert all(p.exitcode == 0 for p in procs)
    assert got == {r: True for r in range(world)}
