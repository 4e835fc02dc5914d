"""Descriptors of the fused multi-model launch (CPU): every item names the right rows, lengths and lists."""
import torch

from muxserve_b200 import mixed, workloads
from oracle.attention_oracle import paged_attention_items_ref, paged_attention_ref


def make_batches(device="cpu", seed=0):
    gen = torch.Generator().manual_seed(seed)
    num_blocks = 4096
    perm = torch.randperm(num_blocks, generator=gen)
    specs = [("llm-7b", 3, 8, 8, 5), ("llm-30b", 6, 13, 13, 3), ("llm-13b", 4, 10, 10, 4), ("gqa", 2, 8, 2, 3)]
    batches, nxt = [], 0
    for name, L, Hq, H, S in specs:
        ctx = workloads.lognormal_context_lens(S, 40, 1.0, 1, 300, gen)
        bt, nxt = workloads.scatter_block_tables(ctx, L, H, 16, perm, nxt)
        batches.append(mixed.ModelBatch(name, L, Hq, H, 128 ** -0.5 * (1.0 + 0.1 * len(batches)), ctx, bt.to(device)))
    return batches, num_blocks, gen


def test_plan_prefix_structure_and_descriptors():
    batches, _, _ = make_batches()
    plan = mixed.build_mixed_plan(batches, "cpu")
    assert [batches[i].name for i in plan.order] == ["llm-30b", "llm-13b", "llm-7b", "gqa"]
    assert plan.layers == [6, 4, 3, 2] and plan.max_group == 4
    assert plan.item_offset == [0, 39, 79, 119, 125] and plan.row_offset == [0, 39, 79, 119, 143]
    assert plan.active(0) == (125, 143) and plan.active(2) == (119, 119) and plan.active(3) == (79, 79)
    assert plan.active(4) == (39, 39) and plan.active(5) == (39, 39)
    # the gqa model: item (s, h) starts at row base + s*8 + h*4 and has 4 rows
    base = plan.row_offset[3]
    assert plan.item_q_row[plan.item_offset[3]:].tolist() == [base + s * 8 + h * 4 for s in range(3) for h in range(2)]
    assert plan.item_group[plan.item_offset[3]:].tolist() == [4] * 6
    b = batches[1]                                           # llm-30b is first in the plan
    assert plan.item_context_len[:39].tolist() == [int(c) for c in b.context_lens for _ in range(13)]
    assert torch.equal(plan.block_tables[5, :39, :b.block_tables.shape[-1]],
                       b.block_tables[5].reshape(39, -1).clamp_min(0))


def test_item_form_equals_per_model_oracle():
    batches, num_blocks, gen = make_batches(seed=3)
    kc = torch.randn(num_blocks, 16, 16, 8, generator=gen)
    vc = torch.randn(num_blocks, 128, 16, generator=gen)
    plan = mixed.build_mixed_plan(batches, "cpu")
    qs = [torch.randn(b.num_seqs, b.num_q_heads, 128, generator=gen) for b in batches]
    packed = mixed.pack_rows(plan, qs)
    layer = 1
    n_items, n_rows = plan.active(layer)
    out = paged_attention_items_ref(packed[:n_rows], kc, vc, plan.block_tables[layer, :n_items],
                                    plan.item_context_len[:n_items], plan.item_q_row[:n_items],
                                    plan.item_group[:n_items], plan.item_scale[:n_items], 16)
    full = torch.zeros(packed.shape)
    full[:n_rows] = out
    per_model = mixed.unpack_rows(plan, full, batches)
    for b, q, got in zip(batches, qs, per_model):
        ref = paged_attention_ref(q, kc, vc, None, b.scale, b.block_tables[layer], b.context_lens, 16)
        assert torch.allclose(got, ref, atol=1e-5, rtol=1e-5), b.name


def _serve_models(tp=1):
    """Three models with their own step builders over ONE allocator, one prefill and a few decode steps each."""
    import numpy as np
    from muxserve_b200.batch_scheduler import BatchScheduler
    from muxserve_b200.memory_manager import KVStorage
    B, max_seq = 16, 256
    kv = KVStorage(8192)
    specs = [("a", 3, 8, 8, [5, 40, 17]), ("deep", 6, 4, 2, [33, 16]), ("mid", 4, 5, 5, [100, 1, 64, 15])]
    models, rid = [], 100
    for name, L, Hq, H, prompts in specs:
        sched = BatchScheduler(L, H, max_seq, B)
        ids = list(range(rid, rid + len(prompts)))
        rid += 50                                            # request ids are global across colocated models
        for r, n in zip(ids, prompts):
            sched.add_request(np.arange(n, dtype=np.int32), r, 32)
        info = sched.try_batch(ids, [])
        blocks = kv.allocate_batch(info[:-1], L, H)
        sched.get_batch_info(info[:-1], blocks)
        models.append(dict(name=name, L=L, Hq=Hq, H=H, sched=sched, ids=ids, scale=0.05 + 0.01 * len(models)))
    return kv, models, B, max_seq


def test_host_library_emits_the_same_mixed_descriptors():
    """mux_batch_scheduler_get_batch_mixed (C++) == build_mixed_plan over the tensors each model's
    get_batch_decode_layered fills, step after step, also in the tensor-parallel row layout."""
    import numpy as np
    kv, models, B, max_seq = _serve_models()
    max_blocks = max_seq // B
    for step in range(20):
        batches = []
        for m in models:
            info = m["sched"].try_batch(m["ids"], [step] * len(m["ids"]))
            blocks = kv.allocate_batch(info[:-1], m["L"], m["H"]) if info[-1] > 0 else np.array([len(m["ids"])], np.int32)
            assert blocks[0] == len(m["ids"])
            ntok, nctx, maxctx, maxblk = m["sched"].get_batch_info(info[:-1], blocks)[:4]
            S = len(m["ids"])
            tok, pos = torch.empty(8, dtype=torch.int32), torch.empty(8, dtype=torch.int32)
            ctx = torch.empty(S, dtype=torch.int32)
            bt = torch.empty((m["L"], S, m["H"], maxblk), dtype=torch.int32)
            slots = torch.empty((S, m["L"], m["H"]), dtype=torch.int64)
            m["sched"].get_batch_decode_layered(info[:-1], blocks, tok, pos, ctx, bt, slots)
            batches.append(mixed.ModelBatch(m["name"], m["L"], m["Hq"], m["H"], m["scale"], ctx, bt))
        for tp, rank in ((1, 0), (4, 2)):
            want = mixed.build_mixed_plan(batches, "cpu", tp=tp, tp_rank=rank)
            got = mixed.plan_from_schedulers([(m["sched"], m["ids"], m["Hq"], m["scale"]) for m in models], "cpu",
                                             max_blocks, tp=tp, tp_rank=rank)
            assert got.order == want.order == [1, 2, 0] and got.layers == want.layers
            assert got.item_offset == want.item_offset and got.row_offset == want.row_offset
            assert got.max_group == want.max_group and got.max_context_len == want.max_context_len
            for name in ("item_context_len", "item_q_row", "item_group", "item_scale"):
                assert torch.equal(getattr(got, name), getattr(want, name)), name
            mb = want.block_tables.shape[-1]
            assert torch.equal(got.block_tables[:, :, :mb], want.block_tables)
            assert int(got.block_tables[:, :, mb:].abs().sum()) == 0
    assert kv.check_invariants()


def test_get_batch_mixed_rejects_bad_input():
    import ctypes as C
    import numpy as np
    from muxserve_b200 import _lib
    kv, models, B, max_seq = _serve_models()
    m = models[0]
    spans, totals = (_lib.MixedSpan * 1)(), np.zeros(5, dtype=np.int32)
    ids = np.asarray(m["ids"], dtype=np.int32)
    call = lambda mm, n=1, tp=1, rank=0, mb=16: _lib.lib().mux_batch_scheduler_get_batch_mixed(
        mm, n, tp, rank, mb, None, None, None, None, None, 0, spans, _lib.i32p(totals))
    arr = (_lib.MixedModel * 1)(_lib.MixedModel(m["sched"]._h, _lib.i32p(ids), ids.size, m["Hq"], 0.1))
    assert call(arr) == -6                                   # the requests are still prompts: decode rows only
    info = m["sched"].try_batch(m["ids"], [7] * len(ids))
    blocks = kv.allocate_batch(info[:-1], m["L"], m["H"]) if info[-1] > 0 else np.array([len(ids)], np.int32)
    m["sched"].get_batch_info(info[:-1], blocks)
    assert call(arr) == 0 and totals[:4].tolist() == [3 * 8, 3 * 8, 3, 1]
    assert call(arr, tp=2, rank=2) == -6 and call(arr, mb=1) == -11
    arr[0].num_q_heads = 12
    assert call(arr) == -7                                   # not a multiple of the kv heads
    arr[0].num_q_heads = 8
    bad = np.asarray([999], dtype=np.int32)
    arr[0].request_ids, arr[0].num_requests = _lib.i32p(bad), 1
    assert call(arr) == -12
