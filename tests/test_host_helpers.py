"""CPU checks of the host-side helpers around the kernels: workload generators and the row / grant
bookkeeping of the persistent device tables (no GPU: the table itself is a CPU tensor here)."""
import numpy as np
import torch

from muxserve_b200 import workloads
from muxserve_b200.device_tables import DeviceBlockTables


def test_scatter_block_tables_never_shares_a_block():
    gen = torch.Generator().manual_seed(0)
    ctx = workloads.lognormal_context_lens(20, 256, 1.0, 16, 4096, gen)
    assert int(ctx.min()) >= 16 and int(ctx.max()) <= 4096
    need = workloads.blocks_needed(ctx, 3, 5, 16)
    perm = torch.randperm(need + 50, generator=gen)
    bt, nxt = workloads.scatter_block_tables(ctx, 3, 5, 16, perm)
    used = bt[bt >= 0]
    assert used.numel() == need == nxt and used.unique().numel() == need
    for s in range(20):
        nb = (int(ctx[s]) + 15) // 16
        assert (bt[:, s, :, :nb] >= 0).all() and (bt[:, s, :, nb:] == -1).all()
    slots = workloads.last_token_slots(bt, ctx, 16, new_tokens=3)
    assert slots.shape == (60, 3, 5)
    s, j = 7, 2                                           # last of the three new tokens of sequence 7
    pos = int(ctx[s]) - 1
    assert int(slots[s * 3 + j, 1, 4]) == int(bt[1, s, 4, pos // 16]) * 16 + pos % 16


def test_device_tables_bookkeeping():
    t = DeviceBlockTables(num_layers=2, num_kv_heads=3, max_rows=3, max_blocks=4, device="cpu")
    LH = 6
    # prefill grant: request 7 gets 2 blocks, request 9 gets 1; request 5 was preempted by the allocator
    req = np.array([7, 2, 0, 9, 1, 0, 5, 1, 0], dtype=np.int32)
    info = np.concatenate([[2], np.arange(100, 100 + 3 * LH)]).astype(np.int32)
    t.stage_grant(req, info)
    assert t.row_of == {7: 0, 9: 1} and t.blocks_of == {7: 2, 9: 1}
    assert t._rows == [0, 0, 1] and t._blks == [0, 1, 0]
    ids = np.concatenate(t._ids, axis=0)
    assert ids.shape == (3, LH) and ids[1].tolist() == list(range(106, 112)) and ids[2].tolist() == list(range(112, 118))
    # decode step without a boundary crossing stages nothing; one with a crossing appends at the next block
    t._rows, t._blks, t._ids = [], [], []
    t.stage_grant(np.array([7, 0, 1, 9, 1, 1], dtype=np.int32), np.concatenate([[2], np.arange(6)]).astype(np.int32))
    assert t._rows == [1] and t._blks == [1] and t.blocks_of[9] == 2
    # rows are recycled
    t.release([7])
    assert t.assign(11) == 0 and t.blocks_of[11] == 0
    t.assign(12)
    try:
        t.assign(13)
        raise AssertionError("expected the table to be full")
    except RuntimeError:
        pass


def test_work_units_cover_every_partition_once_fullest_first():
    import numpy as np
    from muxserve_b200 import ops
    ctx = [1, 512, 513, 0, 2048, 77]
    H, P = 3, 512
    u = ops.work_units(ctx, P, num_kv_heads=H)
    item, part = u & 0xffffff, (u.view(np.uint32) >> 24).astype(np.int64)
    want = {(s * H + h, p) for s, c in enumerate(ctx) for h in range(H) for p in range(max(1, (c + P - 1) // P))}      # an empty context keeps partition 0 (its CTA writes zeros)
    assert len(u) == len(want) and set(zip(item.tolist(), part.tolist())) == want
    per_item = np.repeat(np.asarray(ctx), H)
    tokens = np.minimum(P, per_item[item] - part * P)
    assert (np.diff(tokens) <= 0).all()                      # fullest partitions first
    assert (u >= 0).all()                                    # negative values are reserved for padding
    import pytest
    with pytest.raises(ValueError):
        ops.work_units(ctx, 0, num_kv_heads=H)


def test_prefill_work_units_group_tiles_of_a_prompt_and_start_with_the_longest():
    from muxserve_b200 import ops
    lens = [130, 0, 1000, 128]
    Hq = 3
    u = ops.prefill_work_units(lens, Hq)
    assert u.shape == (sum((n + 127) // 128 for n in lens) * Hq, 2)
    seqs = u[:, 0].tolist()
    assert seqs[0] == 2 and 1 not in seqs                    # longest prompt first, empty prompt absent
    firsts = [seqs.index(s) for s in (2, 0, 3)]
    assert firsts == sorted(firsts)                          # prompts in order of decreasing length
    triples = {(int(s), int(hq) & 0xffff, int(hq) >> 16) for s, hq in u}
    want = {(s, h, t) for s, n in enumerate(lens) for h in range(Hq) for t in range((n + 127) // 128)}
    assert triples == want
    # within one (prompt, head) the last tile comes first
    rows = [(int(hq) >> 16) for s, hq in u if s == 2 and (int(hq) & 0xffff) == 0]
    assert rows == sorted(rows, reverse=True)


def test_suggest_launch_follows_the_measured_rules(monkeypatch):
    """Partition size and ring depth from host-held context lengths (no GPU: the SM count is faked)."""
    import numpy as np
    import torch
    from muxserve_b200 import ops

    class Props:
        multi_processor_count = 148
    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda d: Props)
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    rng = np.random.default_rng(0)
    big = rng.integers(128, 2049, size=64)                   # 64 sequences x 32 heads: far more units than CTA places
    assert ops.suggest_launch(big, 1, num_kv_heads=32) == (2048, 0)          # no split at all
    assert ops.suggest_launch(big, 1, num_kv_heads=4)[0] == 512              # a TP=8 shard: split to fill the GPU
    small = np.clip(np.exp(rng.normal(np.log(256), 1.0, size=156)), 16, 4096).astype(int)
    assert ops.suggest_launch(small, 1)[0] == 128                            # few short items: many short units
    assert ops.suggest_launch(rng.integers(2048, 8193, size=2048), 8) == (512, 0)    # grouped heads keep 512
    assert ops.suggest_launch([], 1) == (512, 0)
