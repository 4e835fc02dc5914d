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
