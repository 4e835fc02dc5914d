"""One fused launch over several colocated models == per-model launches == fp32 oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,psize", [(torch.float16, 0), (torch.bfloat16, 64)])
def test_mixed_launch_matches_per_model_and_oracle(built_lib, dtype, psize):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util as gu
    from muxserve_b200 import mixed, ops
    from oracle.attention_oracle import paged_attention_ref
    from test_mixed_plan import make_batches
    batches, num_blocks, gen = make_batches(device="cuda", seed=9)
    kc = torch.randn(num_blocks, 16, 16, 8, generator=gen).to(dtype).cuda()
    vc = torch.randn(num_blocks, 128, 16, generator=gen).to(dtype).cuda()
    plan = mixed.build_mixed_plan(batches, "cuda")
    qs = [torch.randn(b.num_seqs, b.num_q_heads, 128, generator=gen).to(dtype).cuda() for b in batches]
    packed = mixed.pack_rows(plan, qs)
    for layer in (0, 2, 5):
        n_items, n_rows = plan.active(layer)
        out = torch.full_like(packed, float("nan"))
        ops.paged_attention_mixed(out[:n_rows], packed[:n_rows], kc, vc, plan.block_tables[layer, :n_items],
                                  plan.item_context_len[:n_items], plan.item_q_row[:n_items],
                                  plan.item_group[:n_items], plan.item_scale[:n_items], 16, plan.max_context_len,
                                  plan.max_group, partition_size=psize)
        assert torch.isnan(out[n_rows:]).all()               # rows of models without this layer are untouched
        per_model = mixed.unpack_rows(plan, out, batches)
        for b, q, got in zip(batches, qs, per_model):
            if b.num_layers <= layer:
                continue
            single = torch.empty_like(q)
            ops.paged_attention(single, q, kc, vc, None, b.scale, b.block_tables[layer], b.context_lens.cuda(), 16,
                                int(b.context_lens.max()), partition_size=psize)
            assert torch.equal(got, single), f"{b.name} layer {layer}: fused and single-model launches differ"
            ref = paged_attention_ref(q.cpu(), kc.cpu(), vc.cpu(), None, b.scale, b.block_tables[layer].cpu(),
                                      b.context_lens, 16)
            gu.assert_close(got, ref, f"{b.name} layer {layer}")
    assert ops.device_status() == 0


def test_mixed_fused_decode_step(built_lib):
    """The mixed launch with new rows appended in the same kernel == per-model cache writes + mixed attention."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from muxserve_b200 import mixed, ops, workloads
    from test_mixed_plan import make_batches
    batches, num_blocks, gen = make_batches(device="cuda", seed=21)
    dtype = torch.float16
    kc = torch.randn(num_blocks, 16, 16, 8, generator=gen).to(dtype).cuda()
    vc = torch.randn(num_blocks, 128, 16, generator=gen).to(dtype).cuda()
    kc2, vc2 = kc.clone(), vc.clone()
    plan = mixed.build_mixed_plan(batches, "cuda")
    qs = [torch.randn(b.num_seqs, b.num_q_heads, 128, generator=gen).to(dtype).cuda() for b in batches]
    ks = [torch.randn(b.num_seqs, b.num_kv_heads, 128, generator=gen).to(dtype).cuda() for b in batches]
    vs = [torch.randn(b.num_seqs, b.num_kv_heads, 128, generator=gen).to(dtype).cuda() for b in batches]
    packed = mixed.pack_rows(plan, qs)
    k_items, v_items = mixed.pack_rows(plan, ks), mixed.pack_rows(plan, vs)
    layer = 1
    n_items, n_rows = plan.active(layer)
    # two-op path
    for b, k, v in zip(batches, ks, vs):
        if b.num_layers > layer:
            slots = workloads.last_token_slots(b.block_tables, b.context_lens, 16)[:, layer, :]
            ops.reshape_and_cache(k, v, kc, vc, slots)
    expect = torch.zeros_like(packed)
    args = (plan.block_tables[layer, :n_items], plan.item_context_len[:n_items], plan.item_q_row[:n_items],
            plan.item_group[:n_items], plan.item_scale[:n_items], 16, plan.max_context_len, plan.max_group)
    ops.paged_attention_mixed(expect[:n_rows], packed[:n_rows], kc, vc, *args)
    got = torch.zeros_like(packed)
    ops.paged_attention_mixed(got[:n_rows], packed[:n_rows], kc2, vc2, *args, new_k=k_items[:n_items],
                              new_v=v_items[:n_items])
    assert torch.equal(kc2, kc) and torch.equal(vc2, vc)
    assert torch.equal(got, expect)
    assert ops.device_status() == 0


@pytest.mark.parametrize("psize", [64, 128, 512])
def test_mixed_launch_with_work_list_is_bit_identical(built_lib, psize):
    """The host's list of real (item, partition) pairs changes which CTAs exist, not what they compute."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from muxserve_b200 import mixed, ops
    from test_mixed_plan import make_batches
    batches, num_blocks, gen = make_batches(device="cuda", seed=33)
    dtype = torch.float16
    kc = torch.randn(num_blocks, 16, 16, 8, generator=gen).to(dtype).cuda()
    vc = torch.randn(num_blocks, 128, 16, generator=gen).to(dtype).cuda()
    plan = mixed.build_mixed_plan(batches, "cuda")
    qs = [torch.randn(b.num_seqs, b.num_q_heads, 128, generator=gen).to(dtype).cuda() for b in batches]
    ks = [torch.randn(b.num_seqs, b.num_kv_heads, 128, generator=gen).to(dtype).cuda() for b in batches]
    packed, k_items = mixed.pack_rows(plan, qs), mixed.pack_rows(plan, ks)
    for layer in (0, 3):
        n_items, n_rows = plan.active(layer)
        units = plan.units(layer, psize)
        ctx = plan.item_context_len[:n_items].cpu()
        assert units.shape[0] == int(((ctx + psize - 1) // psize).sum())
        args = (plan.block_tables[layer, :n_items], plan.item_context_len[:n_items], plan.item_q_row[:n_items],
                plan.item_group[:n_items], plan.item_scale[:n_items], 16, plan.max_context_len, plan.max_group)
        a, b = torch.zeros_like(packed), torch.zeros_like(packed)
        ops.paged_attention_mixed(a[:n_rows], packed[:n_rows], kc, vc, *args, partition_size=psize)
        ops.paged_attention_mixed(b[:n_rows], packed[:n_rows], kc, vc, *args, partition_size=psize, units=units)
        assert torch.equal(a, b)
        # the whole decode step (new rows appended in the launch) through the list as well
        kc1, vc1, kc2, vc2 = kc.clone(), vc.clone(), kc.clone(), vc.clone()
        ops.paged_attention_mixed(a[:n_rows], packed[:n_rows], kc1, vc1, *args, partition_size=psize,
                                  new_k=k_items[:n_items], new_v=k_items[:n_items])
        ops.paged_attention_mixed(b[:n_rows], packed[:n_rows], kc2, vc2, *args, partition_size=psize, units=units,
                                  new_k=k_items[:n_items], new_v=k_items[:n_items])
        assert torch.equal(a, b) and torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert ops.device_status() == 0
