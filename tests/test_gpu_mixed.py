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
