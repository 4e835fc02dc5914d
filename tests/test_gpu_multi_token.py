"""Decode steps that append several tokens per sequence in the attention launch itself (one launch per layer):
bit-identical, pool included, to reshape_and_cache of the same rows followed by paged_attention."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(built_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util
    from muxserve_b200 import ops
    return ops, gpu_util


@pytest.mark.parametrize("nt", [2, 8, 16])
@pytest.mark.parametrize("dtype,Hq,H,psize,B", [(torch.bfloat16, 16, 2, 128, 16), (torch.float16, 4, 4, 16, 16),
                                                (torch.float16, 8, 8, 2048, 16), (torch.bfloat16, 8, 1, 64, 32),
                                                (torch.float16, 2, 2, 0, 8)])
def test_fused_multi_token_step_equals_two_ops(env, nt, dtype, Hq, H, psize, B):
    ops, gu = env
    # contexts (counting the new tokens) that put the new rows inside one block, across a block boundary, across a
    # partition boundary, and at the very start of a sequence
    ctx = [nt, nt + 1, 16, 17, 31, 33, 64 + nt // 2, 130, 513, 700, 1000, 2 * nt + 3]
    ctx = [max(c, nt) for c in ctx]
    case, kc, vc = gu.make_case(len(ctx), Hq, H, ctx, B, dtype, seed=nt + H, num_blocks=4096, new_tokens=nt)
    kc2, vc2 = kc.clone(), vc.clone()
    ops.reshape_and_cache(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
    two = torch.empty_like(case.q[0])
    ops.paged_attention(two, case.q[0], kc, vc, None, case.scale, case.block_tables[0], case.context_lens, B,
                        case.max_context_len, partition_size=psize)
    one = torch.full_like(case.q[0], float("nan"))
    units = None if psize == 0 else ops.work_units(ctx, psize, "cuda", num_kv_heads=H)
    ops.decode_attention(one, case.q[0], case.k[0], case.v[0], kc2, vc2, None, case.scale, case.block_tables[0],
                         case.context_lens, B, case.max_context_len, partition_size=psize, units=units, early_kv=True)
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2), "the pool differs from the separate cache write"
    assert torch.equal(one, two)
    _, _, ref = gu.oracle_step(case, kc2, vc2)           # idempotent: the rows are already there
    gu.assert_close(one, ref, f"{nt} new tokens")
    assert ops.device_status() == 0


def test_fused_multi_token_with_rotary_and_mixed_form(env):
    ops, gu = env
    from muxserve_b200 import _lib
    nt, B, Hq, H = 4, 16, 8, 4
    ctx = [4, 19, 130, 513]
    case, kc, vc = gu.make_case(len(ctx), Hq, H, ctx, B, torch.float16, seed=2, num_blocks=1024, new_tokens=nt)
    cache = ops.make_cos_sin_cache(1024, dtype=torch.float16, device="cuda")
    S = len(ctx)
    # separate ops: rotate q at ctx - 1, every new key at its own position, then write and attend
    q, k = case.q[0].clone(), case.k[0].clone()
    lens = case.context_lens.long()
    ops.rotary_embedding(lens - 1, q, None, cache)
    kpos = (lens.view(S, 1) - nt + torch.arange(nt, device="cuda").view(1, nt)).reshape(-1)
    ops.rotary_embedding(kpos, None, k, cache)
    kc2, vc2 = kc.clone(), vc.clone()
    ops.reshape_and_cache(k, case.v[0], kc, vc, case.slot_mapping[:, 0, :])
    want = torch.empty_like(q)
    ops.paged_attention(want, q, kc, vc, None, case.scale, case.block_tables[0], case.context_lens, B,
                        case.max_context_len, partition_size=64)
    got = torch.empty_like(q)
    ops.decode_attention(got, case.q[0], case.k[0], case.v[0], kc2, vc2, None, case.scale, case.block_tables[0],
                         case.context_lens, B, case.max_context_len, partition_size=64, cos_sin_cache=cache)
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2) and torch.equal(got, want)
    # mixed form: items = (sequence, kv head), rows of an item's new tokens consecutive
    kc3, vc3 = gu.make_case(len(ctx), Hq, H, ctx, B, torch.float16, seed=2, num_blocks=1024, new_tokens=nt)[1:]
    G = Hq // H
    n = S * H
    bt = case.block_tables[0].reshape(n, -1).contiguous()
    item_ctx = case.context_lens.repeat_interleave(H)
    row = torch.arange(0, n * G, G, dtype=torch.int32, device="cuda")
    grp = torch.full((n,), G, dtype=torch.int32, device="cuda")
    scl = torch.full((n,), case.scale, dtype=torch.float32, device="cuda")
    new_k = case.k[0].view(S, nt, H, 128).permute(0, 2, 1, 3).reshape(n * nt, 128).contiguous()
    new_v = case.v[0].view(S, nt, H, 128).permute(0, 2, 1, 3).reshape(n * nt, 128).contiguous()
    out = torch.empty((n * G, 128), dtype=torch.float16, device="cuda")
    ops.paged_attention_mixed(out, case.q[0].reshape(n * G, 128), kc3, vc3, bt, item_ctx, row, grp, scl, B,
                              case.max_context_len, G, partition_size=64, new_k=new_k, new_v=new_v, cos_sin_cache=cache)
    assert torch.equal(kc3, kc) and torch.equal(vc3, vc) and torch.equal(out.view(S, Hq, 128), want)
    # a context shorter than its new tokens is reported, nothing is written out of range
    bad = case.context_lens.clone()
    bad[0] = 2
    ops.decode_attention(got, case.q[0], case.k[0], case.v[0], kc2, vc2, None, case.scale, case.block_tables[0], bad, B,
                         case.max_context_len, partition_size=64)
    assert ops.device_status() == _lib.MUX_DEV_BAD_CONTEXT
    with pytest.raises(ValueError):
        ops.decode_attention(got, case.q[0], case.k[0][:S * nt - 1], case.v[0][:S * nt - 1], kc2, vc2, None, case.scale,
                             case.block_tables[0], case.context_lens, B, case.max_context_len)
