"""Launch-overlap flag, clamped group sizes and empty contexts in a work list (through the C ABI)."""
import numpy as np
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


@pytest.mark.parametrize("dtype,Hq,H,psize", [(torch.float16, 8, 8, 2048), (torch.bfloat16, 16, 2, 128),
                                              (torch.float16, 4, 4, 64)])
def test_early_kv_decode_steps_are_bit_identical(env, dtype, Hq, H, psize):
    """A run of back-to-back decode launches over distinct layers gives the same outputs and the same pool with
    and without MUX_ATTN_EARLY_KV, with and without a work list; the first launch is also checked against the oracle."""
    ops, gu = env
    from muxserve_b200 import flexstore, workloads
    L, B = 6, 16
    ctx = torch.tensor([1, 15, 16, 17, 130, 700, 64, 1000, 33, 257], dtype=torch.int32)
    shape = workloads.ModelShape("t", L, Hq, H, len(ctx))
    case = workloads.make_decode_case(shape, ctx, block_size=B, num_blocks=8192, dtype=dtype, device="cuda", seed=5)
    kc, vc = flexstore.allocate_gpu_cache(8192, B, dtype, "cuda")
    workloads.fill_pool_(kc, vc, 6)
    units = ops.work_units(ctx.tolist(), psize, "cuda", num_kv_heads=H)
    results = []
    for early, ul in ((False, None), (True, None), (True, units), (False, units)):
        kc_i, vc_i = kc.clone(), vc.clone()
        outs = torch.full((L,) + tuple(case.q[0].shape), float("nan"), dtype=dtype, device="cuda")
        for rep in range(2):              # twice: the second round overwrites the same slots with the same rows
            for l in range(L):
                ops.decode_attention(outs[l], case.q[l], case.k[l], case.v[l], kc_i, vc_i, None, case.scale,
                                     case.block_tables[l], case.context_lens, B, case.max_context_len,
                                     partition_size=psize, units=ul, early_kv=early)
        torch.cuda.synchronize()
        results.append((outs, kc_i, vc_i))
    base = results[0]
    for outs, kc_i, vc_i in results[1:]:
        assert torch.equal(outs, base[0]) and torch.equal(kc_i, base[1]) and torch.equal(vc_i, base[2])
    kc_c, vc_c, ref = gu.oracle_step(case, kc, vc, layer=0)
    gu.assert_close(base[0][0], ref, "early-KV decode step, layer 0")
    assert ops.device_status() == 0


def test_early_kv_mixed_launches_are_bit_identical(env):
    ops, gu = env
    from muxserve_b200 import mixed
    from test_mixed_plan import make_batches
    batches, num_blocks, gen = make_batches(device="cuda", seed=71)
    dtype = torch.float16
    kc = torch.randn(num_blocks, 16, 16, 8, generator=gen).to(dtype).cuda()
    vc = torch.randn(num_blocks, 128, 16, generator=gen).to(dtype).cuda()
    plan = mixed.build_mixed_plan(batches, "cuda")
    qs = [torch.randn(b.num_seqs, b.num_q_heads, 128, generator=gen).to(dtype).cuda() for b in batches]
    ks = [torch.randn(b.num_seqs, b.num_kv_heads, 128, generator=gen).to(dtype).cuda() for b in batches]
    packed, k_items = mixed.pack_rows(plan, qs), mixed.pack_rows(plan, ks)
    L_max = max(plan.layers)
    res = []
    for early in (False, True):
        kc_i, vc_i = kc.clone(), vc.clone()
        outs = torch.zeros((L_max,) + tuple(packed.shape), dtype=dtype, device="cuda")
        for l in range(L_max):
            n_items, n_rows = plan.active(l)
            ops.paged_attention_mixed(outs[l, :n_rows], packed[:n_rows], kc_i, vc_i, plan.block_tables[l, :n_items],
                                      plan.item_context_len[:n_items], plan.item_q_row[:n_items],
                                      plan.item_group[:n_items], plan.item_scale[:n_items], 16, plan.max_context_len,
                                      plan.max_group, partition_size=64, units=plan.units(l, 64),
                                      new_k=k_items[:n_items], new_v=k_items[:n_items], early_kv=early)
        torch.cuda.synchronize()
        res.append((outs, kc_i, vc_i))
    for other in res[1:]:
        for a, b in zip(res[0], other):
            assert torch.equal(a, b)
    assert ops.device_status() == 0


def test_group_read_from_device_data_never_widens_the_tile(env):
    """A head_mapping that gives a kv head more q heads than the group, and an item_group above max_group, come back
    as status bits; the launch computes at most the tile it was sized for and the next launch is unaffected."""
    ops, gu = env
    from muxserve_b200 import _lib
    ctx = [40, 700, 16]
    case, kc, vc = gu.make_case(len(ctx), 4, 2, ctx, 16, torch.float16, seed=8, num_blocks=512)
    bad = torch.tensor([0, 0, 0, 1], dtype=torch.int32, device="cuda")      # kv head 0: three q heads, group is 2
    out = torch.zeros_like(case.q[0])
    for psize in (0, 64):
        ops.paged_attention(out, case.q[0], kc, vc, bad, case.scale, case.block_tables[0], case.context_lens, 16,
                            case.max_context_len, partition_size=psize)
        assert ops.device_status() == _lib.MUX_DEV_BAD_HEAD_MAPPING
    good = torch.tensor([0, 0, 1, 1], dtype=torch.int32, device="cuda")
    ops.reshape_and_cache(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
    ops.paged_attention(out, case.q[0], kc, vc, good, case.scale, case.block_tables[0], case.context_lens, 16,
                        case.max_context_len)
    _, _, ref = gu.oracle_step(case, kc, vc, head_mapping=good)
    gu.assert_close(out, ref, "after a bad head_mapping")
    assert ops.device_status() == 0

    # mixed form: items claim 5 q heads each while the launch was sized for max_group = 2
    n = 6
    bt = case.block_tables[0].reshape(n, -1).contiguous()
    item_ctx = case.context_lens.repeat_interleave(2)
    q_rows = torch.randn(n * 2 + 8, 128, device="cuda").half()
    o_rows = torch.zeros_like(q_rows)
    row = torch.arange(0, 2 * n, 2, dtype=torch.int32, device="cuda")
    scale = torch.full((n,), case.scale, dtype=torch.float32, device="cuda")
    for psize in (0, 64):
        grp = torch.full((n,), 5, dtype=torch.int32, device="cuda")
        ops.paged_attention_mixed(o_rows, q_rows, kc, vc, bt, item_ctx, row, grp, scale, 16, case.max_context_len, 2,
                                  partition_size=psize)
        assert ops.device_status() == _lib.MUX_DEV_BAD_GROUP
    assert float(o_rows[2 * n:].abs().sum()) == 0.0          # rows beyond the sized tiles were never written
    grp = torch.full((n,), 2, dtype=torch.int32, device="cuda")
    ops.paged_attention_mixed(o_rows, q_rows, kc, vc, bt, item_ctx, row, grp, scale, 16, case.max_context_len, 2)
    assert ops.device_status() == 0 and not torch.isnan(o_rows).any()


def test_work_list_lists_empty_contexts(env):
    """work_units gives a sequence without context its partition 0, so the list form writes the same zero rows as
    the grid form."""
    ops, gu = env
    ctx = [0, 300, 0, 17]
    H = 2
    real = ops.work_units(ctx, 128, num_kv_heads=H)
    assert real.size == (1 + 3 + 1 + 1) * H
    case, kc, vc = gu.make_case(len(ctx), 4, H, [max(c, 1) for c in ctx], 16, torch.float16, seed=13, num_blocks=256)
    lens = torch.tensor(ctx, dtype=torch.int32, device="cuda")
    a = torch.full_like(case.q[0], float("nan"))
    b = torch.full_like(case.q[0], float("nan"))
    ops.paged_attention(a, case.q[0], kc, vc, None, case.scale, case.block_tables[0], lens, 16, 300, partition_size=128)
    ops.paged_attention(b, case.q[0], kc, vc, None, case.scale, case.block_tables[0], lens, 16, 300, partition_size=128,
                        units=torch.from_numpy(real).cuda())
    assert torch.equal(a, b) and not torch.isnan(a).any()
    assert float(a[0].abs().sum()) == 0.0 and float(a[2].abs().sum()) == 0.0
    assert ops.device_status() == 0
