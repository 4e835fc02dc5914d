"""Full benchmark sizes (one layer of config 2 and of config 5), where the CPU oracle would take too long:
properties that hold for any correct implementation, independent of the oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(S, Hq, H, lo, hi, dtype, seed, new_tokens=1):
    import gpu_util as gu
    from muxserve_b200 import workloads
    gen = torch.Generator().manual_seed(seed)
    ctx = workloads.uniform_context_lens(S, lo, hi, gen)
    nblocks = (workloads.blocks_needed(ctx, 1, H, 16) * 5 // 4 + 127) // 128 * 128
    return gu.make_case(S, Hq, H, ctx, 16, dtype, seed, nblocks, new_tokens=new_tokens)


@pytest.mark.parametrize("name,S,Hq,H,lo,hi,dtype", [("config2", 64, 32, 32, 128, 2048, torch.float16),
                                                      ("config5", 256, 64, 8, 2048, 8192, torch.bfloat16)])
def test_full_size_layer_properties(built_lib, name, S, Hq, H, lo, hi, dtype):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from muxserve_b200 import ops
    case, kc, vc = _case(S, Hq, H, lo, hi, dtype, seed=123)
    q, k, v, bt, ctx = case.q[0], case.k[0], case.v[0], case.block_tables[0], case.context_lens
    kc2, vc2 = kc.clone(), vc.clone()
    args = (None, case.scale, bt, ctx, 16, case.max_context_len)
    # 1. fused decode step == cache write + attention, bit for bit, pool included
    ops.reshape_and_cache(k, v, kc, vc, case.slot_mapping[:, 0, :])
    two = torch.empty_like(q)
    ops.paged_attention(two, q, kc, vc, *args)
    one = torch.empty_like(q)
    ops.decode_attention(one, q, k, v, kc2, vc2, *args)
    assert torch.equal(one, two) and torch.equal(kc, kc2) and torch.equal(vc, vc2)
    # 2. the cache write round-trips: the last token of every (sequence, head) reads back as written
    slots = case.slot_mapping[:, 0, :]
    blk, off = (slots // 16).reshape(-1), (slots % 16).reshape(-1)
    assert torch.equal(kc[blk, :, off, :].reshape(S, H, 128), k) and torch.equal(vc[blk, :, off].reshape(S, H, 128), v)
    # 3. the partitioning does not change the answer beyond fp32 re-association
    other = torch.empty_like(q)
    ops.paged_attention(other, q, kc, vc, *args, partition_size=2048 if name == "config2" else 1024)
    assert torch.allclose(other.float(), two.float(), atol=2e-3, rtol=1e-2)
    # 4. softmax weights sum to one: V == 1 gives 1; and the output is linear in V
    ops.paged_attention(other, q, kc, torch.ones_like(vc), *args)
    assert torch.allclose(other.float(), torch.ones_like(other).float(), atol=2e-3)
    ops.paged_attention(other, q, kc, vc * 2, *args)
    assert torch.allclose(other.float(), 2 * two.float(), atol=4e-3, rtol=1e-2)
    # 5. q == 0: every head of a sequence's kv group returns the same mean of V
    ops.paged_attention(other, torch.zeros_like(q), kc, vc, *args)
    grp = other.view(S, H, Hq // H, 128).float()
    assert torch.allclose(grp, grp[:, :, :1].expand_as(grp), atol=1e-6)
    assert ops.device_status() == 0


def _sampled(case, out, kc, vc, new_tokens=1, layer=0, seed=0):
    from oracle.sampled_check import check_decode_rows, pick_sequences
    seqs = pick_sequences(case.context_lens.tolist(), 4, seed)
    return check_decode_rows(out, case.q[layer], case.k[layer], case.v[layer], kc, vc, case.block_tables[layer],
                             case.context_lens, case.scale, 16, seqs, new_tokens=new_tokens)


@pytest.mark.parametrize("name,S,Hq,H,lo,hi,dtype,nt", [
    ("config2", 64, 32, 32, 128, 2048, torch.float16, 1),
    ("config4", 128, 64, 64, 512, 4096, torch.bfloat16, 1),
    ("config4 TP=8 shard", 128, 8, 8, 512, 4096, torch.bfloat16, 1),
    ("config5", 256, 64, 8, 2048, 8192, torch.bfloat16, 8),
])
def test_full_size_launch_against_the_oracle_on_sampled_sequences(built_lib, name, S, Hq, H, lo, hi, dtype, nt):
    """One layer at the benchmark's own shape, launched the way bench.py launches it (work list, the partition size
    and ring depth the launch heuristic picks, early-KV flag): the fp32 oracle on four sampled sequences (all their
    heads, tolerance 2e-3 + 1e-2 * |ref|) and the appended K/V rows bit for bit."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from muxserve_b200 import ops
    case, kc, vc = _case(S, Hq, H, lo, hi, dtype, seed=321, new_tokens=nt)
    ctx = case.context_lens.tolist()
    psize, nst = ops.suggest_launch(ctx, Hq // H, num_kv_heads=H)
    units = ops.work_units(ctx, psize, "cuda", num_kv_heads=H)
    out = torch.full_like(case.q[0], float("nan"))
    if nt <= ops.MAX_FUSED_NEW_TOKENS:
        ops.decode_attention(out, case.q[0], case.k[0], case.v[0], kc, vc, None, case.scale, case.block_tables[0],
                             case.context_lens, 16, case.max_context_len, partition_size=psize, num_stages=nst,
                             units=units, early_kv=True)
    else:
        ops.reshape_and_cache(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
        ops.paged_attention(out, case.q[0], kc, vc, None, case.scale, case.block_tables[0], case.context_lens, 16,
                            case.max_context_len, partition_size=psize, num_stages=nst, units=units)
    assert not torch.isnan(out).any()
    pc = _sampled(case, out, kc, vc, new_tokens=nt)
    assert pc["ok"] and pc["pool_bit_exact"], pc
    assert ops.device_status() == 0


def test_config3_fused_mixed_launches_against_the_oracle(built_lib):
    """Config 3 at its real shape (local heads 8/10/13, batches 48/24/12, lognormal contexts up to 4096): the fused
    mixed launch of a layer every model has, of one only the two deeper models have and of one only the deepest has,
    each with its work list and the per-launch partition size; every model's sampled sequences against the oracle."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from muxserve_b200 import flexstore, mixed, ops, workloads
    from oracle.sampled_check import check_decode_rows, pick_sequences
    dev, dt, nb = "cuda", torch.float16, 1 << 19          # 4 GiB pool
    kc, vc = flexstore.allocate_gpu_cache(nb, 16, dt, dev)
    workloads.fill_pool_(kc, vc, 5)
    gen = torch.Generator().manual_seed(20240531)
    perm = torch.randperm(nb, generator=gen).to(dev)
    layers_kept = 3                                        # block lists for three layers per model are enough
    batches, cases, nxt = [], [], 0
    for name, depth, heads, S in (("llama-7b", 1, 32, 48), ("llama-13b", 2, 40, 24), ("llama-30b", 3, 52, 12)):
        Hl = heads // 4
        ctx = workloads.lognormal_context_lens(S, 256.0, 1.0, 16, 4096, gen)
        case = workloads.make_decode_case(workloads.ModelShape(name, depth, Hl, Hl, S), ctx, block_size=16, num_blocks=nb,
                                          dtype=dt, device=dev, seed=len(cases), block_ids=perm, first_block=nxt)
        nxt = case.extra["next_block"]
        cases.append(case)
        batches.append(mixed.ModelBatch(name, depth, Hl, Hl, 128 ** -0.5, ctx, case.block_tables))
    plan = mixed.build_mixed_plan(batches, dev)
    assert plan.item_offset == [0, 156, 396, 780]
    for l in range(layers_kept):
        n_items, n_rows = plan.active(l)
        ps, ns = ops.suggest_launch(plan.item_context_len_host[:n_items], plan.max_group, dev)
        q = mixed.pack_rows(plan, [c.q[min(l, c.q.shape[0] - 1)] for c in cases])
        k = mixed.pack_items(plan, [c.k[min(l, c.k.shape[0] - 1)] for c in cases])
        v = mixed.pack_items(plan, [c.v[min(l, c.v.shape[0] - 1)] for c in cases])
        out = torch.full_like(q, float("nan"))
        ops.paged_attention_mixed(out[:n_rows], q[:n_rows], kc, vc, plan.block_tables[l, :n_items],
                                  plan.item_context_len[:n_items], plan.item_q_row[:n_items], plan.item_group[:n_items],
                                  plan.item_scale[:n_items], 16, plan.max_context_len, plan.max_group, partition_size=ps,
                                  num_stages=ns, units=plan.units(l, ps), new_k=k[:n_items], new_v=v[:n_items],
                                  early_kv=True)
        assert torch.isnan(out[n_rows:]).all() and not torch.isnan(out[:n_rows]).any()
        for c, b, o in zip(cases, batches, mixed.unpack_rows(plan, out, batches)):
            if b.num_layers <= l:
                continue
            pc = check_decode_rows(o, c.q[l], c.k[l], c.v[l], kc, vc, c.block_tables[l], c.context_lens, c.scale, 16,
                                   pick_sequences(c.context_lens.tolist(), 3, l))
            assert pc["ok"] and pc["pool_bit_exact"], (b.name, l, pc)
    assert ops.device_status() == 0
