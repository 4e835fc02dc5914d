"""CPU checks of the attention / cache-write oracle: known answers that hold for any correct
implementation, agreement of its two formulations, and the CPU-plumbing configuration
(one LLaMA-7B-shaped layer in fp32: 32 heads, head_dim 128, block 16, batch 8, pool 512 blocks)."""
import torch

from muxserve_b200 import flexstore, workloads
from oracle.attention_oracle import (gather_kv, paged_attention_items_ref, paged_attention_ref,
                                     paged_attention_ref_batched)
from oracle.cache_write_oracle import reshape_and_cache_ref


def make_cpu_case(S, Hq, H, lo, hi, seed, num_blocks=512, B=16, dtype=torch.float32):
    gen = torch.Generator().manual_seed(seed)
    ctx = workloads.uniform_context_lens(S, lo, hi, gen)
    while workloads.blocks_needed(ctx, 1, H, B) > num_blocks:      # keep the batch inside the pool
        ctx = (ctx // 2).clamp_min(1)
    shape = workloads.ModelShape("cpu", 1, Hq, H, S)
    case = workloads.make_decode_case(shape, ctx, block_size=B, num_blocks=num_blocks, dtype=dtype, device="cpu",
                                      seed=seed)
    es = torch.empty((), dtype=dtype).element_size()
    kc = torch.randn((num_blocks, *flexstore.get_key_block_shape(B, es)), generator=gen).to(dtype)
    vc = torch.randn((num_blocks, *flexstore.get_value_block_shape(B)), generator=gen).to(dtype)
    return case, kc, vc


def test_pool_geometry():
    assert flexstore.get_key_block_shape(16) == (16, 16, 8)
    assert flexstore.get_value_block_shape(16) == (128, 16)
    assert flexstore.block_bytes(16) == 8192
    n = flexstore.get_num_gpu_blocks(80 * 2 ** 30, 0.5, 16)
    assert n % 128 == 0 and abs(n * 8192 - 40 * 2 ** 30) < 128 * 8192 + 8192


def test_cache_write_oracle_roundtrip():
    case, kc, vc = make_cpu_case(8, 32, 32, 16, 16, seed=1)       # config 1 shape; ctx 16 keeps 256 blocks
    before_k, before_v = kc.clone(), vc.clone()
    reshape_and_cache_ref(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
    for s in range(8):
        for h in (0, 31):
            ctx = int(case.context_lens[s])
            k, v = gather_kv(kc, vc, case.block_tables[0, s, h, :(ctx + 15) // 16], ctx)
            assert torch.equal(k[-1], case.k[0][s, h]) and torch.equal(v[-1], case.v[0][s, h])
    changed_k = (kc != before_k).sum().item()
    assert changed_k <= 8 * 32 * 128 and (vc != before_v).sum().item() <= 8 * 32 * 128


def test_config1_cpu_plumbing_two_formulations_agree():
    case, kc, vc = make_cpu_case(8, 32, 32, 16, 512, seed=7, num_blocks=512)
    ref = paged_attention_ref(case.q[0], kc, vc, None, case.scale, case.block_tables[0], case.context_lens, 16)
    fast = paged_attention_ref_batched(case.q[0], kc, vc, case.scale, case.block_tables[0].clamp_min(0),
                                       case.context_lens, 16)
    assert torch.allclose(ref, fast, atol=1e-5, rtol=1e-5)
    # item form (mixed-model API) on the same data
    S, H = 8, 32
    items_bt = case.block_tables[0].reshape(S * H, -1).clamp_min(0)
    out = paged_attention_items_ref(case.q[0].reshape(S * H, 128), kc, vc, items_bt,
                                    case.context_lens.repeat_interleave(H), torch.arange(S * H),
                                    torch.ones(S * H, dtype=torch.int32), torch.full((S * H,), case.scale), 16)
    assert torch.allclose(out.view(S, H, 128), ref, atol=1e-5, rtol=1e-5)


def test_known_answers():
    case, kc, vc = make_cpu_case(4, 8, 2, 1, 200, seed=3)
    ones = paged_attention_ref(case.q[0], kc, torch.ones_like(vc), None, case.scale, case.block_tables[0],
                               case.context_lens, 16)
    assert torch.allclose(ones, torch.ones_like(ones), atol=1e-6)
    uniform = paged_attention_ref(torch.zeros_like(case.q[0]), kc, vc, None, case.scale, case.block_tables[0],
                                  case.context_lens, 16)
    ctx = int(case.context_lens[1])
    _, v = gather_kv(kc, vc, case.block_tables[0, 1, 0, :(ctx + 15) // 16], ctx)
    assert torch.allclose(uniform[1, 0], v.mean(0), atol=1e-5)
    assert torch.allclose(uniform[1, 3], uniform[1, 0])             # same kv head, same answer
    one = torch.tensor([1, 1, 1, 1], dtype=torch.int32)
    single = paged_attention_ref(case.q[0], kc, vc, None, case.scale, case.block_tables[0], one, 16)
    assert torch.equal(single[2, 5], vc[case.block_tables[0, 2, 1, 0].long(), :, 0].float())


def test_algorithmic_bytes_formula():
    ctx = [128, 2048]
    b = workloads.attention_bytes(ctx, 32, 32, 16)
    assert b == 32 * (128 + 2048) * 512 + 2 * 2 * 32 * 256 + 4 * 32 * (8 + 128) + 8
    assert workloads.cache_write_bytes(64, 32) == 4 * 64 * 32 * 256 + 8 * 64 * 32


def test_rotary_oracle_properties():
    from oracle.rotary_oracle import make_cos_sin_cache, rotary_ref
    cache = make_cos_sin_cache(512)
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(5, 3, 128, generator=gen)
    pos = torch.tensor([0, 1, 7, 100, 511])
    y = rotary_ref(x, pos, cache)
    assert torch.equal(y[0], x[0])                                             # position 0: identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)           # rotations keep the norm
    # relative-position property: <R_p q, R_p' k> depends on p - p' only
    q, k = x[1:2], x[2:3]
    a = (rotary_ref(q, torch.tensor([10]), cache) * rotary_ref(k, torch.tensor([4]), cache)).sum()
    b = (rotary_ref(q, torch.tensor([106]), cache) * rotary_ref(k, torch.tensor([100]), cache)).sum()
    assert torch.allclose(a, b, atol=1e-3)
