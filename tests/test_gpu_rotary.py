"""Rotary embedding: the stand-alone kernel vs the fp32 oracle, and the decode step with rotary fused
in vs rotary kernel + two ops (bit for bit)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(built_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from muxserve_b200 import ops
    import gpu_util
    return ops, gpu_util


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_rotary_kernel_vs_oracle(env, dtype):
    ops, gu = env
    from oracle.rotary_oracle import rotary_ref
    gen = torch.Generator().manual_seed(1)
    T, Hq, H = 37, 8, 2
    cache = ops.make_cos_sin_cache(4096, 10000.0, dtype)
    qkv = torch.randn(T, (Hq + 2 * H) * 128, generator=gen).to(dtype).cuda()      # strided views, as in the model
    q, k, v = qkv.split([Hq * 128, H * 128, H * 128], dim=-1)
    pos = torch.randint(0, 4096, (T,), generator=gen).cuda()
    q0, k0, v0 = q.clone(), k.clone(), v.clone()
    ops.rotary_embedding(pos, q, k, cache)
    for got, x0, heads in ((q, q0, Hq), (k, k0, H)):
        ref = rotary_ref(x0.reshape(T, heads, 128).cpu(), pos.cpu(), cache.cpu())
        err = (got.reshape(T, heads, 128).float().cpu() - ref).abs()
        assert bool((err <= 1e-3 + 4e-3 * ref.abs()).all()), err.max()             # one rounding to the 16-bit dtype
    assert torch.equal(v, v0)
    assert ops.device_status() == 0
    # position 0 is the identity
    q1 = q0.clone()
    ops.rotary_embedding(torch.zeros(T, dtype=torch.int64, device="cuda"), q1, None, cache)
    assert torch.equal(q1, q0)


@pytest.mark.parametrize("dtype,group", [(torch.float16, 1), (torch.bfloat16, 8)])
def test_decode_step_with_fused_rotary(env, dtype, group):
    ops, gu = env
    ctx = [1, 16, 17, 300, 513, 1000, 64]
    H = 2
    case, kc, vc = gu.make_case(len(ctx), H * group, H, ctx, 16, dtype, seed=70, num_blocks=1024)
    cache = ops.make_cos_sin_cache(2048, 10000.0, dtype)
    kc2, vc2 = kc.clone(), vc.clone()
    q, k, v = case.q[0].clone(), case.k[0].clone(), case.v[0].clone()
    # reference flow: rotary in place, cache write, attention
    pos = (case.context_lens - 1).long()
    ops.rotary_embedding(pos, q, k, cache)
    ops.reshape_and_cache(k, v, kc, vc, case.slot_mapping[:, 0, :])
    expect = torch.empty_like(q)
    ops.paged_attention(expect, q, kc, vc, None, case.scale, case.block_tables[0], case.context_lens, 16,
                        case.max_context_len)
    got = torch.full_like(expect, float("nan"))
    ops.decode_attention(got, case.q[0], case.k[0], case.v[0], kc2, vc2, None, case.scale, case.block_tables[0],
                         case.context_lens, 16, case.max_context_len, cos_sin_cache=cache)
    assert torch.equal(kc2.view(torch.int16), kc.view(torch.int16)) and torch.equal(vc2.view(torch.int16), vc.view(torch.int16))
    assert torch.equal(got, expect)
    assert ops.device_status() == 0
