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
