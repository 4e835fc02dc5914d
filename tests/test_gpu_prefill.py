"""GPU parity: prompt-phase attention (tcgen05 kernel) against the fp32 oracle, through the C ABI."""
import pytest
import torch

from oracle.prefill_oracle import prefill_attention_ref
from tests.gpu_util import ATOL, RTOL

pytestmark = pytest.mark.gpu


def _run(prompt_lens, Hq, H, dtype, seed, strided=False, scale=None):
    from muxserve_b200 import ops
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(seed)
    T = int(sum(prompt_lens))
    scale = scale if scale is not None else 128 ** -0.5
    if strided:  # q, k, v as the split views of one fused projection output
        qkv = torch.randn((T, (Hq + 2 * H) * 128), generator=gen).to(dtype).to(dev)
        q, k, v = qkv.split([Hq * 128, H * 128, H * 128], dim=1)
    else:
        q = torch.randn((T, Hq, 128), generator=gen).to(dtype).to(dev)
        k = torch.randn((T, H, 128), generator=gen).to(dtype).to(dev)
        v = torch.randn((T, H, 128), generator=gen).to(dtype).to(dev)
    out = torch.full((T, Hq * 128), float("nan"), dtype=dtype, device=dev)
    cu = ops.cu_seqlens_from_prompt_lens(prompt_lens, dev)
    ops.prefill_attention(out, q, k, v, cu, max(prompt_lens) if prompt_lens else 0, scale)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    ref = prefill_attention_ref(q.reshape(T, Hq, 128), k.reshape(T, H, 128), v.reshape(T, H, 128), prompt_lens, scale)
    got = out.float().cpu().view(T, Hq, 128)
    err = (got - ref).abs()
    bound = ATOL + RTOL * ref.abs()
    assert torch.isfinite(got).all()
    assert (err <= bound).all(), f"max err {err.max().item():.3e} (worst excess {(err - bound).max().item():.3e})"


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_single_tile(dtype):
    _run([128], 2, 2, dtype, 1)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_ragged_multi_tile(dtype):
    _run([1, 5, 127, 128, 129, 300, 777], 4, 4, dtype, 2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gqa_and_strided_views(dtype):
    _run([33, 260, 513], 8, 2, dtype, 3, strided=True)


def test_long_prompt_fp16():
    _run([2048, 1500], 2, 1, torch.float16, 4)


def test_large_logits_trigger_rescale():
    # scale 1.0 on N(0,1) rows gives logits of tens of units: the running maximum keeps growing across tiles
    _run([640], 2, 2, torch.float16, 5, scale=1.0)


def test_empty_and_zero_length():
    _run([0, 17, 0], 2, 2, torch.float16, 6)
    from muxserve_b200 import ops
    dev = torch.device("cuda:0")
    e = torch.empty((0, 256), dtype=torch.float16, device=dev)
    ops.prefill_attention(e, e, e, e, torch.zeros(1, dtype=torch.int32, device=dev), 0, 0.1)


def test_bad_offsets_are_reported_not_read():
    from muxserve_b200 import _lib, ops
    dev = torch.device("cuda:0")
    q = torch.randn((64, 2, 128), dtype=torch.float16, device=dev)
    out = torch.zeros_like(q)
    cu = torch.tensor([0, 9999], dtype=torch.int32, device=dev)   # claims more rows than the tensors hold
    ops.prefill_attention(out, q, q, q, cu, 64, 0.1)
    torch.cuda.synchronize()
    assert ops.device_status() & _lib.MUX_DEV_BAD_CONTEXT
    assert (out == 0).all()


def test_rejects_bad_arguments():
    from muxserve_b200 import _lib, ops
    dev = torch.device("cuda:0")
    q = torch.randn((16, 3, 128), dtype=torch.float16, device=dev)
    k = torch.randn((16, 2, 128), dtype=torch.float16, device=dev)
    cu = torch.tensor([0, 16], dtype=torch.int32, device=dev)
    with pytest.raises(_lib.MuxError):
        ops.prefill_attention(torch.empty_like(q), q, k, k, cu, 16, 0.1)      # 3 q heads over 2 kv heads
    with pytest.raises(_lib.MuxError):
        ops.prefill_attention(torch.empty_like(q), q, q, q, cu, 16, 0.0)      # scale must be positive


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_many_short_prompts_fill_every_sm_twice(dtype):
    """Thousands of short CTAs, two per SM: the hand-offs between warps that run a step apart must hold."""
    gen = torch.Generator().manual_seed(11)
    lens = torch.randint(200, 513, (160,), generator=gen).tolist()
    _run(lens, 8, 8, dtype, 12)


# ---- prompt cache write in the same launch ----------------------------------------------------------------
def _fused_case(lens, Hq, H, dtype, B, seed, spoil=False):
    from muxserve_b200 import flexstore, ops, workloads
    from oracle.cache_write_oracle import reshape_and_cache_ref
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(seed)
    lens_t = torch.tensor(lens, dtype=torch.int32)
    T, L, nblk = int(lens_t.sum()), 2, 4096
    tables, _ = workloads.scatter_block_tables(lens_t, L, H, B, torch.randperm(nblk, generator=gen).to(dev))
    slots = workloads.prompt_slots(tables, lens_t, B)                     # [T, L, H]; the op gets the layer-1 slice
    if spoil:
        slots[3, 1, 0] = -1                                               # padding row: skipped
        slots[T - 2, 1, H - 1] = nblk * B + 5                             # outside the pool: reported and skipped
        slots[40:48, 1, 0] = slots[40:48, 1, 0].flip(0)                   # a group of 8 that is not a run
    q = torch.randn((T, Hq, 128), generator=gen).to(dtype).to(dev)
    k = torch.randn((T, H, 128), generator=gen).to(dtype).to(dev)
    v = torch.randn((T, H, 128), generator=gen).to(dtype).to(dev)
    kc, vc = flexstore.allocate_gpu_cache(nblk, B, dtype, dev)
    workloads.fill_pool_(kc, vc, seed + 1)
    kc_c, vc_c = kc.cpu().clone(), vc.cpu().clone()
    out = torch.full((T, Hq, 128), float("nan"), dtype=dtype, device=dev)
    cu = ops.cu_seqlens_from_prompt_lens(lens, dev)
    ops.prefill_attention(out, q, k, v, cu, max(lens), 128 ** -0.5, key_cache=kc, value_cache=vc,
                          slot_mapping=slots[:, 1, :])
    torch.cuda.synchronize()
    status = ops.device_status()
    ok = slots[:, 1, :].cpu().clone()
    ok[ok >= nblk * B] = -1
    reshape_and_cache_ref(k.cpu(), v.cpu(), kc_c, vc_c, ok)
    assert torch.equal(kc.cpu().view(torch.int16), kc_c.view(torch.int16)), "key pool differs"
    assert torch.equal(vc.cpu().view(torch.int16), vc_c.view(torch.int16)), "value pool differs"
    ref = prefill_attention_ref(q, k, v, lens, 128 ** -0.5)
    err = (out.float().cpu() - ref).abs()
    assert (err <= ATOL + RTOL * ref.abs()).all()
    return status


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B", [8, 16, 32])
def test_fused_prompt_cache_write_bit_exact(dtype, B):
    assert _fused_case([1, 7, 64, 100, 129, 300, 515], 4, 4, dtype, B, 21 + B) == 0


def test_fused_prompt_cache_write_gqa_writes_each_kv_head_once():
    assert _fused_case([33, 260, 513, 128], 8, 2, torch.bfloat16, 16, 31) == 0


def test_fused_prompt_cache_write_padding_bad_slots_and_broken_runs():
    from muxserve_b200 import _lib
    assert _fused_case([200, 90], 2, 2, torch.float16, 16, 41, spoil=True) == _lib.MUX_DEV_BAD_SLOT


@pytest.mark.parametrize("B", [8, 16, 32])
def test_fused_prompt_cache_write_from_block_tables(B):
    """The block lists stand in for the slot mapping: same pool contents as reshape_and_cache with getPromptSlots' slots."""
    from muxserve_b200 import flexstore, ops, workloads
    from oracle.cache_write_oracle import reshape_and_cache_ref
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(70 + B)
    lens = [5, 64, 130, 257, 1]
    lens_t = torch.tensor(lens, dtype=torch.int32)
    T, L, H, Hq, nblk, dtype = int(lens_t.sum()), 3, 2, 4, 1024, torch.float16
    tables, _ = workloads.scatter_block_tables(lens_t, L, H, B, torch.randperm(nblk, generator=gen).to(dev))
    slots = workloads.prompt_slots(tables, lens_t, B)
    q = torch.randn((T, Hq, 128), generator=gen).to(dtype).to(dev)
    k = torch.randn((T, H, 128), generator=gen).to(dtype).to(dev)
    v = torch.randn((T, H, 128), generator=gen).to(dtype).to(dev)
    kc, vc = flexstore.allocate_gpu_cache(nblk, B, dtype, dev)
    workloads.fill_pool_(kc, vc, 3)
    kc_c, vc_c = kc.cpu().clone(), vc.cpu().clone()
    out = torch.empty_like(q)
    ops.prefill_attention(out, q, k, v, ops.cu_seqlens_from_prompt_lens(lens, dev), max(lens), 128 ** -0.5,
                          key_cache=kc, value_cache=vc, block_tables=tables[2])       # a [S, H, max_blocks] layer slice
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    reshape_and_cache_ref(k.cpu(), v.cpu(), kc_c, vc_c, slots[:, 2, :].cpu())
    assert torch.equal(kc.cpu().view(torch.int16), kc_c.view(torch.int16))
    assert torch.equal(vc.cpu().view(torch.int16), vc_c.view(torch.int16))
    ref = prefill_attention_ref(q, k, v, lens, 128 ** -0.5)
    err = (out.float().cpu() - ref).abs()
    assert (err <= ATOL + RTOL * ref.abs()).all()


@pytest.mark.parametrize("seed", range(12))
def test_prefill_fuzz(seed):
    """Random prompt sets, head layouts, dtypes, block sizes and hand-over forms (none / slot mapping / block lists)."""
    import random
    from muxserve_b200 import flexstore, ops, workloads
    from oracle.cache_write_oracle import reshape_and_cache_ref
    rng = random.Random(1000 + seed)
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(2000 + seed)
    dtype = rng.choice([torch.float16, torch.bfloat16])
    H = rng.choice([1, 2, 3, 4])
    Hq = H * rng.choice([1, 2, 4])
    B = rng.choice([8, 16, 32])
    nprompts = rng.randint(1, 24)
    lens = [rng.choice([0, 1, rng.randint(2, 63), rng.randint(64, 400), rng.randint(400, 900)]) for _ in range(nprompts)]
    if sum(lens) == 0:
        lens[0] = 17
    mode = rng.choice(["none", "slots", "tables"])
    scale = rng.choice([128 ** -0.5, 0.05, 0.3])
    lens_t = torch.tensor(lens, dtype=torch.int32)
    T, L, nblk = int(lens_t.sum()), 2, 2048
    q = torch.randn((T, Hq, 128), generator=gen).to(dtype).to(dev)
    k = torch.randn((T, H, 128), generator=gen).to(dtype).to(dev)
    v = torch.randn((T, H, 128), generator=gen).to(dtype).to(dev)
    out = torch.full((T, Hq, 128), float("nan"), dtype=dtype, device=dev)
    cu = ops.cu_seqlens_from_prompt_lens(lens, dev)
    kw = {}
    if mode != "none":
        tables, _ = workloads.scatter_block_tables(lens_t, L, H, B, torch.randperm(nblk, generator=gen).to(dev))
        slots = workloads.prompt_slots(tables, lens_t, B)
        kc, vc = flexstore.allocate_gpu_cache(nblk, B, dtype, dev)
        workloads.fill_pool_(kc, vc, seed)
        kc_c, vc_c = kc.cpu().clone(), vc.cpu().clone()
        kw = dict(key_cache=kc, value_cache=vc)
        kw.update(slot_mapping=slots[:, 1, :]) if mode == "slots" else kw.update(block_tables=tables[1])
    ops.prefill_attention(out, q, k, v, cu, max(lens) + rng.choice([0, 0, 77]), scale, **kw)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    ref = prefill_attention_ref(q, k, v, lens, scale)
    got = out.float().cpu()
    assert torch.isfinite(got).all()
    err = (got - ref).abs()
    assert (err <= ATOL + RTOL * ref.abs()).all(), f"max err {err.max().item():.3e}"
    if mode != "none":
        reshape_and_cache_ref(k.cpu(), v.cpu(), kc_c, vc_c, slots[:, 1, :].cpu())
        assert torch.equal(kc.cpu().view(torch.int16), kc_c.view(torch.int16))
        assert torch.equal(vc.cpu().view(torch.int16), vc_c.view(torch.int16))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_prefill_work_list_is_bit_identical(dtype):
    """units= removes the CTAs of tiles a prompt does not have and reorders the rest; results and pool writes are the same."""
    import numpy as np
    from muxserve_b200 import flexstore, ops, workloads
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(77)
    lens = [300, 5, 0, 1025, 128, 64, 700]
    lens_t = torch.tensor(lens, dtype=torch.int32)
    T, Hq, H, B, nblk = int(lens_t.sum()), 4, 2, 16, 1024
    q = torch.randn((T, Hq, 128), generator=gen).to(dtype).to(dev)
    k = torch.randn((T, H, 128), generator=gen).to(dtype).to(dev)
    v = torch.randn((T, H, 128), generator=gen).to(dtype).to(dev)
    cu = ops.cu_seqlens_from_prompt_lens(lens, dev)
    tables, _ = workloads.scatter_block_tables(lens_t, 1, H, B, torch.randperm(nblk, generator=gen).to(dev))
    real = ops.prefill_work_units(lens, Hq)
    assert real.shape == (sum((n + 127) // 128 for n in lens) * Hq, 2)
    padded = np.concatenate([real, np.full((5, 2), -1, dtype=np.int32)])
    units = torch.from_numpy(padded).to(dev)
    outs, pools = [], []
    for u in (None, units):
        kc, vc = flexstore.allocate_gpu_cache(nblk, B, dtype, dev)
        workloads.fill_pool_(kc, vc, 5)
        out = torch.zeros_like(q)
        ops.prefill_attention(out, q, k, v, cu, max(lens), 128 ** -0.5, key_cache=kc, value_cache=vc,
                              block_tables=tables[0], units=u)
        outs.append(out)
        pools.append((kc, vc))
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(pools[0][0], pools[1][0]) and torch.equal(pools[0][1], pools[1][1])
