"""reshape_and_cache through the C ABI vs the scatter-copy oracle: bit-exact on the whole pool."""
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
@pytest.mark.parametrize("B", [8, 16, 32])
def test_cache_write_bit_exact(env, dtype, B):
    ops, gu = env
    ctx = [1, 5, B, B + 1, 3 * B - 1, 100, 17, 64]
    case, kc, vc = gu.make_case(len(ctx), 6, 6, ctx, B, dtype, seed=10 + B, num_blocks=512)
    kc_c, vc_c = kc.cpu().clone(), vc.cpu().clone()
    ops.reshape_and_cache(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
    from oracle.cache_write_oracle import reshape_and_cache_ref
    reshape_and_cache_ref(case.k[0].cpu(), case.v[0].cpu(), kc_c, vc_c, case.slot_mapping[:, 0, :].cpu())
    assert torch.equal(kc.cpu().view(torch.int16), kc_c.view(torch.int16))     # untouched slots unchanged too
    assert torch.equal(vc.cpu().view(torch.int16), vc_c.view(torch.int16))
    assert ops.device_status() == 0


def test_cache_write_strided_qkv_views_and_layer_slice(env):
    """k, v as views of one fused qkv tensor (llama.py:157-158); slots as the [:, layer, :] slice of [T, L, H]."""
    ops, gu = env
    T, Hq, H, L, B = 9, 8, 4, 3, 16
    gen = torch.Generator().manual_seed(5)
    qkv = torch.randn(T, (Hq + 2 * H) * 128, generator=gen).half().cuda()
    q, k, v = qkv.split([Hq * 128, H * 128, H * 128], dim=-1)
    kc = torch.zeros(256, 16, B, 8, dtype=torch.float16, device="cuda")
    vc = torch.zeros(256, 128, B, dtype=torch.float16, device="cuda")
    slots = torch.randperm(256 * B, generator=gen)[:T * L * H].view(T, L, H).cuda()
    slots[2, 1, 3] = -1          # padding row is skipped
    ops.reshape_and_cache(k, v, kc, vc, slots[:, 1, :])
    kc_c, vc_c = torch.zeros_like(kc).cpu(), torch.zeros_like(vc).cpu()
    from oracle.cache_write_oracle import reshape_and_cache_ref
    reshape_and_cache_ref(k.cpu().reshape(T, H, 128), v.cpu().reshape(T, H, 128), kc_c, vc_c, slots[:, 1, :].cpu())
    assert torch.equal(kc.cpu(), kc_c) and torch.equal(vc.cpu(), vc_c)
    assert int((vc != 0).sum()) > 0


def test_cache_write_multi_token_runs(env):
    """Eight new tokens per sequence in consecutive slots, crossing block boundaries."""
    ops, gu = env
    ctx = [8, 21, 16, 40, 129, 9]
    case, kc, vc = gu.make_case(len(ctx), 8, 2, ctx, 16, torch.bfloat16, seed=77, num_blocks=256, new_tokens=8)
    kc_c, vc_c = kc.cpu().clone(), vc.cpu().clone()
    ops.reshape_and_cache(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
    from oracle.cache_write_oracle import reshape_and_cache_ref
    reshape_and_cache_ref(case.k[0].cpu(), case.v[0].cpu(), kc_c, vc_c, case.slot_mapping[:, 0, :].cpu())
    assert torch.equal(kc.cpu().view(torch.int16), kc_c.view(torch.int16))
    assert torch.equal(vc.cpu().view(torch.int16), vc_c.view(torch.int16))


def test_cache_write_bad_slot_is_skipped_and_reported(env):
    ops, gu = env
    from muxserve_b200 import _lib
    kc = torch.zeros(8, 16, 16, 8, dtype=torch.float16, device="cuda")
    vc = torch.zeros(8, 128, 16, dtype=torch.float16, device="cuda")
    k = torch.ones(2, 1, 128, dtype=torch.float16, device="cuda")
    slots = torch.tensor([[3], [8 * 16 + 5]], dtype=torch.int64, device="cuda")   # second slot is outside the pool
    ops.reshape_and_cache(k, k, kc, vc, slots)
    assert ops.device_status() == _lib.MUX_DEV_BAD_SLOT
    assert ops.device_status() == 0                      # reading clears
    assert float(kc.sum()) == 128.0 and float(vc.sum()) == 128.0


def test_cache_write_empty_and_errors(env):
    ops, gu = env
    kc = torch.zeros(8, 16, 16, 8, dtype=torch.float16, device="cuda")
    vc = torch.zeros(8, 128, 16, dtype=torch.float16, device="cuda")
    empty = torch.empty(0, 2, 128, dtype=torch.float16, device="cuda")
    ops.reshape_and_cache(empty, empty, kc, vc, torch.empty(0, 2, dtype=torch.int64, device="cuda"))
    k = torch.ones(1, 2, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(TypeError):
        ops.reshape_and_cache(k.bfloat16(), k.bfloat16(), kc, vc, torch.zeros(1, 2, dtype=torch.int64, device="cuda"))
    with pytest.raises(RuntimeError):
        ops.reshape_and_cache(k.cpu(), k.cpu(), kc, vc, torch.zeros(1, 2, dtype=torch.int64))


# ---- many tokens: the run-based kernel (taken from 256 tokens up) ----------------------------------------
def _check_against_oracle(ops, k, v, kc, vc, slots):
    from oracle.cache_write_oracle import reshape_and_cache_ref
    kc_c, vc_c = kc.cpu().clone(), vc.cpu().clone()
    ops.reshape_and_cache(k, v, kc, vc, slots)
    T, H = slots.shape
    reshape_and_cache_ref(k.cpu().reshape(T, H, 128), v.cpu().reshape(T, H, 128), kc_c, vc_c, slots.cpu())
    assert torch.equal(kc.cpu().view(torch.int16), kc_c.view(torch.int16))
    assert torch.equal(vc.cpu().view(torch.int16), vc_c.view(torch.int16))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B", [8, 16, 32])
def test_prompt_cache_write_bit_exact(env, dtype, B):
    """Every token of ragged prompts, slots as the reference's getPromptSlots gives them (csrc/batch_scheduler.h:42-56)."""
    ops, gu = env
    from muxserve_b200 import flexstore, workloads
    gen = torch.Generator().manual_seed(100 + B)
    lens = torch.tensor([300, 17, 1000, 5, 64, 1, 2 * B], dtype=torch.int32)
    L, H, nblk = 2, 3, 2048
    tables, _ = workloads.scatter_block_tables(lens, L, H, B, torch.randperm(nblk, generator=gen).cuda())
    slots = workloads.prompt_slots(tables, lens, B)          # [T, L, H]
    T = int(lens.sum())
    qkv = torch.randn((T, 5 * H * 128), generator=gen).to(dtype).cuda()       # k, v as strided views
    k, v = qkv[:, H * 128:2 * H * 128], qkv[:, 3 * H * 128:4 * H * 128]
    kc, vc = flexstore.allocate_gpu_cache(nblk, B, dtype, "cuda")
    workloads.fill_pool_(kc, vc, 7)
    _check_against_oracle(ops, k, v, kc, vc, slots[:, 1, :])
    assert ops.device_status() == 0


def test_many_token_cache_write_unaligned_runs(env):
    """Eight new tokens per sequence starting at arbitrary offsets: short runs that straddle blocks and CTAs' windows."""
    ops, gu = env
    ctx = [8 + 3 * i for i in range(44)]                   # 352 rows
    case, kc, vc = gu.make_case(len(ctx), 4, 2, ctx, 16, torch.float16, seed=78, num_blocks=1024, new_tokens=8)
    _check_against_oracle(ops, case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
    assert ops.device_status() == 0


def test_many_token_cache_write_scattered_padding_and_bad_slots(env):
    ops, gu = env
    from muxserve_b200 import _lib
    gen = torch.Generator().manual_seed(9)
    T, H, B, nblk = 300, 2, 16, 128
    slots = torch.randperm(nblk * B, generator=gen)[:T * H].view(T, H).clone()
    slots[5, 0] = -1                   # padding rows are skipped silently
    slots[64, 1] = -1
    slots[100, 0] = nblk * B + 3       # outside the pool: skipped and reported
    k = torch.randn((T, H, 128), generator=gen).half().cuda()
    v = torch.randn((T, H, 128), generator=gen).half().cuda()
    kc = torch.zeros(nblk, 16, B, 8, dtype=torch.float16, device="cuda")
    vc = torch.zeros(nblk, 128, B, dtype=torch.float16, device="cuda")
    ok = slots.clone()
    ok[100, 0] = -1
    from oracle.cache_write_oracle import reshape_and_cache_ref
    kc_c, vc_c = kc.cpu().clone(), vc.cpu().clone()
    ops.reshape_and_cache(k, v, kc, vc, slots.cuda())
    reshape_and_cache_ref(k.cpu(), v.cpu(), kc_c, vc_c, ok)
    assert torch.equal(kc.cpu(), kc_c) and torch.equal(vc.cpu(), vc_c)
    assert ops.device_status() == _lib.MUX_DEV_BAD_SLOT
