"""paged_attention through the C ABI vs the fp32 gather oracle (tolerance 2e-3 abs + 1e-2 rel)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(built_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from muxserve_b200 import ops
    import gpu_util
    return ops, gu_mod()


def gu_mod():
    import gpu_util
    return gpu_util


def run(ops, gu, case, kc, vc, head_mapping=None, **kw):
    ops.reshape_and_cache(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
    out = torch.full_like(case.q[0], float("nan"))
    ops.paged_attention(out, case.q[0], kc, vc, head_mapping, case.scale, case.block_tables[0],
                        case.context_lens, case.block_size, case.max_context_len, **kw)
    return out


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B", [16, 8, 32])
@pytest.mark.parametrize("group", [1, 8])
def test_attention_ragged(env, dtype, B, group):
    ops, gu = env
    ctx = [1, 2, B - 1, B, B + 1, 255, 256, 257, 300, 511, 77, 1000]
    H = 3
    case, kc, vc = gu.make_case(len(ctx), H * group, H, ctx, B, dtype, seed=3 + B + group, num_blocks=2048)
    out = run(ops, gu, case, kc, vc)
    kc_c, vc_c, ref = gu.oracle_step(case, kc, vc)
    assert torch.equal(kc.cpu().view(torch.int16), kc_c.view(torch.int16))
    gu.assert_close(out, ref, f"B={B} G={group} {dtype}")
    assert ops.device_status() == 0


@pytest.mark.parametrize("psize,stages", [(16, 4), (64, 4), (128, 8), (512, 8), (1024, 12), (4096, 16)])
def test_attention_partition_sizes(env, psize, stages):
    """Every partitioning gives the same answer (single partition up to 63 partitions per sequence)."""
    ops, gu = env
    ctx = [1000, 17, 513, 64, 2, 999]
    case, kc, vc = gu.make_case(len(ctx), 4, 4, ctx, 16, torch.float16, seed=21, num_blocks=1024)
    out = run(ops, gu, case, kc, vc, partition_size=psize, num_stages=stages)
    _, _, ref = gu.oracle_step(case, kc, vc)
    gu.assert_close(out, ref, f"partition {psize}")
    assert ops.device_status() == 0


@pytest.mark.parametrize("group", [2, 4, 5, 16, 12])
def test_attention_group_sizes(env, group):
    """GQA groups that do not fill, or overflow, one 8-head tile."""
    ops, gu = env
    ctx = [300, 31, 129, 16]
    case, kc, vc = gu.make_case(len(ctx), 2 * group, 2, ctx, 16, torch.bfloat16, seed=group, num_blocks=512)
    out = run(ops, gu, case, kc, vc)
    _, _, ref = gu.oracle_step(case, kc, vc)
    gu.assert_close(out, ref, f"group {group}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_attention_short_contexts_cancellation(env, dtype):
    """Few-token contexts: the output is a signed mix of two or three V rows and is often near zero,
    so any loss of precision in the softmax weights shows against the absolute tolerance."""
    ops, gu = env
    gen = torch.Generator().manual_seed(99)
    ctx = torch.randint(1, 7, (96,), generator=gen).tolist()
    case, kc, vc = gu.make_case(len(ctx), 8, 4, ctx, 16, dtype, seed=40, num_blocks=1024)
    vc.mul_(4.0)                                  # larger values, larger cancellation
    out = run(ops, gu, case, kc, vc)
    _, _, ref = gu.oracle_step(case, kc, vc)
    gu.assert_close(out, ref, f"short contexts {dtype}")


def test_attention_head_mapping_interleaved(env):
    """head_mapping need not be contiguous groups: q head hq reads kv head hq % H."""
    ops, gu = env
    ctx = [100, 260, 15]
    H, G = 4, 3
    case, kc, vc = gu.make_case(len(ctx), H * G, H, ctx, 16, torch.float16, seed=8, num_blocks=512)
    hm = (torch.arange(H * G, dtype=torch.int32) % H).cuda()
    out = run(ops, gu, case, kc, vc, head_mapping=hm)
    _, _, ref = gu.oracle_step(case, kc, vc, head_mapping=hm)
    gu.assert_close(out, ref, "interleaved head_mapping")
    hm2 = (torch.arange(H * G, dtype=torch.int32) // G).cuda()
    out2 = run(ops, gu, case, kc, vc, head_mapping=hm2)
    out3 = run(ops, gu, case, kc, vc, head_mapping=None)
    assert torch.equal(out2, out3)
    assert ops.device_status() == 0


def test_attention_strided_q_and_2d_shapes(env):
    """q as a view of a fused qkv tensor [S, (Hq+2H)*D]; out 2-D [S, Hq*D]."""
    ops, gu = env
    ctx = [33, 200, 90, 7]
    Hq = H = 5
    case, kc, vc = gu.make_case(len(ctx), Hq, H, ctx, 16, torch.float16, seed=12, num_blocks=512)
    S = len(ctx)
    qkv = torch.zeros(S, 3 * Hq * 128, dtype=torch.float16, device="cuda")
    qkv[:, :Hq * 128] = case.q[0].reshape(S, -1)
    q_view = qkv[:, :Hq * 128]
    ops.reshape_and_cache(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
    out = torch.empty(S, Hq * 128, dtype=torch.float16, device="cuda")
    ops.paged_attention(out, q_view, kc, vc, None, case.scale, case.block_tables[0], case.context_lens, 16,
                        case.max_context_len)
    _, _, ref = gu.oracle_step(case, kc, vc)
    gu.assert_close(out.view(S, Hq, 128), ref, "strided q")


def test_attention_poisoned_padding_and_stale_tails(env):
    """Block-table entries past a list's end point at a NaN block and the unwritten tail of every
    last block is NaN: neither may reach the output (the reference leaves both uninitialised)."""
    ops, gu = env
    ctx = [1, 17, 40, 255, 130, 300]
    case, kc, vc = gu.make_case(len(ctx), 4, 4, ctx, 16, torch.float16, seed=31, num_blocks=1024)
    used = case.block_tables[case.block_tables >= 0].long()
    free = torch.ones(1024, dtype=torch.bool, device="cuda")
    free[used] = False
    poison = int(torch.nonzero(free)[0])
    kc[poison], vc[poison] = float("nan"), float("nan")
    case.block_tables[case.block_tables < 0] = poison
    for s, c in enumerate(ctx):
        if c % 16:
            ids = case.block_tables[0, s, :, (c - 1) // 16].long()
            kc[ids, :, c % 16:, :] = float("nan")
            vc[ids, :, c % 16:] = float("nan")
    out = run(ops, gu, case, kc, vc)
    assert not torch.isnan(out).any()
    kc_c, vc_c = torch.nan_to_num(kc.cpu(), nan=0.0), torch.nan_to_num(vc.cpu(), nan=0.0)
    from oracle.attention_oracle import paged_attention_ref
    ref = paged_attention_ref(case.q[0].cpu(), kc_c, vc_c, None, case.scale, case.block_tables[0].cpu(),
                              case.context_lens.cpu(), 16)
    gu.assert_close(out, ref, "poisoned")


def test_attention_known_answers(env):
    """Properties that hold for any correct implementation, independent of the oracle."""
    ops, gu = env
    ctx = [1, 50, 257]
    case, kc, vc = gu.make_case(len(ctx), 8, 2, ctx, 16, torch.float16, seed=2, num_blocks=256)
    ops.reshape_and_cache(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
    out = torch.empty_like(case.q[0])
    # V == 1 everywhere -> output == 1
    ops.paged_attention(out, case.q[0], kc, torch.ones_like(vc), None, case.scale, case.block_tables[0],
                        case.context_lens, 16, case.max_context_len)
    assert torch.allclose(out.float(), torch.ones_like(out).float(), atol=1e-3)
    # a one-token context returns that token's V row
    ops.paged_attention(out, case.q[0], kc, vc, None, case.scale, case.block_tables[0], case.context_lens, 16,
                        case.max_context_len)
    v_new = case.v[0].view(3, 2, 128)[0]                       # seq 0, both kv heads
    assert torch.equal(out[0].view(2, 4, 128), v_new.unsqueeze(1).expand(2, 4, 128))
    # q == 0 -> uniform weights -> mean of V over the context
    ops.paged_attention(out, torch.zeros_like(case.q[0]), kc, vc, None, case.scale, case.block_tables[0],
                        case.context_lens, 16, case.max_context_len)
    from oracle.attention_oracle import gather_kv
    _, v = gather_kv(kc.cpu(), vc.cpu(), case.block_tables[0, 2, 1, :17].cpu(), 257)
    assert torch.allclose(out[2, 4].float().cpu(), v.mean(0), atol=2e-3, rtol=1e-2)


def test_attention_many_partitions_and_repeated_launches(env):
    """Thousands of small partitions, launched back to back on one workspace."""
    ops, gu = env
    gen = torch.Generator().manual_seed(5)
    ctx = torch.randint(1, 400, (192,), generator=gen).tolist()
    case, kc, vc = gu.make_case(len(ctx), 8, 8, ctx, 16, torch.float16, seed=77, num_blocks=40000)
    _, _, ref = gu.oracle_step(case, kc, vc)
    for rep in range(3):
        out = run(ops, gu, case, kc, vc, partition_size=32)
        gu.assert_close(out, ref, f"repeat {rep}")
    assert ops.device_status() == 0


@pytest.mark.parametrize("dtype,B,group,psize", [(torch.float16, 16, 1, 0), (torch.bfloat16, 16, 8, 128),
                                                 (torch.float16, 8, 2, 64), (torch.bfloat16, 32, 12, 0)])
def test_fused_decode_step_equals_two_ops(env, dtype, B, group, psize):
    """decode_attention == reshape_and_cache then paged_attention: pool and output, bit for bit."""
    ops, gu = env
    ctx = [1, 2, B, B + 1, 2 * B, 255, 256, 257, 513, 1000, 77, 16, 17, 512]
    H = 3
    case, kc, vc = gu.make_case(len(ctx), H * group, H, ctx, B, dtype, seed=50 + B, num_blocks=2048)
    kc2, vc2 = kc.clone(), vc.clone()
    expect = run(ops, gu, case, kc, vc, partition_size=psize)
    # k, v as strided views of a fused qkv buffer
    S = len(ctx)
    kv = torch.zeros(S, 2 * H * 128, dtype=dtype, device="cuda")
    kv[:, :H * 128] = case.k[0].reshape(S, -1)
    kv[:, H * 128:] = case.v[0].reshape(S, -1)
    got = torch.full_like(expect, float("nan"))
    ops.decode_attention(got, case.q[0], kv[:, :H * 128], kv[:, H * 128:], kc2, vc2, None, case.scale,
                         case.block_tables[0], case.context_lens, B, case.max_context_len, partition_size=psize)
    assert torch.equal(kc2.view(torch.int16), kc.view(torch.int16))
    assert torch.equal(vc2.view(torch.int16), vc.view(torch.int16))
    assert torch.equal(got, expect)
    _, _, ref = gu.oracle_step(case, kc, vc)
    gu.assert_close(got, ref, "fused decode step")
    assert ops.device_status() == 0


def test_attention_dirty_workspace_through_c_abi(env, built_lib):
    """Straight through the C ABI with a caller workspace full of garbage: nothing in it needs
    to be initialised."""
    import ctypes as C
    ops, gu = env
    from muxserve_b200 import _lib
    ctx = [700, 33, 300, 1]
    case, kc, vc = gu.make_case(len(ctx), 8, 2, ctx, 16, torch.float16, seed=15, num_blocks=512)
    ops.reshape_and_cache(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
    q, bt = case.q[0], case.block_tables[0]
    out = torch.full_like(q, float("nan"))
    a = _lib.AttnArgs(
        out=out.data_ptr(), q=q.data_ptr(), q_seq_stride=q.stride(0), q_head_stride=q.stride(1),
        out_seq_stride=out.stride(0), out_head_stride=out.stride(1), key_cache=kc.data_ptr(),
        value_cache=vc.data_ptr(), num_blocks=kc.shape[0], head_mapping=None, block_tables=bt.data_ptr(),
        bt_seq_stride=bt.stride(0), bt_head_stride=bt.stride(1), context_lens=case.context_lens.data_ptr(),
        scale=case.scale, num_seqs=len(ctx), num_q_heads=8, num_kv_heads=2, head_size=128, block_size=16,
        max_context_len=case.max_context_len, dtype=_lib.MUX_DTYPE_F16, partition_size=64, num_stages=0, flags=0)
    need = built_lib.mux_paged_attention_workspace_size(C.byref(a))
    ws = torch.full((need,), 0xA5, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(2):
        assert built_lib.mux_paged_attention(C.byref(a), ws.data_ptr(), need, stream) == 0
    torch.cuda.synchronize()
    _, _, ref = gu.oracle_step(case, kc, vc)
    gu.assert_close(out, ref, "dirty workspace")
    assert ops.device_status() == 0


def test_attention_edge_cases(env):
    ops, gu = env
    from muxserve_b200 import _lib
    kc = torch.randn(64, 16, 16, 8, device="cuda").half()
    vc = torch.randn(64, 128, 16, device="cuda").half()
    # empty batch
    e = torch.empty(0, 4, 128, dtype=torch.float16, device="cuda")
    ops.paged_attention(e, e, kc, vc, None, 0.1, torch.empty(0, 4, 1, dtype=torch.int32, device="cuda"),
                        torch.empty(0, dtype=torch.int32, device="cuda"), 16, 0)
    # a zero-length context yields zeros and touches no block
    q = torch.randn(2, 4, 128, device="cuda").half()
    out = torch.full_like(q, float("nan"))
    bt = torch.zeros(2, 4, 2, dtype=torch.int32, device="cuda")
    ops.paged_attention(out, q, kc, vc, None, 0.1, bt, torch.tensor([0, 20], dtype=torch.int32, device="cuda"), 16, 20)
    assert float(out[0].abs().sum()) == 0.0 and not torch.isnan(out[1]).any()
    assert ops.device_status() == 0
    # out-of-range block ids and over-long contexts are reported, not dereferenced
    bt[1, 2, 0] = 64
    ops.paged_attention(out, q, kc, vc, None, 0.1, bt, torch.tensor([5, 20], dtype=torch.int32, device="cuda"), 16, 20)
    assert ops.device_status() == _lib.MUX_DEV_BAD_BLOCK_ID
    bt[1, 2, 0] = 0
    ops.paged_attention(out, q, kc, vc, None, 0.1, bt, torch.tensor([5, 33], dtype=torch.int32, device="cuda"), 16, 32)
    assert ops.device_status() == _lib.MUX_DEV_BAD_CONTEXT
    with pytest.raises(ValueError):
        ops.paged_attention(out, q, kc, vc, None, 0.1, bt, torch.tensor([5, 20], dtype=torch.int32, device="cuda"), 16, 64)
    with pytest.raises(ValueError):
        ops.paged_attention(out, q, kc, vc, None, 0.1, bt, torch.tensor([5, 20], dtype=torch.int32, device="cuda"), 8, 20)


def test_attention_max_context_8192_gqa(env):
    """Longest configured context (8192 + 8 new tokens) with the GQA group of 8."""
    ops, gu = env
    ctx = [8200, 2048, 5000]
    case, kc, vc = gu.make_case(len(ctx), 8, 1, ctx, 16, torch.bfloat16, seed=4, num_blocks=2048, new_tokens=8)
    ops.reshape_and_cache(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
    out = torch.empty_like(case.q[0])
    for psize in (0, 512, 2048):
        ops.paged_attention(out, case.q[0], kc, vc, None, case.scale, case.block_tables[0], case.context_lens, 16,
                            case.max_context_len, partition_size=psize)
        _, _, ref = gu.oracle_step(case, kc, vc)
        gu.assert_close(out, ref, f"ctx 8200 partition {psize}")


def test_bounded_wait_runs_out_and_is_reported(env, built_lib):
    """A wait that nothing satisfies ends by itself: status bit set, kernel returns, later launches work."""
    import time
    ops, gu = env
    from muxserve_b200 import _lib
    assert ops.device_status() == 0
    t0 = time.perf_counter()
    assert built_lib.mux_selftest_wait_timeout(torch.cuda.current_stream().cuda_stream) == 0
    assert ops.device_status() == _lib.MUX_DEV_WAIT_TIMEOUT        # synchronises: the kernel has ended
    assert time.perf_counter() - t0 < 5.0
    case, kc, vc = gu.make_case(2, 2, 2, [40, 700], 16, torch.float16, seed=1, num_blocks=256)
    out = run(ops, gu, case, kc, vc)
    _, _, ref = gu.oracle_step(case, kc, vc)
    gu.assert_close(out, ref, "after a timed-out wait")
    assert ops.device_status() == 0


@pytest.mark.parametrize("Hq,H,psize", [(8, 8, 64), (16, 2, 128), (4, 4, 512)])
def test_work_list_changes_the_grid_not_the_result(env, Hq, H, psize):
    """units= (real (item, partition) pairs from host-held context lengths, -1 padded) is bit-identical to the full grid,
    for the plain op and for the fused decode step."""
    ops, gu = env
    import numpy as np
    ctx = [1, 63, 64, 65, 700, 129, 4, 1000]
    case, kc, vc = gu.make_case(len(ctx), Hq, H, ctx, 16, torch.float16, seed=55, num_blocks=2048)
    real = ops.work_units(ctx, psize, num_kv_heads=H)
    assert real.size == sum((c + psize - 1) // psize for c in ctx) * H
    padded = np.full((real.size + 37,), -1, dtype=np.int32)
    padded[:real.size] = real
    units = torch.from_numpy(padded).cuda()
    a, b = torch.empty_like(case.q[0]), torch.empty_like(case.q[0])
    ops.paged_attention(a, case.q[0], kc, vc, None, case.scale, case.block_tables[0], case.context_lens, 16,
                        case.max_context_len, partition_size=psize)
    ops.paged_attention(b, case.q[0], kc, vc, None, case.scale, case.block_tables[0], case.context_lens, 16,
                        case.max_context_len, partition_size=psize, units=units)
    assert torch.equal(a, b)
    kc1, vc1, kc2, vc2 = kc.clone(), vc.clone(), kc.clone(), vc.clone()
    ops.decode_attention(a, case.q[0], case.k[0], case.v[0], kc1, vc1, None, case.scale, case.block_tables[0],
                         case.context_lens, 16, case.max_context_len, partition_size=psize)
    ops.decode_attention(b, case.q[0], case.k[0], case.v[0], kc2, vc2, None, case.scale, case.block_tables[0],
                         case.context_lens, 16, case.max_context_len, partition_size=psize, units=units)
    assert torch.equal(a, b) and torch.equal(kc1, kc2) and torch.equal(vc1, vc2)
    assert ops.device_status() == 0
    with pytest.raises(ValueError):
        ops.paged_attention(b, case.q[0], kc, vc, None, case.scale, case.block_tables[0], case.context_lens, 16,
                            case.max_context_len, units=units)        # the list needs its partition size
