"""The allocation-free attention entry point (`mux_paged_attention_static_scratch`).

It exists for hosts that must not call cudaMalloc while serving (memory budget fixed at start-up,
GPU shared with other processes, allocation calls not permitted on their path): the flash-decoding
scratch is a fixed array inside the library instead of a caller buffer.  The checks: called straight
through the C ABI it gives the same output as the ordinary entry point, twice in a row on different
inputs (the second call finds the first call's leftovers in the shared array), and a problem whose
scratch would not fit is refused with MUX_ERR_TOO_LARGE.  This file sorts last on purpose.
"""
import ctypes as C

import pytest
import torch


def _args(_lib, out, q, kc, vc, bt, ctx, scale, max_ctx, psize):
    S, Hq, _ = q.shape
    return _lib.AttnArgs(
        out=out.data_ptr(), q=q.data_ptr(), q_seq_stride=q.stride(0), q_head_stride=q.stride(1),
        out_seq_stride=out.stride(0), out_head_stride=out.stride(1),
        key_cache=kc.data_ptr(), value_cache=vc.data_ptr(), num_blocks=kc.shape[0], head_mapping=None,
        block_tables=bt.data_ptr(), bt_seq_stride=bt.stride(0), bt_head_stride=bt.stride(1),
        context_lens=ctx.data_ptr(), scale=scale, num_seqs=S, num_q_heads=Hq, num_kv_heads=bt.shape[1],
        seq_rows=None, head_size=128, block_size=kc.shape[2], max_context_len=max_ctx,
        dtype=_lib.MUX_DTYPE_F16 if q.dtype == torch.float16 else _lib.MUX_DTYPE_BF16,
        partition_size=psize, num_stages=0)


@pytest.mark.gpu
def test_static_scratch_matches_caller_workspace_twice(built_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util as gu
    from muxserve_b200 import _lib, ops
    stream = torch.cuda.current_stream().cuda_stream
    # second case: other lengths and fewer partitions, so stale partials of the first call sit in the array
    for n, (ctx, dtype, group, psize) in enumerate([([1500, 40, 700, 2047, 513, 64], torch.float16, 1, 128),
                                                     ([300, 1100, 90, 258], torch.bfloat16, 4, 256)]):
        case, kc, vc = gu.make_case(len(ctx), 3 * group, 3, ctx, 16, dtype, seed=60 + n, num_blocks=2048)
        ops.reshape_and_cache(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
        expect = torch.empty_like(case.q[0])
        ops.paged_attention(expect, case.q[0], kc, vc, None, case.scale, case.block_tables[0], case.context_lens,
                            16, case.max_context_len, partition_size=psize)
        got = torch.full_like(expect, float("nan"))
        a = _args(_lib, got, case.q[0], kc, vc, case.block_tables[0], case.context_lens, case.scale,
                  case.max_context_len, psize)
        assert built_lib.mux_paged_attention_workspace_size(C.byref(a)) > 0      # the scratch really is in use
        rc = built_lib.mux_paged_attention_static_scratch(C.byref(a), stream)
        assert rc == 0, built_lib.mux_strerror(rc)
        torch.cuda.synchronize()
        gu.assert_close(got, expect.float().cpu(), f"static scratch, call {n + 1}")
        _, _, ref = gu.oracle_step(case, kc, vc)
        gu.assert_close(got, ref, f"static scratch vs oracle, call {n + 1}")
    assert ops.device_status() == 0


def test_static_scratch_refuses_what_does_not_fit(built_lib):
    """Checked on the host before anything is launched, so this needs no GPU."""
    from muxserve_b200 import _lib
    a = _lib.AttnArgs(dtype=0, head_size=128, block_size=16, num_seqs=4096, num_q_heads=32, num_kv_heads=32,
                      num_blocks=1 << 20, max_context_len=8192, partition_size=512)
    for f in ("out", "q", "key_cache", "value_cache", "block_tables", "context_lens"):
        setattr(a, f, 0x1000)
    assert built_lib.mux_paged_attention_workspace_size(C.byref(a)) > (16 << 20)
    rc = built_lib.mux_paged_attention_static_scratch(C.byref(a), None)
    assert rc == -13 and b"capacity" in built_lib.mux_strerror(rc)
    assert built_lib.mux_paged_attention_static_scratch(None, None) == -1
