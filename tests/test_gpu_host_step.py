"""HostDecodeStep (host buffers -> device -> host, per layer) against the ops called directly, with and without a work list."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("use_units", [False, True])
def test_host_decode_step_matches_direct_ops(built_lib, use_units):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util as gu
    from muxserve_b200 import ops, workloads
    from muxserve_b200.host_step import HostDecodeStep
    ctx = [40, 700, 17, 513, 64, 1]
    L, Hq, H, B, psize = 3, 8, 4, 16, 256
    shape = workloads.ModelShape("t", L, Hq, H, len(ctx))
    ctx_t = torch.tensor(ctx, dtype=torch.int32)
    case = workloads.make_decode_case(shape, ctx_t, block_size=B, num_blocks=4096, dtype=torch.float16, device="cuda",
                                      seed=3)
    from muxserve_b200 import flexstore
    kc, vc = flexstore.allocate_gpu_cache(4096, B, torch.float16, "cuda")
    workloads.fill_pool_(kc, vc, 4)
    kc2, vc2 = kc.clone(), vc.clone()
    # direct: fused decode step per layer
    want = torch.empty((L, len(ctx), Hq, 128), dtype=torch.float16, device="cuda")
    for l in range(L):
        ops.decode_attention(want[l], case.q[l], case.k[l], case.v[l], kc, vc, None, case.scale, case.block_tables[l],
                             case.context_lens, B, case.max_context_len, partition_size=psize)
    units_host, cap = None, 0
    if use_units:
        real = ops.work_units(ctx, psize, num_kv_heads=H)
        cap = (real.size + 63) // 64 * 64
        padded = np.full((cap,), -1, dtype=np.int32)
        padded[:real.size] = real
        units_host = torch.from_numpy(padded).pin_memory()
    hs = HostDecodeStep(shape, B, torch.float16, kc2, vc2, case.block_tables.shape[-1], partition_size=psize,
                        units_capacity=cap)
    pin = lambda t: t.cpu().pin_memory()
    out_h = torch.empty((L, len(ctx), Hq, 128), dtype=torch.float16).pin_memory()
    hs.run(pin(case.q), pin(case.k), pin(case.v), pin(case.block_tables.clamp_min(0)), pin(case.slot_mapping),
           pin(case.context_lens), out_h, case.max_context_len, units_host=units_host)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert torch.equal(out_h, want.cpu())
    assert torch.equal(kc2, kc) and torch.equal(vc2, vc)
    assert hs.h2d_bytes > 0 and hs.d2h_bytes == out_h.numel() * 2
