"""Seeded random sweep over shapes and options of the attention ops against the fp32 oracle."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", list(range(24)))
def test_random_shapes_against_oracle(built_lib, seed):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util as gu
    from muxserve_b200 import ops
    rnd = random.Random(seed)
    B = rnd.choice([8, 16, 16, 32])
    dtype = rnd.choice([torch.float16, torch.bfloat16])
    H = rnd.randint(1, 5)
    G = rnd.choice([1, 1, 2, 3, 4, 7, 8, 9, 16])
    S = rnd.randint(1, 6)
    ctx = [rnd.choice([1, 2, B - 1, B, B + 1, rnd.randint(1, 700), rnd.randint(1, 130)]) for _ in range(S)]
    psize = rnd.choice([0, B, 2 * B, 4 * B, 128, 256, 1024])
    psize = psize // B * B
    stages = rnd.choice([0, 4, 8, 12, 16])
    fused = rnd.random() < 0.5
    interleaved = rnd.random() < 0.3
    case, kc, vc = gu.make_case(S, H * G, H, ctx, B, dtype, seed=1000 + seed, num_blocks=1024)
    hm = None
    if interleaved:
        hm = (torch.arange(H * G, dtype=torch.int32) % H).cuda()
    out = torch.full_like(case.q[0], float("nan"))
    kw = dict(partition_size=psize, num_stages=stages)
    if fused:
        ops.decode_attention(out, case.q[0], case.k[0], case.v[0], kc, vc, hm, case.scale, case.block_tables[0],
                             case.context_lens, B, case.max_context_len, **kw)
    else:
        ops.reshape_and_cache(case.k[0], case.v[0], kc, vc, case.slot_mapping[:, 0, :])
        ops.paged_attention(out, case.q[0], kc, vc, hm, case.scale, case.block_tables[0], case.context_lens, B,
                            case.max_context_len, **kw)
    kc_before, vc_before = kc.clone(), vc.clone()
    # oracle on the pool as it was before the write (oracle_step writes its own copy)
    kc_c, vc_c, ref = gu.oracle_step(case, kc, vc, head_mapping=hm)
    what = f"seed {seed}: B={B} {dtype} H={H} G={G} ctx={ctx} P={psize} st={stages} fused={fused} hm={interleaved}"
    assert torch.equal(kc_before.cpu().view(torch.int16), kc_c.view(torch.int16)), what
    assert torch.equal(vc_before.cpu().view(torch.int16), vc_c.view(torch.int16)), what
    gu.assert_close(out, ref, what)
    assert ops.device_status() == 0, what
