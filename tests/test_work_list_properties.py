"""Property tests (hypothesis) of the host-built work lists that size the attention launches: whatever lengths the
scheduler holds, every real unit of work is listed exactly once, nothing else is, and the order is the one the
kernels rely on (fullest units first, so that the tail of a launch is made of short ones)."""
import numpy as np
from hypothesis import given, settings, strategies as st

from muxserve_b200 import ops

lens_lists = st.lists(st.integers(min_value=0, max_value=9000), min_size=0, max_size=40)


@settings(max_examples=150, deadline=None)
@given(lens=lens_lists, psize=st.sampled_from([16, 128, 256, 512, 2048, 4096]), heads=st.integers(1, 5))
def test_decode_work_list_is_exactly_the_set_of_real_partitions(lens, psize, heads):
    if lens and (max(lens) + psize - 1) // psize > 128:
        return                                             # the packed form refuses more than 128 partitions
    u = ops.work_units(lens, psize, num_kv_heads=heads).view(np.uint32)
    item, part = (u & 0xffffff).astype(np.int64), (u >> 24).astype(np.int64)
    want = {(s * heads + h, p) for s, n in enumerate(lens) for h in range(heads)
            for p in range(max(1, (n + psize - 1) // psize))}
    got = list(zip(item.tolist(), part.tolist()))
    assert len(got) == len(set(got)) and set(got) == want
    ctx = np.repeat(np.asarray(lens, dtype=np.int64), heads)
    tokens = np.minimum(psize, np.maximum(ctx[item] - part * psize, 0)) if len(got) else np.zeros(0)
    assert (np.diff(tokens) <= 0).all(), "units are not listed fullest first"


@settings(max_examples=100, deadline=None)
@given(lens=st.lists(st.integers(min_value=0, max_value=5000), min_size=0, max_size=20), heads=st.integers(1, 6))
def test_prompt_work_list_is_exactly_the_set_of_real_query_tiles(lens, heads):
    u = ops.prefill_work_units(lens, heads)
    seq, head, qt = u[:, 0].astype(np.int64), (u[:, 1] & 0xffff).astype(np.int64), (u[:, 1].view(np.uint32) >> 16).astype(np.int64)
    want = {(s, h, t) for s, n in enumerate(lens) for h in range(heads) for t in range((n + 127) // 128)}
    got = list(zip(seq.tolist(), head.tolist(), qt.tolist()))
    assert len(got) == len(set(got)) and set(got) == want
    if len(got):
        order = [lens[s] for s in seq.tolist()]
        assert order == sorted(order, reverse=True), "prompts are not in order of decreasing length"


@settings(max_examples=100, deadline=None)
@given(lens=st.lists(st.integers(min_value=1, max_value=8192), min_size=1, max_size=300), group=st.sampled_from([1, 2, 4, 8]))
def test_suggested_launch_is_always_a_launch_the_library_accepts(lens, group):
    import torch

    class Props:
        multi_processor_count = 148
    orig = torch.cuda.get_device_properties, torch.cuda.current_device       # no GPU here: the SM count is faked
    torch.cuda.get_device_properties, torch.cuda.current_device = (lambda *_a, **_k: Props()), (lambda: 0)
    try:
        psize, stages = ops.suggest_launch(lens, group)
    finally:
        torch.cuda.get_device_properties, torch.cuda.current_device = orig
    assert psize % 16 == 0 and 16 <= psize <= 8192
    assert stages in (0, 4, 8, 12, 16)
    assert (max(lens) + psize - 1) // psize <= 128 or psize >= 512      # the packed work list can name every partition
