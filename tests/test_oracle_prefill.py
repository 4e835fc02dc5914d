"""CPU: the prompt-attention oracle against an element-wise restatement, and the prompt slot helper."""
import math

import torch

from muxserve_b200 import workloads
from oracle.prefill_oracle import prefill_attention_ref


def _brute(q, k, v, lens, scale):
    T, Hq, D = q.shape
    group = Hq // k.shape[1]
    out = torch.zeros((T, Hq, D), dtype=torch.float64)
    start = 0
    for n in lens:
        for t in range(n):
            for h in range(Hq):
                kv = h // group
                logits = [float(q[start + t, h].double() @ k[start + u, kv].double()) * scale for u in range(t + 1)]
                m = max(logits)
                w = [math.exp(x - m) for x in logits]
                z = sum(w)
                acc = torch.zeros(D, dtype=torch.float64)
                for u in range(t + 1):
                    acc += (w[u] / z) * v[start + u, kv].double()
                out[start + t, h] = acc
        start += n
    return out


def test_oracle_matches_elementwise_restatement():
    gen = torch.Generator().manual_seed(0)
    lens = [1, 7, 0, 12]
    T = sum(lens)
    q = torch.randn((T, 4, 128), generator=gen)
    k = torch.randn((T, 2, 128), generator=gen)
    v = torch.randn((T, 2, 128), generator=gen)
    ref = prefill_attention_ref(q, k, v, lens, 0.09)
    assert torch.allclose(ref.double(), _brute(q, k, v, lens, 0.09), atol=1e-5, rtol=1e-5)


def test_first_token_of_every_prompt_returns_its_own_value():
    gen = torch.Generator().manual_seed(1)
    lens = [3, 5]
    q = torch.randn((8, 2, 128), generator=gen)
    k = torch.randn((8, 2, 128), generator=gen)
    v = torch.randn((8, 2, 128), generator=gen)
    ref = prefill_attention_ref(q, k, v, lens, 0.1)
    assert torch.allclose(ref[0], v[0]) and torch.allclose(ref[3], v[3])


def test_prompt_slots_follow_the_block_lists():
    lens = torch.tensor([5, 33, 16], dtype=torch.int32)
    tables, _ = workloads.scatter_block_tables(lens, 2, 3, 16, torch.randperm(200, generator=torch.Generator().manual_seed(2)))
    slots = workloads.prompt_slots(tables, lens, 16)
    assert slots.shape == (54, 2, 3) and slots.dtype == torch.int64
    row = 0
    for s, n in enumerate(lens.tolist()):
        for t in range(n):
            want = tables[:, s, :, t // 16].long() * 16 + t % 16
            assert torch.equal(slots[row], want)
            row += 1
    # the last token of every prompt is the slot the decode path appends after (same formula, new_tokens = 1)
    last = workloads.last_token_slots(tables, lens, 16, 1)
    assert torch.equal(slots[torch.tensor([4, 37, 53])], last)
    assert workloads.prefill_flops([2, 3], 4) == 4 * 128 * 4 * (3 + 6)
