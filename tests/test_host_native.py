"""This repository's C++ allocator and step builder (through the C ABI) must match the
reference bit-exactly: golden traces, the Python oracle and the compiled reference."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from host_trace import run_alloc_trace, run_engine_trace
from oracle.host_oracle import BatchSchedulerRef, KVStorageRef
from test_host_oracle import replay_known_answers

GOLDEN = json.loads((Path(__file__).parent / "golden" / "host_traces.json").read_text())


@pytest.fixture(scope="module")
def native(built_lib):
    from muxserve_b200.batch_scheduler import BatchScheduler
    from muxserve_b200.memory_manager import KVStorage
    return KVStorage, BatchScheduler


def test_known_answers(native):
    replay_known_answers(native[0])


@pytest.mark.parametrize("case", GOLDEN["engine"], ids=lambda c: f"seed{c['params']['seed']}")
def test_engine_golden(native, case):
    got = run_engine_trace(native[0], native[1], **case["params"])
    assert got == case["records"]


@pytest.mark.parametrize("case", GOLDEN["alloc"], ids=lambda c: f"seed{c['params']['seed']}")
def test_alloc_golden(native, case):
    assert run_alloc_trace(native[0], **case["params"]) == case["records"]


def test_config1_alloc_trace_200_requests(native):
    """The 200-request alloc/free trace on a 512-block pool, bit-exact against the oracle."""
    params = dict(seed=2024, num_blocks=512, L=1, H=32, n_requests=200, steps=600, max_logical=3, free_frac=0.3)
    assert run_alloc_trace(native[0], **params) == run_alloc_trace(KVStorageRef, **params)


@pytest.mark.parametrize("seed", [7, 8, 9, 10])
def test_engine_vs_oracle_random(native, seed):
    params = dict(seed=seed, num_blocks=72 + 8 * seed, L=2, H=3, B=4, max_seq_len=80, n_requests=20, steps=150,
                  max_new=30, free_prob=0.03)
    assert run_engine_trace(native[0], native[1], **params) == run_engine_trace(KVStorageRef, BatchSchedulerRef, **params)


@pytest.mark.parametrize("seed", [201, 202])
def test_engine_vs_compiled_reference(native, ref_classes, seed):
    KV, BS = ref_classes
    params = dict(seed=seed, num_blocks=90, L=2, H=2, B=8, max_seq_len=96, n_requests=18, steps=120, max_new=40,
                  free_prob=0.03)
    assert run_engine_trace(native[0], native[1], **params) == run_engine_trace(KV, BS, **params)
    ap = dict(seed=seed, num_blocks=128, L=2, H=2, n_requests=120, steps=300, max_logical=8, free_frac=0.3)
    assert run_alloc_trace(native[0], **ap) == run_alloc_trace(KV, **ap)


def test_allocator_invariants_and_counters(native):
    KV = native[0]
    kv = KV(64)
    assert kv.check_invariants() and kv.num_free() == 64
    r = kv.allocate_batch(np.array([1, 2, 0, 2, 3, 0], dtype=np.int32), 2, 2)
    assert r[0] == 2 and len(r) == 1 + 20
    assert kv.check_invariants() and kv.num_free() == 44 and kv.num_blocks_allocated() == 20
    assert sorted(r[1:].tolist()) == list(range(44, 64))
    # exhaustion: request 3 cannot fit even if nothing is preempted -> [0], nothing changes
    r = kv.allocate_batch(np.array([3, 12, 0], dtype=np.int32), 2, 2)
    assert r.tolist() == [0] and kv.num_free() == 44
    assert kv.free_batch([1, 2, 12345]) == 20 and kv.num_free() == 64 and kv.check_invariants()
    # freed blocks are the next to be reused, request 2's last
    assert kv.free_list()[-12:].tolist() == list(range(52, 64))


def test_allocator_rejects_what_the_reference_cannot_handle(native):
    from muxserve_b200._lib import MuxError
    kv = native[0](32)
    kv.allocate_batch(np.array([1, 4, 0], dtype=np.int32), 1, 2)
    before = kv.free_list().tolist()
    # a known request asking for fewer blocks than it holds makes the reference index outside its free list
    with pytest.raises(MuxError):
        kv.allocate_batch(np.array([1, 1, 0], dtype=np.int32), 1, 2)
    assert kv.free_list().tolist() == before and kv.check_invariants()
    with pytest.raises(MuxError):
        kv.allocate(1000)


def test_scheduler_errors_and_state(native):
    from muxserve_b200._lib import MuxError
    KV, BS = native
    sched = BS(2, 3, 64, 4)
    with pytest.raises(MuxError):
        sched.try_batch([5], [])
    sched.add_request(np.arange(6, dtype=np.int32), 11, 5)
    st = sched.request_state(11)
    assert st == dict(context_len=6, num_physical_blocks=0, logical_block_idx=1, logical_block_offset=1, num_outputs=0)
    # granting more blocks than the per-request table holds is refused, not written out of bounds
    info = sched.try_batch([11], [])
    too_many = np.concatenate([[1], np.arange(17 * 6)]).astype(np.int32)
    with pytest.raises(MuxError):
        sched.get_batch_info(np.array([11, 17, 0], dtype=np.int32), too_many)
    assert info.tolist() == [11, 2, 0, 2]


def test_known_answer_metadata_trace(native):
    """BatchScheduler(L=2,H=3,maxSeq=64,B=4) + KVStorage(128): values recorded from the compiled reference."""
    KV, BS = native
    kv, sched = KV(128), BS(2, 3, 64, 4)
    sched.add_request(np.arange(6, dtype=np.int32), 11, 5)
    sched.add_request(np.arange(3, dtype=np.int32), 12, 5)
    info = sched.try_batch([11, 12], [])
    assert info.tolist() == [11, 2, 0, 12, 1, 0, 3]
    blocks = kv.allocate_batch(info[:-1], 2, 3)
    assert blocks.tolist() == [2] + list(range(110, 128))
    binfo = sched.get_batch_info(info[:-1], blocks)
    assert binfo == [9, 0, 0, 0, 2, 3, 6, 3]
    slot = torch.empty((9, 2, 3), dtype=torch.int64)
    bt = torch.empty((0, 0, 0, 0), dtype=torch.int32)
    tok, pos = torch.empty(16, dtype=torch.int32), torch.empty(16, dtype=torch.int32)
    ctx = torch.empty(0, dtype=torch.int32)
    sched.get_batch(info[:-1], blocks, tok, pos, ctx, bt, slot)
    assert slot[0].tolist() == [[440, 444, 448], [452, 456, 460]]
    assert slot[8].tolist() == [[490, 494, 498], [502, 506, 510]]
    assert tok.tolist() == [0, 1, 2, 3, 4, 5, 0, 1, 2] + [0] * 7
    # decode 1
    info = sched.try_batch([11, 12], [20, 21])
    assert info.tolist() == [11, 0, 1, 12, 0, 1, 0]
    blocks = np.array([2], dtype=np.int32)
    binfo = sched.get_batch_info(info[:-1], blocks)
    assert binfo == [2, 2, 7, 2, 2, 3]
    slot = torch.empty((2, 2, 3), dtype=torch.int64)
    bt = torch.empty((2, 2, 2, 3), dtype=torch.int32)
    tok, pos = torch.empty(8, dtype=torch.int32), torch.empty(8, dtype=torch.int32)
    ctx = torch.empty(2, dtype=torch.int32)
    sched.get_batch(info[:-1], blocks, tok, pos, ctx, bt, slot)
    assert pos[:2].tolist() == [6, 3] and ctx.tolist() == [7, 4]
    assert slot[0].tolist() == [[466, 470, 474], [478, 482, 486]]
    assert slot[1].tolist() == [[491, 495, 499], [503, 507, 511]]
    layered = bt.permute(2, 0, 3, 1)          # [L, S, H, blk] as llm_runtime.py:327
    assert layered[0, 0].tolist() == [[110, 116], [111, 117], [112, 118]]
    assert layered[1, 0].tolist() == [[113, 119], [114, 120], [115, 121]]
    assert layered[0, 1, :, 0].tolist() == [122, 123, 124] and layered[1, 1, :, 0].tolist() == [125, 126, 127]
    assert layered[:, 1, :, 1].abs().sum() == 0   # padding is zero here (uninitialised in the reference)
    # decode 2: request 12 crosses a block boundary
    info = sched.try_batch([11, 12], [22, 23])
    assert info.tolist() == [11, 0, 1, 12, 1, 1, 1]
    blocks = kv.allocate_batch(info[:-1], 2, 3)
    assert blocks.tolist() == [2] + list(range(104, 110))
    sched.get_batch_info(info[:-1], blocks)
    bt2 = torch.empty((2, 2, 2, 2, 3)[1:], dtype=torch.int32)
    bt_l = torch.empty((2, 2, 3, 2), dtype=torch.int32)
    sched.get_batch_decode_layered(info[:-1], blocks, tok, pos, ctx, bt_l, slot)
    assert slot[1].tolist() == [[416, 420, 424], [428, 432, 436]]
    assert bt_l[0, 1].tolist() == [[122, 104], [123, 105], [124, 106]]
    assert bt_l[1, 0].tolist() == [[113, 119], [114, 120], [115, 121]]
    del bt2
