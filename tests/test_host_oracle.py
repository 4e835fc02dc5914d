"""Pins the Python restatement of the allocator / step builder (oracle/host_oracle.py)
against the golden traces recorded from the compiled reference and, when it is
available, against the compiled reference itself on fresh seeds."""
import json
from pathlib import Path

import numpy as np
import pytest

from host_trace import run_alloc_trace, run_engine_trace
from oracle.host_oracle import BatchSchedulerRef, KVStorageRef

GOLDEN = json.loads((Path(__file__).parent / "golden" / "host_traces.json").read_text())


def replay_known_answers(KV):
    ka = GOLDEN["known_answers"]
    for name, (nblocks, L, H) in (("kv16_L1_H2", (16, 1, 2)), ("kv64_L2_H2", (64, 2, 2))):
        kv = KV(nblocks)
        for step in ka[name]:
            if "rows" in step:
                got = np.asarray(kv.allocate_batch(np.array(step["rows"], dtype=np.int32), L, H)).tolist()
                assert got == step["result"], (name, step)
                assert kv.get_new_blocks_allocated() == step["new"], (name, step)
            else:
                assert kv.free_batch(step["free"]) == step["freed"], (name, step)
    assert np.asarray(KV(8).allocate(3)).tolist() == ka["allocate_3_of_8"]


def test_oracle_known_answers():
    replay_known_answers(KVStorageRef)


@pytest.mark.parametrize("case", GOLDEN["engine"], ids=lambda c: f"seed{c['params']['seed']}")
def test_oracle_engine_golden(case):
    got = run_engine_trace(KVStorageRef, BatchSchedulerRef, **case["params"])
    assert got == case["records"]


@pytest.mark.parametrize("case", GOLDEN["alloc"], ids=lambda c: f"seed{c['params']['seed']}")
def test_oracle_alloc_golden(case):
    assert run_alloc_trace(KVStorageRef, **case["params"]) == case["records"]


@pytest.mark.parametrize("seed", [101, 102, 103])
def test_oracle_vs_compiled_reference(ref_classes, seed):
    KV, BS = ref_classes
    params = dict(seed=seed, num_blocks=80, L=2, H=2, B=4, max_seq_len=64, n_requests=16, steps=80, free_prob=0.04)
    assert run_engine_trace(KVStorageRef, BatchSchedulerRef, **params) == run_engine_trace(KV, BS, **params)
    ap = dict(seed=seed, num_blocks=96, L=2, H=3, n_requests=80, steps=200, max_logical=6, free_frac=0.35)
    assert run_alloc_trace(KVStorageRef, **ap) == run_alloc_trace(KV, **ap)
