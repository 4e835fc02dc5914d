"""Generates ``host_traces.json`` by running the COMPILED REFERENCE allocator and step builder.

Needs the reference checkout (``python -m oracle.build_ref`` compiles its
``csrc/memory_manager.cpp`` and ``csrc/batch_scheduler.cpp`` where they lie).  The
fixture travels to machines without the checkout.

    python tests/golden/make_host_traces.py
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from host_trace import run_alloc_trace, run_engine_trace  # noqa: E402
from oracle import build_ref  # noqa: E402

ENGINE_CASES = [
    dict(seed=1, num_blocks=160, L=2, H=3, B=4, max_seq_len=64, n_requests=10, steps=60, max_new=20, free_prob=0.03),
    dict(seed=2, num_blocks=96, L=1, H=2, B=8, max_seq_len=64, n_requests=12, steps=60, max_new=24, free_prob=0.05),
    dict(seed=3, num_blocks=64, L=2, H=2, B=4, max_seq_len=48, n_requests=14, steps=70, free_prob=0.05),   # tight pool: preemption
    dict(seed=4, num_blocks=256, L=3, H=1, B=16, max_seq_len=96, n_requests=8, steps=50, max_prompt=60, max_new=30, free_prob=0.02),
]
ALLOC_CASES = [
    dict(seed=11, num_blocks=64, L=1, H=2, n_requests=40, steps=80),
    dict(seed=12, num_blocks=512, L=2, H=2, n_requests=200, steps=400, max_logical=12, free_frac=0.3),
    dict(seed=13, num_blocks=48, L=2, H=3, n_requests=60, steps=120),
]


def known_answers(KV, BS):
    """Small hand-driven sequences (every value below is what the compiled reference returns)."""
    out = {}
    kv = KV(16)
    seq = []
    for rows in ([1, 2, 0, 2, 2, 0, 3, 2, 0], [1, 1, 1, 2, 1, 1, 3, 1, 1], [3, 3, 0]):
        r = kv.allocate_batch(np.array(rows, dtype=np.int32), 1, 2)
        seq.append(dict(rows=rows, result=np.asarray(r).tolist(), new=kv.get_new_blocks_allocated()))
    seq.append(dict(free=[1, 99], freed=kv.free_batch([1, 99])))
    seq.append(dict(free=[2], freed=kv.free_batch([2])))
    for rows in ([4, 1, 0], [5, 100, 0]):
        r = kv.allocate_batch(np.array(rows, dtype=np.int32), 1, 2)
        seq.append(dict(rows=rows, result=np.asarray(r).tolist(), new=kv.get_new_blocks_allocated()))
    out["kv16_L1_H2"] = seq
    kv = KV(64)
    seq = []
    for rows in ([7, 2, 0], [7, 1, 1]):
        r = kv.allocate_batch(np.array(rows, dtype=np.int32), 2, 2)
        seq.append(dict(rows=rows, result=np.asarray(r).tolist(), new=kv.get_new_blocks_allocated()))
    seq.append(dict(free=[7], freed=kv.free_batch([7])))
    out["kv64_L2_H2"] = seq
    kv = KV(8)
    out["allocate_3_of_8"] = np.asarray(kv.allocate(3)).tolist()
    return out


def main():
    if not build_ref.build_ref():
        raise SystemExit("reference checkout not found; cannot regenerate fixtures")
    KV, BS = build_ref.load_ref()
    data = dict(
        provenance="outputs of the reference's csrc/memory_manager.cpp and csrc/batch_scheduler.cpp compiled CPU-only",
        known_answers=known_answers(KV, BS),
        engine=[dict(params=c, records=run_engine_trace(KV, BS, **c)) for c in ENGINE_CASES],
        alloc=[dict(params=c, records=run_alloc_trace(KV, **c)) for c in ALLOC_CASES],
    )
    path = Path(__file__).with_name("host_traces.json")
    path.write_text(json.dumps(data, separators=(",", ":")))
    print(path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
