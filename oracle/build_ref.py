"""Compiles the reference's own host C++ (allocator, step builder) into ``oracle/_ref``.

TEST INFRASTRUCTURE ONLY.  The two files are compiled where they lie in the
reference checkout (they are never copied into this repository) with
``torch.utils.cpp_extension.load``; the resulting pybind modules are written to
``oracle/_ref/`` (git-ignored).  ``load_ref()`` imports the prebuilt modules on a
machine where the checkout is absent.

    python -m oracle.build_ref [/path/to/reference]

Without an argument the checkout is looked for where ``MUXSERVE_REFERENCE`` points, else in a directory
``reference`` beside this repository.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"
DEFAULT_REFERENCE = Path(os.environ.get("MUXSERVE_REFERENCE") or Path(__file__).resolve().parents[2] / "reference")
MODULES = {"ref_memory_manager": "csrc/memory_manager.cpp", "ref_batch_scheduler": "csrc/batch_scheduler.cpp"}


def build_ref(reference: Path = DEFAULT_REFERENCE, verbose: bool = False) -> bool:
    """Builds both modules; returns False when the reference checkout is absent."""
    if not (reference / "csrc" / "memory_manager.cpp").exists():
        return False
    from torch.utils.cpp_extension import load
    REF_DIR.mkdir(exist_ok=True)
    for name, rel in MODULES.items():
        load(name=name, sources=[str(reference / rel)], extra_cflags=["-O2", "-std=c++17"],
             build_directory=str(REF_DIR), verbose=verbose)
    return True


def _import(name: str):
    path = REF_DIR / f"{name}.so"
    if not path.exists():
        return None
    import torch  # noqa: F401  (libtorch symbols must be loaded first)
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_ref():
    """Returns (KVStorage, BatchScheduler) of the compiled reference, or None if not built."""
    mm, bs = _import("ref_memory_manager"), _import("ref_batch_scheduler")
    if mm is None or bs is None:
        return None
    return mm.KVStorage, bs.BatchScheduler


if __name__ == "__main__":
    ref = Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_REFERENCE
    ok = build_ref(ref, verbose=True)
    print("built" if ok else f"reference checkout not found at {ref}", REF_DIR)
