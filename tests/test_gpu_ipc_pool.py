"""The pool is owned by one process and used by others through CUDA IPC, as FlexStore exports it
(muxserve/flexstore/manager.py:893-911, rebuilt in muxserve/flexserver/model_loader.py:44-49): a
second process appends K/V into the owner's pool, the owner attends over it."""
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _writer(kc, vc, k, v, slots, done):
    sys.path.insert(0, str(ROOT))
    from muxserve_b200 import ops
    ops.reshape_and_cache(k, v, kc, vc, slots)         # kc / vc are IPC views of the parent's memory
    torch.cuda.synchronize()
    done.put(ops.device_status())


def test_second_process_writes_into_the_shared_pool(built_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util as gu
    from muxserve_b200 import ops
    ctx = [40, 17, 300, 64]
    case, kc, vc = gu.make_case(len(ctx), 4, 4, ctx, 16, torch.float16, seed=91, num_blocks=512)
    _, _, ref = gu.oracle_step(case, kc, vc)           # oracle: cache write + attention on CPU copies
    mpc = mp.get_context("spawn")
    done = mpc.Queue()
    slots = case.slot_mapping[:, 0, :].contiguous()
    proc = mpc.Process(target=_writer, args=(kc, vc, case.k[0], case.v[0], slots, done))
    proc.start()
    status = done.get(timeout=120)
    proc.join(timeout=60)
    assert proc.exitcode == 0 and status == 0
    out = torch.empty_like(case.q[0])
    ops.paged_attention(out, case.q[0], kc, vc, None, case.scale, case.block_tables[0], case.context_lens, 16,
                        case.max_context_len)
    gu.assert_close(out, ref, "pool written by another process")


def _metadata_writer(meta_k, meta_v, k, v, slots, done):
    sys.path.insert(0, str(ROOT))
    from muxserve_b200 import flexstore, ops
    kc, vc = flexstore.rebuild_tensor(meta_k), flexstore.rebuild_tensor(meta_v)   # as model_loader.py:44-49 does
    ops.reshape_and_cache(k, v, kc, vc, slots)
    torch.cuda.synchronize()
    done.put((ops.device_status(), tuple(kc.shape), tuple(vc.shape)))


def test_pool_exported_as_metadata_dictionaries(built_lib):
    """The service's own hand-over format: get_tensor_metadata dictionaries (manager.py:893-911) sent to the worker."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import gpu_util as gu
    from muxserve_b200 import flexstore, ops
    ctx = [33, 130, 9]
    case, kc, vc = gu.make_case(len(ctx), 2, 2, ctx, 16, torch.bfloat16, seed=92, num_blocks=256)
    _, _, ref = gu.oracle_step(case, kc, vc)
    meta_k, meta_v = flexstore.get_tensor_metadata(kc), flexstore.get_tensor_metadata(vc)
    assert set(meta_k) == {"tensor_size", "tensor_stride", "tensor_offset", "storage_cls", "dtype", "storage_device",
                           "storage_handle", "storage_size_bytes", "storage_offset_bytes", "requires_grad",
                           "ref_counter_handle", "ref_counter_offset", "event_handle", "event_sync_required"}
    mpc = mp.get_context("spawn")
    done = mpc.Queue()
    proc = mpc.Process(target=_metadata_writer,
                       args=(meta_k, meta_v, case.k[0], case.v[0], case.slot_mapping[:, 0, :].contiguous(), done))
    proc.start()
    status, kshape, vshape = done.get(timeout=120)
    proc.join(timeout=60)
    assert proc.exitcode == 0 and status == 0
    assert kshape == tuple(kc.shape) and vshape == tuple(vc.shape)
    out = torch.empty_like(case.q[0])
    ops.paged_attention(out, case.q[0], kc, vc, None, case.scale, case.block_tables[0], case.context_lens, 16,
                        case.max_context_len)
    gu.assert_close(out, ref, "pool rebuilt from metadata in another process")
