"""The peer-memory all-reduce's protocol and arithmetic on ONE GPU: all ranks of a world run as one cooperative
launch over local buffers (mux_tp_allreduce_emulated), and a rank that never joins makes the bounded wait run out."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(built_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from muxserve_b200 import _lib, ops, tp_comm
    return _lib, ops, tp_comm


def rank_order_sum(inputs):
    acc = torch.zeros_like(inputs[0], dtype=torch.float32)
    for x in inputs:                       # the kernel adds in rank order, in fp32
        acc += x.float()
    return acc.to(inputs[0].dtype)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("algo", [1, 2])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_emulated_world_sums_exactly_and_identically(env, world, algo, dtype):
    _lib, ops, tp_comm = env
    gen = torch.Generator(device="cuda").manual_seed(100 * world + algo)
    cap = 128 * 8192 * 2                   # the largest message of the benchmark configurations: [128, 8192] 16-bit
    buffers = None
    # a run of calls over ONE set of exchange buffers: epochs advance, slots alternate, sizes change
    for count, ctas in ((8, 0), (128 * 8192, 0), (64 * 4096, 0), (64 * 4096, 3), (1000 * 8, 7), (128 * 8192, 16), (8, 1)):
        if algo == 1 and count * 2 * world > tp_comm.buffer_size(world, cap) // 2:
            continue
        xs = [torch.randn(count, generator=gen, device="cuda").to(dtype) for _ in range(world)]
        outs, buffers = tp_comm.all_reduce_emulated(xs, cap, algo=algo, num_ctas=ctas, buffers=buffers)
        torch.cuda.synchronize()
        want = rank_order_sum(xs)
        for r, o in enumerate(outs):
            assert torch.equal(o, want), f"world {world} algo {algo} count {count}: rank {r} differs"
    assert ops.device_status() == 0


def test_emulated_in_place_and_auto_choice(env):
    _lib, ops, tp_comm = env
    gen = torch.Generator(device="cuda").manual_seed(5)
    for count in (64 * 4096, 128 * 8192):          # 512 KiB -> one-shot, 2 MiB -> two-shot
        xs = [torch.randn(count, generator=gen, device="cuda").to(torch.bfloat16) for _ in range(4)]
        want = rank_order_sum(xs)
        world = len(xs)
        nbytes = tp_comm.buffer_size(world, count * 2)
        bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        arr = lambda ts: (C.c_void_p * world)(*[t.data_ptr() for t in ts])
        for _ in range(3):                          # in place: after the first call x holds the sum, so re-seed
            ys = [x.clone() for x in xs]
            _lib.check(_lib.lib().mux_tp_allreduce_emulated(world, arr(bufs), nbytes, arr(ys), arr(ys), count,
                                                            _lib.MUX_DTYPE_BF16, 0, 0,
                                                            torch.cuda.current_stream().cuda_stream), "emulated")
            torch.cuda.synchronize()
            for y in ys:
                assert torch.equal(y, want)
    assert ops.device_status() == 0


def test_argument_errors_come_back_before_any_launch(env):
    _lib, ops, tp_comm = env
    L = _lib.lib()
    x = torch.zeros(64, dtype=torch.float16, device="cuda")
    nbytes = tp_comm.buffer_size(2, 128)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    comm = _lib.TpComm(world=2, rank=0, buffer_bytes=nbytes)
    comm.buffers[0], comm.buffers[1] = bufs[0].data_ptr(), bufs[1].data_ptr()
    s = torch.cuda.current_stream().cuda_stream
    assert L.mux_tp_allreduce(C.byref(comm), x.data_ptr(), x.data_ptr(), 12, 0, 0, 0, s) == -5     # not whole vectors
    assert L.mux_tp_allreduce(C.byref(comm), x.data_ptr(), x.data_ptr(), 64, 7, 0, 0, s) == -2     # dtype
    assert L.mux_tp_allreduce(C.byref(comm), x.data_ptr(), x.data_ptr(), 64, 0, 9, 0, s) == -6     # algo
    assert L.mux_tp_allreduce(C.byref(comm), x.data_ptr(), x.data_ptr(), 1 << 20, 0, 0, 0, s) == -13   # too large
    assert L.mux_tp_allreduce(C.byref(comm), None, x.data_ptr(), 64, 0, 0, 0, s) == -1
    comm.rank = 2
    assert L.mux_tp_allreduce(C.byref(comm), x.data_ptr(), x.data_ptr(), 64, 0, 0, 0, s) == -6
    comm.rank, comm.world = 0, 9
    assert L.mux_tp_allreduce(C.byref(comm), x.data_ptr(), x.data_ptr(), 64, 0, 0, 0, s) == -6
    assert tp_comm.lib().mux_tp_allreduce_buffer_size(1, 64) == 0
    assert ops.device_status() == 0


def test_a_rank_that_never_joins_ends_in_a_timeout_not_a_hang(env):
    """Rank 0 of a two-rank world runs alone (nobody plays rank 1, whose buffer is just local memory): its wait for
    rank 1's flag runs out after a bounded number of polls, the status word says so and the GPU stays usable."""
    import time
    _lib, ops, tp_comm = env
    L = _lib.lib()
    x = torch.ones(64, dtype=torch.float16, device="cuda")
    nbytes = tp_comm.buffer_size(2, 128)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    comm = _lib.TpComm(world=2, rank=0, buffer_bytes=nbytes)
    comm.buffers[0], comm.buffers[1] = bufs[0].data_ptr(), bufs[1].data_ptr()
    assert ops.device_status() == 0
    t0 = time.perf_counter()
    for algo in (1, 2):
        assert L.mux_tp_allreduce(C.byref(comm), x.data_ptr(), x.data_ptr(), 64, 0, algo, 1,
                                  torch.cuda.current_stream().cuda_stream) == 0
        assert ops.device_status() == _lib.MUX_DEV_WAIT_TIMEOUT          # synchronises: the kernel has ended
    assert time.perf_counter() - t0 < 30.0
    # the device still works
    ys = [torch.randn(4096, device="cuda").half() for _ in range(2)]
    outs, _ = tp_comm.all_reduce_emulated(ys)
    assert torch.equal(outs[0], rank_order_sum(ys))
    assert ops.device_status() == 0
