"""The o_proj GEMM fused with the TP all-reduce: the tcgen05 GEMM alone against torch, and the exchange for a
whole world emulated on one GPU (one cooperative launch over local buffers) against the rank-order sum of the
rounded partial products."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env(built_lib):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from muxserve_b200 import ops, tp_comm
    return ops, tp_comm


def _close(got, want_f32, dtype):
    """Within two roundings of the tensor type of the exact fp32 product."""
    eps = 2.0 ** (-8 if dtype == torch.bfloat16 else -11)
    err = (got.float() - want_f32).abs()
    return bool((err <= 2 * eps * want_f32.abs() + 1e-3).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (128, 8192, 1024), (128, 8192, 4096), (64, 4096, 512), (1, 64, 64), (77, 640, 1984)])
def test_gemm_alone_matches_torch(env, dtype, m, n, k):
    ops, tp_comm = env
    gen = torch.Generator(device="cuda").manual_seed(m + n + k)
    a = torch.randn((m, k), generator=gen, device="cuda").to(dtype)
    w = (torch.randn((n, k), generator=gen, device="cuda") / k ** 0.5).to(dtype)
    out = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
    tp_comm.oproj(a, w, out)
    torch.cuda.synchronize()
    want = a.float() @ w.float().T
    assert not torch.isnan(out).any()
    assert _close(out, want, dtype), float((out.float() - want).abs().max())
    # strided operands: views of wider tensors
    big_a = torch.zeros((m, k + 64), dtype=dtype, device="cuda")
    big_a[:, :k] = a
    big_o = torch.zeros((m, n + 8), dtype=dtype, device="cuda")
    tp_comm.oproj(big_a[:, :k], w, big_o[:, :n])
    assert torch.equal(big_o[:, :n], out) and float(big_o[:, n:].abs().sum()) == 0.0
    # early weights: a chain of launches whose activations are each written by the kernel directly ahead
    chain = []
    for i in range(4):
        a_i = torch.empty_like(a)
        o_i = torch.full((m, n), float("nan"), dtype=dtype, device="cuda")
        a_i.copy_(a).mul_(i + 1)                      # the producer of this launch's activations
        tp_comm.oproj(a_i, w, o_i, early_w=True)
        chain.append((a_i, o_i))
    torch.cuda.synchronize()
    for a_i, o_i in chain:
        ref_i = torch.empty_like(o_i)
        tp_comm.oproj(a_i, w, ref_i)
        assert torch.equal(o_i, ref_i), "early weight fetch changed the result"
    assert ops.device_status() == 0


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("algo", [1, 2])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_emulated_world_sums_the_rounded_partials_in_rank_order(env, world, dtype, algo):
    ops, tp_comm = env
    m, n, k = 100, 512, 256
    gen = torch.Generator(device="cuda").manual_seed(world)
    buffers = None
    for call in range(3):                       # epochs advance, data areas alternate
        a_list = [torch.randn((m, k), generator=gen, device="cuda").to(dtype) for _ in range(world)]
        w_list = [(torch.randn((n, k), generator=gen, device="cuda") / k ** 0.5).to(dtype) for _ in range(world)]
        outs, buffers = tp_comm.oproj_allreduce_emulated(a_list, w_list, buffers, algo=algo)
        # every rank's partial through the same GEMM (bit-identical rounding), then the rank-order fp32 sum
        acc = torch.zeros((m, n), dtype=torch.float32, device="cuda")
        exact = torch.zeros((m, n), dtype=torch.float32, device="cuda")
        for a, w in zip(a_list, w_list):
            part = torch.empty((m, n), dtype=dtype, device="cuda")
            tp_comm.oproj(a, w, part)
            acc += part.float()
            exact += a.float() @ w.float().T
        want = acc.to(dtype)
        for r, o in enumerate(outs):
            assert torch.equal(o, want), f"world {world} call {call}: rank {r} differs"
        # and the whole thing stays near the exact fp32 product (each partial and the sum are rounded once)
        eps = 2.0 ** (-8 if dtype == torch.bfloat16 else -11)
        assert float((want.float() - exact).abs().max()) <= (world + 1) * eps * float(exact.abs().max()) + 1e-3
    assert ops.device_status() == 0


def test_argument_errors(env):
    import ctypes as C
    ops, tp_comm = env
    from muxserve_b200 import _lib
    a = torch.zeros((8, 64), dtype=torch.float16, device="cuda")
    w = torch.zeros((64, 64), dtype=torch.float16, device="cuda")
    o = torch.zeros((8, 64), dtype=torch.float16, device="cuda")
    L, s = _lib.lib(), torch.cuda.current_stream().cuda_stream
    def call(**kw):
        args = tp_comm._oproj_args(a, w, o)
        for k_, v in kw.items():
            setattr(args, k_, v)
        return L.mux_tp_oproj_allreduce(None, C.byref(args), s)
    assert call() == 0
    assert call(m=129) == -6 and call(n=96) == -6 and call(k=32) == -6 and call(dtype=5) == -2
    assert call(a_row_stride=63) == -5 and call(out_row_stride=8) == -6
    assert call(a=None) == -1 and call(flags=2) == -6 and call(flags=1) == 0
    with pytest.raises(ValueError):
        tp_comm.oproj(a, w[:, :32], o)
    assert ops.device_status() == 0
