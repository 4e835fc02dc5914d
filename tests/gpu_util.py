"""Shared helpers of the GPU parity tests: build a seeded case, run the CUDA ops through the
C ABI and the CPU oracle on the same inputs."""
from __future__ import annotations

import torch

from muxserve_b200 import flexstore, ops, workloads
from oracle.attention_oracle import paged_attention_ref
from oracle.cache_write_oracle import reshape_and_cache_ref

# Tolerance of the attention output in fp16 / bf16 against the fp32 oracle.
ATOL, RTOL = 2e-3, 1e-2


def make_case(S, Hq, H, ctx, B, dtype, seed, num_blocks, new_tokens=1):
    shape = workloads.ModelShape("test", 1, Hq, H, S)
    ctx = torch.as_tensor(ctx, dtype=torch.int32)
    case = workloads.make_decode_case(shape, ctx, block_size=B, num_blocks=num_blocks, dtype=dtype,
                                      device="cuda", seed=seed, new_tokens=new_tokens)
    kc, vc = flexstore.allocate_gpu_cache(num_blocks, B, dtype, "cuda")
    workloads.fill_pool_(kc, vc, seed + 1)
    return case, kc, vc


def oracle_step(case, kc, vc, head_mapping=None, layer=0):
    """CPU: cache write then attention, on copies of the pool.  Returns (kc_cpu, vc_cpu, out fp32)."""
    kc_c, vc_c = kc.cpu().clone(), vc.cpu().clone()
    reshape_and_cache_ref(case.k[layer].cpu(), case.v[layer].cpu(), kc_c, vc_c, case.slot_mapping[:, layer, :].cpu())
    out = paged_attention_ref(case.q[layer].cpu(), kc_c, vc_c,
                              None if head_mapping is None else head_mapping.cpu(), case.scale,
                              case.block_tables[layer].cpu(), case.context_lens.cpu(), case.block_size)
    return kc_c, vc_c, out


def assert_close(out, ref, what=""):
    out = out.float().cpu()
    err = (out - ref).abs()
    tol = ATOL + RTOL * ref.abs()
    bad = err > tol
    assert not torch.isnan(out).any(), f"{what}: NaN in output"
    assert not bad.any(), f"{what}: max abs err {err.max().item():.3e}, {int(bad.sum())} elements out of tolerance"
