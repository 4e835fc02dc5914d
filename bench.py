#!/usr/bin/env python
"""Benchmark of the decode attention path (reshape_and_cache + paged_attention over all layers).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c3|c4|c5|prefill] [--impl native|reference]

A step is one decode step of the path: for every layer one cache write of the new
tokens and one paged attention over the sequence batch.  Prints ONE JSON line.
``--impl reference`` times the CPU oracle (the reference has no CPU implementation
of these ops; its kernels live in an un-vendored fork) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = ("paged decode-attn tokens/s (reshape_and_cache + paged_attention over all layers; "
          "achieved HBM GB/s and fraction of peak in `roofline`)")

# name -> global (un-sharded) shape.  Workload text follows the benchmark configurations.
WORKLOADS = {
    "c2": dict(desc="LLaMA-7B shape fp16 decode: 32 layers, 32 heads (MHA), head_dim 128, batch 64, "
                    "context_lens U[128,2048], block_size 16, 1 new token/seq",
               L=32, Hq=32, H=32, S=64, lo=128, hi=2048, dtype="f16", new_tokens=1),
    "c4": dict(desc="LLaMA-65B shape bf16 decode: 80 layers, 64 heads (MHA), batch 128, context_lens U[512,4096], "
                    "block_size 16",
               L=80, Hq=64, H=64, S=128, lo=512, hi=4096, dtype="bf16", new_tokens=1),
    "c5": dict(desc="Llama-2-70B shape bf16 GQA decode: 80 layers, 64 q heads / 8 kv heads, batch 256, "
                    "context_lens U[2048,8192], block_size 16, 8 new tokens/seq",
               L=80, Hq=64, H=8, S=256, lo=2048, hi=8192, dtype="bf16", new_tokens=8),
}
# config 3: three colocated LLaMA models sharing one pool on 4 GPUs (TP=4 -> local heads 8/10/13), batches 48/24/12
C3_MODELS = [("llama-7b", 32, 32, 48), ("llama-13b", 40, 40, 24), ("llama-30b", 60, 52, 12)]   # name, layers, heads, batch
C3_TP = 4
C3_DESC = ("three colocated LLaMA models (7B/13B/30B: 32/40/52 heads, 32/40/60 layers, head_dim 128, fp16) sharing one "
           "head-granular pool, TP=4 share of one GPU (local heads 8/10/13), batches 48/24/12, context_lens lognormal "
           "(median 256, sigma 1.0) clipped to [16,4096], block lists interleaved randomly, one fused launch per layer")
BLOCK = 16
DTYPES = {"f16": torch.float16, "bf16": torch.bfloat16}
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the fused decode kernel, from the ncu capture
# summarised in profiles/paged_attn_kernel_c2_fused_small.md (same per-launch work as a layer of c2, smaller pool).
NCU_DRAM_BYTES_PER_LAUNCH = {"c2": 1204193000 + 14504960}


_JSON_OUT = None


def claim_stdout():
    """Keeps the process's stdout for the ONE JSON line: native libraries write there too (NCCL prints its
    version banner to fd 1), so fd 1 is pointed at stderr and the line goes out through a saved duplicate."""
    global _JSON_OUT
    if _JSON_OUT is None:
        sys.stdout.flush()
        _JSON_OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line: dict) -> None:
    out = _JSON_OUT if _JSON_OUT is not None else sys.stdout
    print(json.dumps(line), file=out, flush=True)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["c3", "prefill"], default="c2")
    ap.add_argument("--pool-frac", type=float, default=0.6, help="fraction of HBM given to the KV pool")
    ap.add_argument("--partition-size", type=int, default=0)
    ap.add_argument("--num-stages", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (small profiler captures)")
    ap.add_argument("--batch", type=int, default=0, help="override the batch size (small profiler captures)")
    ap.add_argument("--prompt-len", type=int, default=0, help="prefill workload: every prompt has this length")
    ap.add_argument("--heads", type=int, default=0, help="prefill workload: override the head count (small captures)")
    ap.add_argument("--seed", type=int, default=20240531)
    ap.add_argument("--eager", action="store_true",
                    help="time Python-issued launches instead of replaying a CUDA graph of one step")
    ap.add_argument("--two-op", action="store_true",
                    help="time reshape_and_cache + paged_attention as separate calls instead of the fused decode step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-tp", action="store_true", help="skip the tensor-parallel leg at N > 1")
    ap.add_argument("--no-units", action="store_true",
                    help="launch one CTA per (item, partition index) instead of the host's work list")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="target CPU time of the cpu_baseline sample")
    return ap.parse_args()


def hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback 6650 GB/s (MEASURED_PEAKS.json absent)"


# ----------------------------------------------------------------------------- clocks
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (read-only NVML)."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost"}

    def __init__(self, device_index: int, period_s: float = 0.01):
        super().__init__(daemon=True)
        self.period = period_s
        self.samples, self.reason_bits, self.sm_max = [], 0, None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception as exc:  # NVML missing: fall back to one nvidia-smi query per sample
            self.err = repr(exc)
            self.dev = device_index

    def _sample(self):
        if self.ok:
            nv = self.nv
            mhz = int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
            try:
                bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
            except Exception:
                bits = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
            return mhz, bits
        out = subprocess.run(["nvidia-smi", "-i", str(self.dev), "--query-gpu=clocks.sm,clocks.max.sm,"
                              "clocks_event_reasons.active", "--format=csv,noheader,nounits"],
                             capture_output=True, text=True, timeout=5).stdout.strip().split(",")
        self.sm_max = int(out[1])
        return int(out[0]), int(out[2], 16)

    def run(self):
        while not self._stop_evt.is_set():
            try:
                mhz, bits = self._sample()
                self.samples.append(mhz)
                self.reason_bits |= bits
            except Exception:
                pass
            self._stop_evt.wait(self.period)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=5)
        s = sorted(self.samples)
        reasons = [name for bit, name in self.REASONS.items() if self.reason_bits & bit]
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.sm_max, "reasons": reasons,
                "samples": len(s)}


# ----------------------------------------------------------------------------- CPU oracle legs
def compact_layer_to_cpu(case, kc, vc, layer):
    """Copies the blocks one layer touches into a small CPU pool with renumbered ids."""
    bt = case.block_tables[layer]
    valid = bt >= 0
    ids = bt[valid].long()
    remap = torch.zeros_like(bt)
    remap[valid] = torch.arange(ids.numel(), dtype=torch.int32, device=bt.device)
    return kc[ids].cpu(), vc[ids].cpu(), remap.cpu()


def cpu_attention_step(q, k_new, v_new, kc, vc, bt, slots, ctx, scale, seqs):
    """One layer of the path on the CPU oracle for the first `seqs` sequences."""
    from oracle.attention_oracle import paged_attention_ref_batched
    from oracle.cache_write_oracle import reshape_and_cache_ref
    T_per = k_new.shape[0] // q.shape[0]
    reshape_and_cache_ref(k_new[:seqs * T_per], v_new[:seqs * T_per], kc, vc, slots[:seqs * T_per])
    return paged_attention_ref_batched(q[:seqs], kc, vc, scale, bt[:seqs], ctx[:seqs], BLOCK)


def time_cpu_sample(q, k_new, v_new, kc, vc, bt, slots, ctx, scale, budget_s, reps_max=500):
    """Times the oracle on all sequences of one layer, repeating until about `budget_s` seconds are spent."""
    S = q.shape[0]
    times = []
    t_all = time.perf_counter()
    while len(times) < reps_max and (not times or time.perf_counter() - t_all < budget_s):
        t0 = time.perf_counter()
        cpu_attention_step(q, k_new, v_new, kc, vc, bt, slots, ctx, scale, S)
        times.append(time.perf_counter() - t0)
    return sum(times) / len(times), len(times)


def synth_cpu_layer(w, seed, seqs=None):
    """A compact CPU-only layer of workload `w` (no GPU involved): pool = exactly the blocks it needs, shuffled."""
    from muxserve_b200 import workloads
    gen = torch.Generator().manual_seed(seed)
    S = w["S"] if seqs is None else min(seqs, w["S"])
    ctx = workloads.uniform_context_lens(w["S"], w["lo"], w["hi"], gen)[:S]
    nblk = workloads.blocks_needed(ctx, 1, w["H"], BLOCK)
    perm = torch.randperm(nblk, generator=gen)
    bt, _ = workloads.scatter_block_tables(ctx, 1, w["H"], BLOCK, perm)
    slots = workloads.last_token_slots(bt, ctx, BLOCK, w["new_tokens"])[:, 0, :]
    dt = DTYPES[w["dtype"]]
    kc = torch.randn((nblk, 16, BLOCK, 8), generator=gen).to(dt)
    vc = torch.randn((nblk, 128, BLOCK), generator=gen).to(dt)
    q = torch.randn((S, w["Hq"], 128), generator=gen).to(dt)
    k = torch.randn((S * w["new_tokens"], w["H"], 128), generator=gen).to(dt)
    v = torch.randn((S * w["new_tokens"], w["H"], 128), generator=gen).to(dt)
    return q, k, v, kc, vc, bt[0].clamp_min(0), slots, ctx


def run_reference(args):
    """CPU arm: the oracle on all host threads; a step is one layer of the workload over a bounded
    number of sequences, scaled to the full layer count."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    # calibrate on 2 sequences, then size the per-step sample so that the whole run stays near 2 minutes
    q, k, v, kc, vc, bt, slots, ctx = synth_cpu_layer(w, args.seed, seqs=2)
    t0 = time.perf_counter()
    cpu_attention_step(q, k, v, kc, vc, bt, slots, ctx, 128 ** -0.5, 2)
    t_seq = (time.perf_counter() - t0) / 2
    budget = 120.0
    seqs = int(max(1, min(w["S"], budget / max(1e-6, (args.steps + args.warmup) * t_seq))))
    q, k, v, kc, vc, bt, slots, ctx = synth_cpu_layer(w, args.seed, seqs=seqs)
    for _ in range(args.warmup):
        cpu_attention_step(q, k, v, kc, vc, bt, slots, ctx, 128 ** -0.5, seqs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_attention_step(q, k, v, kc, vc, bt, slots, ctx, 128 ** -0.5, seqs)
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    tokens_per_s = seqs / (dt * w["L"])            # one layer timed; a decode step runs L of them
    sample = (f"each step = 1 of {w['L']} layers over {seqs} of {w['S']} sequences on the CPU oracle "
              f"(fp32 PyTorch gather attention + scatter cache write); tokens/s = sequences / (step time x {w['L']} layers)")
    line = {
        "impl": "reference", "metric": METRIC, "value": tokens_per_s, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3 * w["L"] * (w["S"] / seqs),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": f"{args.workload}: {w['desc']}", "block_size": BLOCK, "seed": args.seed},
        "cpu_baseline": {"value": tokens_per_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tokens_per_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference ships no CPU (or CUDA) source for these ops; this arm is the oracle port",
    }
    emit(line)


# ----------------------------------------------------------------------------- native arm
def run_native(args):
    import torch.distributed as dist
    from muxserve_b200 import flexstore, ops, workloads
    from muxserve_b200.host_step import HostDecodeStep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl native needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w = dict(WORKLOADS[args.workload])
    if args.layers > 0:
        w["L"] = args.layers
    if args.batch > 0:
        w["S"] = args.batch
    dt = DTYPES[w["dtype"]]
    L, S, Hq, H, NT = w["L"], w["S"], w["Hq"], w["H"], w["new_tokens"]

    # ---- pool sized as FlexStore does, a fraction of HBM ----
    total_mem = torch.cuda.get_device_properties(dev).total_memory
    num_blocks = flexstore.get_num_gpu_blocks(total_mem, args.pool_frac, BLOCK)
    kc, vc = flexstore.allocate_gpu_cache(num_blocks, BLOCK, dt, dev)
    workloads.fill_pool_(kc, vc, args.seed + 17 * rank)

    # every replica gets the same context lengths (the same work per GPU, which is what weak scaling
    # compares); pool contents, block scatter and q/k/v differ by rank
    gen = torch.Generator().manual_seed(args.seed)
    ctx = workloads.uniform_context_lens(S, w["lo"], w["hi"], gen)
    per_layer = workloads.blocks_needed(ctx, 1, H, BLOCK)
    L_res = max(1, min(L, int(num_blocks * 0.98) // per_layer))     # distinct resident layers
    shape = workloads.ModelShape(args.workload, L_res, Hq, H, S)
    case = workloads.make_decode_case(shape, ctx, block_size=BLOCK, num_blocks=num_blocks, dtype=dt, device=dev,
                                      seed=args.seed + 1000 * rank, new_tokens=NT)
    ctx_list = ctx.tolist()
    attn_bytes = workloads.attention_bytes(ctx_list, Hq, H, BLOCK)
    cw_bytes = workloads.cache_write_bytes(S * NT, H)
    out = torch.empty((S, Hq, 128), dtype=dt, device=dev)
    psize, nst = args.partition_size, args.num_stages
    # Work list from the context lengths the host scheduler holds (it uploads them every step): the real
    # (sequence, kv head, partition) triples, fullest first, padded to a fixed length for the captured graph.
    units = units_host = None
    if not args.no_units:
        psize = psize or ops.suggest_partition_size(S * H, Hq // H, dev)
        import numpy as np
        real = ops.work_units(ctx_list, psize, num_kv_heads=H)
        cap = (real.size + 127) // 128 * 128
        units_np = np.full((cap,), -1, dtype=np.int32)
        units_np[:real.size] = real
        units_host = torch.from_numpy(units_np).pin_memory()
        units = units_host.to(dev)

    fused = NT == 1 and not args.two_op

    def layer(l, ev=None, fuse=fused):
        r = l % L_res
        if fuse:      # one launch: append the new token and attend
            if ev is not None:
                ev[0].record()
            ops.decode_attention(out, case.q[r], case.k[r], case.v[r], kc, vc, None, case.scale, case.block_tables[r],
                                 case.context_lens, BLOCK, case.max_context_len, partition_size=psize,
                                 num_stages=nst, units=units)
        else:
            ops.reshape_and_cache(case.k[r], case.v[r], kc, vc, case.slot_mapping[:, r, :])
            if ev is not None:
                ev[0].record()
            ops.paged_attention(out, case.q[r], kc, vc, None, case.scale, case.block_tables[r], case.context_lens,
                                BLOCK, case.max_context_len, partition_size=psize, num_stages=nst, units=units)
        if ev is not None:
            ev[1].record()

    def step(events=None, fuse=fused):
        for l in range(L):
            layer(l, None if events is None else events[l], fuse)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident leg ----
    for _ in range(max(3, args.warmup)):
        step()
    status_warm = ops.device_status()
    events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(L)]
              for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    graph = None
    if not args.eager:
        try:
            torch.cuda.synchronize()
            l0 = ops.launch_count
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            per_step_launches = ops.launch_count - l0
            graph.replay()
            torch.cuda.synchronize()
        except Exception as exc:      # capture refused: time the Python-issued launches instead
            print(f"bench: CUDA graph capture failed ({type(exc).__name__}: {exc}); timing eager launches",
                  file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    barrier()
    sampler.start()
    launches0 = ops.launch_count
    e0.record()
    for i in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            step(events[i])
    e1.record()
    gpu_launches = ops.launch_count - launches0 if graph is None else per_step_launches * args.steps
    barrier()
    clocks = sampler.stop()
    ms_local = e0.elapsed_time(e1) / args.steps
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps
    ms_ranks = [ms_local]
    if world > 1:          # every rank's own time, to tell a slow GPU from a slow path
        t = torch.tensor([ms_local], dtype=torch.float64, device=dev)
        gathered = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(gathered, t)
        ms_ranks = [float(g.item()) for g in gathered]
    if graph is not None:
        # the kernel-level span cannot be bracketed inside a graph: a second, eager pass of the same
        # steps with CUDA events around every attention launch gives it
        barrier()
        e0.record()
        for i in range(args.steps):
            step(events[i])
        e1.record()
        barrier()
        ms_eager = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    else:
        ms_eager = ms_step
    eager_span_ms = sum(a.elapsed_time(b) for evs in events for a, b in evs) / (args.steps * L)
    # Under graph replay with the fused step a layer IS one attention launch (+ its merge kernel), so
    # step time / layers bounds the launch duration from above, gaps included, without the extra
    # serialisation that event records between the launches of the eager pass introduce.
    attn_ms = ms_step / L if (graph is not None and fused) else eager_span_ms
    status = ops.device_status() | status_warm

    # ---- the same step with the two reference-signature ops (separate cache-write launch) ----
    two_op = None
    if fused:
        for _ in range(3):
            step(fuse=False)
        run2 = lambda: step(fuse=False)
        if graph is not None:
            try:
                torch.cuda.synchronize()
                g2 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g2):
                    step(fuse=False)
                g2.replay()
                torch.cuda.synchronize()
                run2 = g2.replay
            except Exception:
                torch.cuda.synchronize()
        barrier()
        e0.record()
        for _ in range(args.steps):
            run2()
        e1.record()
        barrier()
        ms2 = max_over_ranks(e0.elapsed_time(e1)) / args.steps
        two_op = {"ms_per_step": ms2, "tokens_per_s": world * S / (ms2 * 1e-3),
                  "whole_path_gbs": (attn_bytes + cw_bytes) * L / (ms2 * 1e-3) / 1e9,
                  "note": "reshape_and_cache and paged_attention as two calls per layer"}

    # ---- end-to-end leg: host buffers, copies inside the timed region ----
    e2e = None
    if not args.no_e2e:
        hs = HostDecodeStep(workloads.ModelShape(args.workload, L, Hq, H, S), BLOCK, dt, kc, vc,
                            case.block_tables.shape[-1], new_tokens=NT, partition_size=psize, num_stages=nst,
                            units_capacity=0 if units_host is None else units_host.numel())
        rep = [l % L_res for l in range(L)]
        pin = lambda t: t.cpu().pin_memory()
        qh, kh, vh = pin(case.q[rep]), pin(case.k[rep]), pin(case.v[rep])
        bth = pin(case.block_tables[rep].clamp_min(0))
        smh = pin(case.slot_mapping[:, rep, :].contiguous())
        ch = pin(case.context_lens)
        oh = torch.empty((L, S, Hq, 128), dtype=dt).pin_memory()
        run_e2e = lambda: hs.run(qh, kh, vh, bth, smh, ch, oh, case.max_context_len, units_host=units_host)
        for _ in range(3):
            run_e2e()
        e2e_mode = "eager"
        if not args.eager:
            # the whole host-driven step (copies on their streams + launches) as one CUDA graph
            try:
                torch.cuda.synchronize()
                ge = torch.cuda.CUDAGraph()
                with torch.cuda.graph(ge):
                    run_e2e()
                ge.replay()
                torch.cuda.synchronize()
                run_e2e, e2e_mode = ge.replay, "CUDA graph replay (copies and launches captured together)"
            except Exception as exc:   # capture of the multi-stream step refused: keep the eager pipeline
                e2e_mode = f"eager (graph capture failed: {type(exc).__name__})"
                torch.cuda.synchronize()
        barrier()
        e0.record()
        for _ in range(args.steps):
            run_e2e()
        e1.record()
        barrier()
        ms_e2e = max_over_ranks(e0.elapsed_time(e1)) / args.steps
        e2e = {"value": world * S / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": hs.h2d_bytes, "d2h_bytes_per_step": hs.d2h_bytes, "launch": e2e_mode,
               "how": "HostDecodeStep.run: pinned host q/k/v/block_tables/slot_mapping/context_lens -> device, "
                      "ops, out -> pinned host, per layer on copy streams overlapped with the kernels"}
        status |= ops.device_status()
        del qh, kh, vh, bth, smh, oh

    # ---- tensor-parallel leg (N > 1): the same model sharded by kv head + NCCL all-reduce of the output ----
    tp = None
    if world > 1 and not args.no_tp and H % world == 0:
        Hl, Hql = H // world, Hq // world
        full = torch.zeros((S, Hq * 128), dtype=dt, device=dev)
        # the shard's own partition size and work list (fewer items per launch than the whole model has)
        tp_psize, tp_units = args.partition_size, None
        if not args.no_units:
            tp_psize = tp_psize or ops.suggest_partition_size(S * Hl, Hq // H, dev)
            tp_units = ops.work_units(ctx_list, tp_psize, dev, num_kv_heads=Hl)

        def tp_step(allreduce=True, attention=True):
            for l in range(L):
                r = l % L_res
                if attention and fused:
                    ops.decode_attention(out[:, :Hql], case.q[r][:, :Hql], case.k[r][:, :Hl], case.v[r][:, :Hl], kc, vc,
                                         None, case.scale, case.block_tables[r][:, :Hl], case.context_lens, BLOCK,
                                         case.max_context_len, partition_size=tp_psize, num_stages=nst, units=tp_units)
                elif attention:
                    ops.reshape_and_cache(case.k[r][:, :Hl], case.v[r][:, :Hl], kc, vc, case.slot_mapping[:, r, :Hl])
                    ops.paged_attention(out[:, :Hql], case.q[r][:, :Hql], kc, vc, None, case.scale,
                                        case.block_tables[r][:, :Hl], case.context_lens, BLOCK, case.max_context_len,
                                        partition_size=tp_psize, num_stages=nst, units=tp_units)
                if allreduce:
                    dist.all_reduce(full)

        tp_mode = "eager"

        def timed(fn):
            nonlocal tp_mode
            for _ in range(3):
                fn()
            run = fn
            if not args.eager:      # kernels and NCCL all-reduces of one step as one CUDA graph
                try:
                    torch.cuda.synchronize()
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        fn()
                    g.replay()
                    torch.cuda.synchronize()
                    run, tp_mode = g.replay, "CUDA graph replay"
                except Exception as exc:
                    tp_mode = f"eager (graph capture failed: {type(exc).__name__})"
                    torch.cuda.synchronize()
            barrier()
            e0.record()
            for _ in range(args.steps):
                run()
            e1.record()
            barrier()
            return max_over_ranks(e0.elapsed_time(e1)) / args.steps

        ms_tp = timed(tp_step)
        ms_ar = timed(lambda: tp_step(attention=False))
        ms_at = timed(lambda: tp_step(allreduce=False))
        tp = {"tp": world, "scaling": "strong", "tokens_per_s": S / (ms_tp * 1e-3), "ms_per_step": ms_tp,
              "attention_only_ms_per_step": ms_at, "allreduce_only_ms_per_step": ms_ar,
              "allreduce_bytes": full.numel() * full.element_size(), "launch": tp_mode,
              "note": "kv heads sharded over ranks (no cross-GPU traffic in attention); one NCCL all-reduce of the "
                      "[batch, hidden] output per layer"}

    # ---- CPU baseline on a bounded sample (rank 0, N = 1 only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        kcc, vcc, btc = compact_layer_to_cpu(case, kc, vc, 0)
        # slots of layer 0 renumbered into the compact pool
        slots = workloads.last_token_slots(btc.unsqueeze(0), ctx, BLOCK, NT)[:, 0, :]
        t_layer, reps = time_cpu_sample(case.q[0].cpu(), case.k[0].cpu(), case.v[0].cpu(), kcc, vcc, btc, slots,
                                        ctx, case.scale, args.cpu_seconds)
        cpu = {"value": S / (t_layer * L), "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"layer 0 of {L} (all {S} sequences, its own KV blocks copied to a compact host pool), "
                         f"mean of {reps} runs of {t_layer:.3f} s ({reps * t_layer:.0f} s of CPU work) on the CPU oracle, "
                         f"scaled x{L} layers"}

    if rank == 0:
        peak, peak_src = hbm_peak()
        launch_bytes = attn_bytes + (cw_bytes if fused else 0)
        achieved = launch_bytes / (attn_ms * 1e-3) / 1e9
        path_gbs = (attn_bytes + cw_bytes) * L / (ms_step * 1e-3) / 1e9
        traffic = NCU_DRAM_BYTES_PER_LAUNCH.get(args.workload) if args.batch == 0 else None
        line = {
            "metric": METRIC, "value": world * S / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": f"{args.workload}: {w['desc']}", "block_size": BLOCK, "seed": args.seed,
                       "pool": f"{num_blocks} blocks = {num_blocks * 8192 / 1e9:.1f} GB ({args.pool_frac:.0%} of HBM), "
                               "block lists scattered without replacement over the whole pool",
                       "resident_layers": L_res, "layers": L,
                       "l2": f"no flush: one step streams {attn_bytes * min(L, L_res) / 1e9:.1f} GB of distinct KV "
                             "blocks, far above the 126 MB L2",
                       "placement": ("1 model on 1 GPU" if world == 1 else
                                     f"{world} independent model replicas, one per GPU, no data-path collective"),
                       "partition_size": psize or "library default", "num_stages": nst or "library default",
                       "work_list": "none" if units is None else
                       f"{int((units >= 0).sum())} (sequence, kv head, partition) units from the host's context lengths",
                       "launch": "CUDA graph replay of one step" if graph is not None else "eager (Python call per op)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic,
                         "kernel": ("paged_attn_kernel<fused cache write> (+ merge kernel)" if fused else
                                    "paged_attn_kernel (+ merge kernel)"),
                         "algorithmic_bytes_per_launch": launch_bytes, "avg_launch_ms": attn_ms,
                         "peak_source": peak_src, "whole_path_gbs": path_gbs,
                         "whole_path_frac": path_gbs / peak,
                         "span": ("timed region / launches (graph replay, one attention launch per layer)"
                                  if (graph is not None and fused) else
                                  "CUDA events around every attention launch"),
                         "eager_span_ms": eager_span_ms},
            "step": ("decode_attention per layer (cache write fused into the attention launch)" if fused else
                     "reshape_and_cache + paged_attention per layer"),
            "eager_ms_per_step": ms_eager, "ms_per_step_by_rank": ms_ranks,
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": gpu_launches,
            "clocks": clocks, "device_status": status,
        }
        if two_op is not None:
            line["two_op"] = two_op
        if tp is not None:
            line["tp"] = tp
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def run_native_c3(args):
    """Config 3: the per-GPU share of three colocated models, one fused attention launch per layer index
    (layers 0-31 serve all three models, 32-39 two, 40-59 one) plus one cache write per model and layer."""
    import torch.distributed as dist
    from muxserve_b200 import flexstore, mixed, ops, workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    dt = torch.float16
    total_mem = torch.cuda.get_device_properties(dev).total_memory
    num_blocks = flexstore.get_num_gpu_blocks(total_mem, args.pool_frac, BLOCK)
    kc, vc = flexstore.allocate_gpu_cache(num_blocks, BLOCK, dt, dev)
    workloads.fill_pool_(kc, vc, args.seed)
    gen = torch.Generator().manual_seed(args.seed)               # same batch on every rank (TP shares sequences)
    perm = torch.randperm(num_blocks, generator=gen).to(dev)
    batches, cases, nxt = [], [], 0
    for name, L, heads, S in C3_MODELS:
        Hl = heads // C3_TP
        ctx = workloads.lognormal_context_lens(S, 256.0, 1.0, 16, 4096, gen)
        case = workloads.make_decode_case(workloads.ModelShape(name, L, Hl, Hl, S), ctx, block_size=BLOCK,
                                          num_blocks=num_blocks, dtype=dt, device=dev, seed=args.seed + len(cases),
                                          block_ids=perm, first_block=nxt, input_layers=4)
        nxt = case.extra["next_block"]
        cases.append(case)
        batches.append(mixed.ModelBatch(name, L, Hl, Hl, 128 ** -0.5, ctx, case.block_tables))
    plan = mixed.build_mixed_plan(batches, dev)
    L_max = max(plan.layers)
    packed_q = [mixed.pack_rows(plan, [c.q[i % c.q.shape[0]] for c in cases]) for i in range(4)]
    packed_k = [mixed.pack_rows(plan, [c.k[i % c.k.shape[0]] for c in cases]) for i in range(4)]
    packed_v = [mixed.pack_rows(plan, [c.v[i % c.v.shape[0]] for c in cases]) for i in range(4)]
    out = torch.empty_like(packed_q[0])
    psize, nst = args.partition_size, args.num_stages
    fused = not args.two_op
    attn_bytes, cw_bytes = [], []
    for l in range(L_max):
        a = w = 0
        for b in batches:
            if b.num_layers > l:
                a += workloads.attention_bytes(b.context_lens.tolist(), b.num_q_heads, b.num_kv_heads, BLOCK)
                w += workloads.cache_write_bytes(b.num_seqs, b.num_kv_heads)
        attn_bytes.append(a)
        cw_bytes.append(w)

    unit_psize = psize or 512     # the work lists are built for an explicit partition size (512 = library default)

    def step(events=None):
        for l in range(L_max):
            n_items, n_rows = plan.active(l)
            new_kv = {}
            if fused:      # one launch per layer index: every model's cache write and attention
                new_kv = dict(new_k=packed_k[l % 4][:n_items], new_v=packed_v[l % 4][:n_items])
            else:
                for c in cases:
                    if c.shape.num_layers > l:
                        r = l % c.k.shape[0]
                        ops.reshape_and_cache(c.k[r], c.v[r], kc, vc, c.slot_mapping[:, l, :])
            if events is not None:
                events[l][0].record()
            ops.paged_attention_mixed(out[:n_rows], packed_q[l % 4][:n_rows], kc, vc, plan.block_tables[l, :n_items],
                                      plan.item_context_len[:n_items], plan.item_q_row[:n_items],
                                      plan.item_group[:n_items], plan.item_scale[:n_items], BLOCK,
                                      plan.max_context_len, plan.max_group, partition_size=unit_psize, num_stages=nst,
                                      units=None if args.no_units else plan.units(l, unit_psize), **new_kv)
            if events is not None:
                events[l][1].record()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    events = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(L_max)]
              for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    graph = None
    if not args.eager:
        try:
            torch.cuda.synchronize()
            l0 = ops.launch_count
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            per_step_launches = ops.launch_count - l0
            graph.replay()
            torch.cuda.synchronize()
        except Exception as exc:      # capture refused: time the Python-issued launches instead
            print(f"bench: CUDA graph capture failed ({type(exc).__name__}: {exc}); timing eager launches",
                  file=sys.stderr)
            graph = None
            torch.cuda.synchronize()
    barrier()
    sampler.start()
    launches0 = ops.launch_count
    e0.record()
    for i in range(args.steps):
        if graph is not None:
            graph.replay()
        else:
            step(events[i])
    e1.record()
    gpu_launches = ops.launch_count - launches0 if graph is None else per_step_launches * args.steps
    barrier()
    clocks = sampler.stop()
    from muxserve_b200.parallel import max_over_ranks
    ms_step = max_over_ranks(e0.elapsed_time(e1), dev) / args.steps
    if graph is not None:
        barrier()
        e0.record()
        for i in range(args.steps):
            step(events[i])
        e1.record()
        barrier()
        ms_eager = max_over_ranks(e0.elapsed_time(e1), dev) / args.steps
    else:
        ms_eager = ms_step
    attn_ms = sum(a.elapsed_time(b) for evs in events for a, b in evs) / args.steps     # all layers of a step
    status = ops.device_status()
    if rank == 0:
        peak, peak_src = hbm_peak()
        S_total = sum(b.num_seqs for b in batches)
        # under graph replay with the fused step a layer index is exactly one attention launch (+ its merge kernel):
        # the launches' time is the timed region (gaps included); the eager pass's per-launch events carry the
        # Python call overhead of 60 small launches and are reported beside it
        span_ms = ms_step if (graph is not None and fused) else attn_ms
        achieved = (sum(attn_bytes) + (sum(cw_bytes) if fused else 0)) / (span_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": world * S_total / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "c3: " + C3_DESC, "block_size": BLOCK, "seed": args.seed,
                       "pool": f"{num_blocks} blocks = {num_blocks * 8192 / 1e9:.1f} GB ({args.pool_frac:.0%} of HBM)",
                       "items_per_launch": plan.item_offset, "layers": plan.layers,
                       "launch": "CUDA graph replay of one step" if graph is not None else "eager (Python call per op)",
                       "placement": "one TP=4 rank's share per GPU; value counts each GPU's share as its own batch",
                       "step": ("one fused launch per layer index (all models' cache writes + attention)" if fused else
                                "one reshape_and_cache per model and layer + one fused attention launch per layer index")},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "kernel": "paged_attn_kernel<mixed> (+ merge)",
                         "algorithmic_bytes_per_step": sum(attn_bytes), "attention_ms_per_step": span_ms,
                         "eager_span_ms": attn_ms, "peak_source": peak_src,
                         "span": ("timed region (graph replay, one attention launch per layer index)"
                                  if (graph is not None and fused) else "CUDA events around every attention launch"),
                         "whole_path_gbs": (sum(attn_bytes) + sum(cw_bytes)) / (ms_step * 1e-3) / 1e9},
            "cpu_baseline": None, "e2e": None, "gpu_launches": gpu_launches, "clocks": clocks, "device_status": status,
            "eager_ms_per_step": ms_eager,
        }
        emit(line)
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------- prompt phase (secondary workload)
PREFILL = dict(desc="LLaMA-7B shape fp16 prompt phase: 32 layers, 32 heads (MHA), head_dim 128, 16 prompts with lengths "
                    "U[128,2048] (the context range of config 2), block_size 16; per layer causal prompt attention + "
                    "cache write of every prompt token, one launch per layer",
               L=32, Hq=32, H=32, S=16, lo=128, hi=2048, dtype="f16")
PREFILL_METRIC = ("prompt-phase tokens/s (prompt attention + prompt cache write over all layers; achieved tensor TFLOP/s "
                  "of the attention kernel and fraction of peak in `roofline`)")


def tensor_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops_sustained"]), \
                "measured (MEASURED_PEAKS.json bf16_tflops_sustained: the kernel is timed inside a long step)"
        except Exception:
            pass
    return 1400.0, "fallback 1400 TFLOP/s sustained (MEASURED_PEAKS.json absent)"


def run_native_prefill(args):
    import torch.distributed as dist
    from muxserve_b200 import flexstore, ops, workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl native needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w = dict(PREFILL)
    if args.layers > 0:
        w["L"] = args.layers
    if args.batch > 0:
        w["S"] = args.batch
    if args.heads > 0:
        w["Hq"] = w["H"] = args.heads
    if args.prompt_len > 0:
        w["lo"] = w["hi"] = args.prompt_len
    dt = DTYPES[w["dtype"]]
    L, Hq, H, S = w["L"], w["Hq"], w["H"], w["S"]
    gen = torch.Generator().manual_seed(args.seed)           # every replica draws the same prompts
    lens = workloads.uniform_context_lens(S, w["lo"], w["hi"], gen)
    T = int(lens.sum())
    max_len = int(lens.max())
    nblk = workloads.blocks_needed(lens, L, H, BLOCK)
    num_blocks = nblk + 1024
    kc, vc = flexstore.allocate_gpu_cache(num_blocks, BLOCK, dt, dev)
    perm = torch.randperm(num_blocks, generator=gen).to(dev)
    tables, _ = workloads.scatter_block_tables(lens, L, H, BLOCK, perm)
    slots = workloads.prompt_slots(tables, lens, BLOCK)      # [T, L, H]
    Lq = min(L, 4)                                           # distinct per-layer inputs, cycled
    q = torch.randn((Lq, T, Hq, 128), generator=gen).to(dt).to(dev)
    k = torch.randn((Lq, T, H, 128), generator=gen).to(dt).to(dev)
    v = torch.randn((Lq, T, H, 128), generator=gen).to(dt).to(dev)
    out = torch.empty((T, Hq, 128), dtype=dt, device=dev)
    cu = ops.cu_seqlens_from_prompt_lens(lens.tolist(), dev)
    scale = 128 ** -0.5
    slot_layers = [slots[:, l, :] for l in range(L)]

    # work list from the prompt lengths the host holds (input_metadata.prompt_lens is a host list in the reference)
    punits = None if args.no_units else ops.prefill_work_units(lens.tolist(), Hq, dev)

    def step():          # one launch per layer: prompt attention with the cache write of every token inside
        for l in range(L):
            i = l % Lq
            ops.prefill_attention(out, q[i], k[i], v[i], cu, max_len, scale, key_cache=kc, value_cache=vc,
                                  slot_mapping=slot_layers[l], units=punits)

    def step_two_op():   # the reference's two calls per layer
        for l in range(L):
            i = l % Lq
            ops.prefill_attention(out, q[i], k[i], v[i], cu, max_len, scale)
            ops.reshape_and_cache(k[i], v[i], kc, vc, slot_layers[l])

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream()
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    launches0 = ops.launch_count
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    launches = ops.launch_count - launches0
    # the same step as two ops per layer
    for _ in range(3):
        step_two_op()
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        step_two_op()
    e1.record(stream)
    barrier()
    two_op_ms = e0.elapsed_time(e1) / args.steps
    # the kernel alone: events around every (fused) launch of a few more steps
    att_ms = []
    for _ in range(3):
        evs = []
        for l in range(L):
            i = l % Lq
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            ops.prefill_attention(out, q[i], k[i], v[i], cu, max_len, scale, key_cache=kc, value_cache=vc,
                                  slot_mapping=slot_layers[l], units=punits)
            b.record(stream)
            evs.append((a, b))
        torch.cuda.synchronize()
        att_ms += [a.elapsed_time(b) for a, b in evs]
    att = sum(att_ms) / len(att_ms)
    status = ops.device_status()
    # e2e: what the host supplies per step in the reference (prompt lengths -> cu_seqlens, the [T, L, H] int64
    # slot mapping) goes up from pinned memory, the last-token rows the sampler reads come back
    cu_h = cu.cpu().pin_memory()
    slots_h = slots.cpu().pin_memory()
    tables_h = tables.cpu().pin_memory()
    last_rows = (cu[1:].long() - 1)
    last_h = torch.empty((S, Hq, 128), dtype=dt).pin_memory()
    cu_d, slots_d, tables_d = torch.empty_like(cu), torch.empty_like(slots), torch.empty_like(tables)

    punits_h = None if punits is None else punits.cpu().pin_memory()
    punits_d = None if punits is None else torch.empty_like(punits)

    def e2e_step():      # the reference's hand-over: the [T, L, H] int64 slot mapping goes up every step
        if punits_h is not None:
            punits_d.copy_(punits_h, non_blocking=True)
        cu_d.copy_(cu_h, non_blocking=True)
        slots_d.copy_(slots_h, non_blocking=True)
        for l in range(L):
            i = l % Lq
            ops.prefill_attention(out, q[i], k[i], v[i], cu_d, max_len, scale, key_cache=kc, value_cache=vc,
                                  slot_mapping=slots_d[:, l, :], units=punits_d)
        last_h.copy_(out[last_rows], non_blocking=True)

    def e2e_step_tables():   # the prompts' block lists [L, S, H, max_blocks] int32 go up instead
        if punits_h is not None:
            punits_d.copy_(punits_h, non_blocking=True)
        cu_d.copy_(cu_h, non_blocking=True)
        tables_d.copy_(tables_h, non_blocking=True)
        for l in range(L):
            i = l % Lq
            ops.prefill_attention(out, q[i], k[i], v[i], cu_d, max_len, scale, key_cache=kc, value_cache=vc,
                                  block_tables=tables_d[l], units=punits_d)
        last_h.copy_(out[last_rows], non_blocking=True)

    e2e = None
    if not args.no_e2e:
        for _ in range(3):
            e2e_step()
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            e2e_step()
        e1.record(stream)
        barrier()
        e2e_ms = e0.elapsed_time(e1) / args.steps
        for _ in range(3):
            e2e_step_tables()
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            e2e_step_tables()
        e1.record(stream)
        barrier()
        e2e_tables_ms = e0.elapsed_time(e1) / args.steps
    t = torch.tensor([ms, e2e_ms if not args.no_e2e else 0.0, att, e2e_tables_ms if not args.no_e2e else 0.0],
                     dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms, att, e2e_tables_ms = (float(x) for x in t)
    if rank == 0:
        flops = workloads.prefill_flops(lens.tolist(), Hq)
        peak, peak_src = tensor_peak()
        achieved = flops / (att * 1e-3) / 1e12
        line = {
            "metric": PREFILL_METRIC, "value": T * world / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": f"prefill: {w['desc']}", "layers": L, "heads": Hq, "prompts": S,
                       "prompt_len_range": [w["lo"], w["hi"]], "prompt_tokens": T, "max_prompt_len": max_len,
                       "block_size": BLOCK, "seed": args.seed, "replicas": world,
                       "l2": "no flush: one step streams q/k/v of 4 distinct layers and writes a fresh region of the pool"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": None, "peak_source": peak_src,
                         "kernel": "prefill_attn_kernel (with the cache write inside)", "kernel_ms": att,
                         "flops": "useful causal FLOPs: 4*128 per (query, visible key) and q head"},
            "gpu_launches": launches, "clocks": clocks, "device_status": status,
            "two_op": {"ms_per_step": two_op_ms, "note": "prefill_attention + reshape_and_cache per layer"},
        }
        if not args.no_e2e:
            line["e2e"] = {"value": T * world / (e2e_ms * 1e-3), "unit": "tokens/s",
                           "h2d_bytes_per_step": cu_h.numel() * 4 + slots_h.numel() * 8,
                           "d2h_bytes_per_step": last_h.numel() * last_h.element_size(),
                           "with_block_tables": {"value": T * world / (e2e_tables_ms * 1e-3), "unit": "tokens/s",
                                                 "h2d_bytes_per_step": cu_h.numel() * 4 + tables_h.numel() * 4,
                                                 "note": "block lists uploaded instead of the slot mapping"}}
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = prefill_cpu_baseline(w, lens, args)
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def prefill_cpu_baseline(w, lens, args):
    """Oracle port on the host cores: one layer of the shortest prompts that fill the time budget."""
    from oracle.prefill_oracle import prefill_attention_ref
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    gen = torch.Generator().manual_seed(args.seed + 1)
    sample = sorted(lens.tolist())[:max(1, len(lens) // 4)]
    T = sum(sample)
    dt = DTYPES[w["dtype"]]
    q = torch.randn((T, w["Hq"], 128), generator=gen).to(dt)
    k = torch.randn((T, w["H"], 128), generator=gen).to(dt)
    v = torch.randn((T, w["H"], 128), generator=gen).to(dt)
    times = []
    t_all = time.perf_counter()
    while not times or (time.perf_counter() - t_all < args.cpu_seconds and len(times) < 50):
        t0 = time.perf_counter()
        prefill_attention_ref(q, k, v, sample, 128 ** -0.5)
        times.append(time.perf_counter() - t0)
    per_layer = sum(times) / len(times)
    return {"value": T / (per_layer * w["L"]), "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"attention of one of {w['L']} layers over the {len(sample)} shortest prompts ({T} tokens), "
                      f"{len(times)} repetitions; tokens/s = tokens / (layer time x {w['L']})"}


def main():
    args = parse_args()
    claim_stdout()
    if args.impl == "reference":
        if args.workload in ("c3", "prefill"):
            raise SystemExit("--impl reference supports c2, c4, c5")
        run_reference(args)
    elif args.workload == "c3":
        run_native_c3(args)
    elif args.workload == "prefill":
        run_native_prefill(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
