#!/usr/bin/env python
"""Benchmark of the decode attention path (reshape_and_cache + paged_attention over all layers).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload all|c2|c3|c4|c5|prefill] [--impl native|reference]

A step is one decode step of the path: for every layer the cache write of the new tokens and
the paged attention over the sequence batch (one fused launch per layer when one token per
sequence is appended).  Prints ONE JSON line.

* 1 GPU (default): the headline is configuration 2 (LLaMA-7B shape, fp16); the `configs` object of
  the same line carries configurations 3, 4, 5 and the prompt phase, each with its own roofline
  fraction and an oracle check of sampled rows, all over the one KV pool.
* N > 1 GPUs (torchrun): the headline is configuration 4 (LLaMA-65B shape, bf16) sharded by KV head
  over the N ranks with the all-reduce of the [batch, hidden] output after every layer — the
  partition the reference runs (tensor parallel, muxserve/flexserver/models/llama.py:100-117,131-137,162).
* ``--impl reference`` times the CPU oracle (the reference has no CPU implementation of these ops;
  its kernels live in an un-vendored fork) on the host cores, on the same workload.
"""
from __future__ import annotations

import argparse
import hashlib
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
                    "block_size 16, 1 new token/seq",
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
PREFILL = dict(desc="LLaMA-7B shape fp16 prompt phase: 32 layers, 32 heads (MHA), head_dim 128, 16 prompts with lengths "
                    "U[128,2048] (the context range of config 2), block_size 16; per layer causal prompt attention + "
                    "cache write of every prompt token, one launch per layer",
               L=32, Hq=32, H=32, S=16, lo=128, hi=2048, dtype="f16")
BLOCK = 16
DTYPES = {"f16": torch.float16, "bf16": torch.bfloat16}
FALLBACK_HBM_GBS = 6650.0
TARGET_REGION_S = 1.0          # timed time per measurement: regions of exactly K steps are repeated up to this


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


_T0 = time.perf_counter()


def log(*a):
    print(f"bench [{time.perf_counter() - _T0:6.1f} s]:", *a, file=sys.stderr, flush=True)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--workload", choices=["all", "c2", "c3", "c4", "c5", "prefill"], default="all",
                    help="all: the headline plus every other configuration as sub-results; one name: only that one")
    ap.add_argument("--pool-frac", type=float, default=0.6, help="fraction of HBM given to the KV pool")
    ap.add_argument("--partition-size", type=int, default=0)
    ap.add_argument("--num-stages", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (small profiler captures)")
    ap.add_argument("--batch", type=int, default=0, help="override the batch size (small profiler captures)")
    ap.add_argument("--prompt-len", type=int, default=0, help="prefill workload: every prompt has this length")
    ap.add_argument("--heads", type=int, default=0, help="prefill workload: override the head count (small captures)")
    ap.add_argument("--seed", type=int, default=20240531)
    ap.add_argument("--block-size", type=int, default=16, choices=[16, 32],
                    help="tokens per pool block for the whole run (16: the configurations' value; 32: MuxServe's default)")
    ap.add_argument("--eager", action="store_true",
                    help="time Python-issued launches instead of replaying a CUDA graph of one step")
    ap.add_argument("--two-op", action="store_true",
                    help="time reshape_and_cache + paged_attention as separate calls instead of the fused decode step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-serving", action="store_true", help="skip the e2e_serving leg (host scheduler + allocator in the loop)")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check of sampled rows (profiler captures)")
    ap.add_argument("--no-tp-extras", action="store_true", help="N > 1: only the headline (no sweep, no other configs)")
    ap.add_argument("--no-units", action="store_true",
                    help="launch one CTA per (item, partition index) instead of the host's work list")
    ap.add_argument("--no-early-kv", action="store_true", help="do not set MUX_ATTN_EARLY_KV on the decode launches")
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


def tensor_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops_sustained"]), \
                "measured (MEASURED_PEAKS.json bf16_tflops_sustained: the kernel is timed inside a long step)"
        except Exception:
            pass
    return 1400.0, "fallback 1400 TFLOP/s sustained (MEASURED_PEAKS.json absent)"


def kernel_source_sha() -> str:
    """Identifies the build of the attention kernels: DRAM traffic captured with ncu is only quoted for the
    build it was captured on."""
    h = hashlib.sha256()
    for name in ("paged_attention.cu", "attn_common.cuh", "ptx.cuh", "rope.cuh"):
        h.update((ROOT / "muxserve_b200" / "csrc" / name).read_bytes())
    return h.hexdigest()[:16]


def ncu_traffic(workload: str, algorithmic_bytes: int):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the table of ncu captures kept with the
    profile summaries: the entry is used only when it was captured on the current kernel sources; it holds the
    ratio traffic / algorithmic bytes of a smaller launch of the same shape, scaled to this launch."""
    p = ROOT / "profiles" / "dram_traffic.json"
    if not p.exists():
        return None, "no capture table"
    try:
        table = json.loads(p.read_text())
        e = table["entries"].get(workload)
        if e is None:
            return None, "no capture of this workload"
        if table.get("kernel_source_sha") != kernel_source_sha():
            return None, "kernel sources changed since the ncu capture"
        ratio = e["dram_bytes_per_launch"] / e["algorithmic_bytes_per_launch"]
        return int(round(ratio * algorithmic_bytes)), f"ncu capture {e['summary']} (ratio {ratio:.4f} x algorithmic bytes)"
    except Exception as exc:
        return None, f"capture table unreadable ({type(exc).__name__})"


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
def cpu_attention_step(q, k_new, v_new, kc, vc, bt, slots, ctx, scale, seqs):
    """One layer of the path on the CPU oracle for the first `seqs` sequences."""
    from oracle.attention_oracle import paged_attention_ref_batched
    from oracle.cache_write_oracle import reshape_and_cache_ref
    T_per = k_new.shape[0] // q.shape[0]
    reshape_and_cache_ref(k_new[:seqs * T_per], v_new[:seqs * T_per], kc, vc, slots[:seqs * T_per])
    return paged_attention_ref_batched(q[:seqs], kc, vc, scale, bt[:seqs], ctx[:seqs], BLOCK)


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


def cpu_sample_rate(w, seed, budget_s, cores, reps_max=200):
    """tokens/s of the CPU oracle on workload `w`: one layer over a bounded number of sequences, repeated for about
    `budget_s` seconds, scaled to the layer count.  Returns (tokens/s, description, measured seconds per repetition)."""
    torch.set_num_threads(cores)
    q, k, v, kc, vc, bt, slots, ctx = synth_cpu_layer(w, seed, seqs=2)
    t0 = time.perf_counter()
    cpu_attention_step(q, k, v, kc, vc, bt, slots, ctx, 128 ** -0.5, 2)
    t_seq = (time.perf_counter() - t0) / 2
    seqs = int(max(1, min(w["S"], (budget_s / 4) / max(1e-6, t_seq))))       # a repetition takes ~ a quarter of the budget
    q, k, v, kc, vc, bt, slots, ctx = synth_cpu_layer(w, seed, seqs=seqs)
    cpu_attention_step(q, k, v, kc, vc, bt, slots, ctx, 128 ** -0.5, seqs)     # warm-up
    times, t_all = [], time.perf_counter()
    while len(times) < reps_max and (not times or time.perf_counter() - t_all < budget_s):
        t0 = time.perf_counter()
        cpu_attention_step(q, k, v, kc, vc, bt, slots, ctx, 128 ** -0.5, seqs)
        times.append(time.perf_counter() - t0)
    dt = sum(times) / len(times)
    rate = seqs / (dt * w["L"])
    sample = (f"1 of {w['L']} layers over {seqs} of {w['S']} sequences on the CPU oracle (fp32 PyTorch gather attention + "
              f"scatter cache write), mean of {len(times)} repetitions of {dt:.3f} s; tokens/s = sequences / (time x {w['L']} layers)")
    return rate, sample, dt, seqs


def run_reference(args):
    """CPU arm: the oracle on all host threads, on the workload the native arm's headline uses at this N.
    A step is one layer of the workload over a bounded number of sequences (the measured step time is
    printed as it was measured); tokens/s scales it to the full layer count."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload if args.workload in WORKLOADS else ("c2" if args.gpus <= 1 else "c4")
    w = WORKLOADS[name]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    # calibrate on 2 sequences, then size the per-step sample so that the whole run stays near 2 minutes
    q, k, v, kc, vc, bt, slots, ctx = synth_cpu_layer(w, args.seed, seqs=2)
    t0 = time.perf_counter()
    cpu_attention_step(q, k, v, kc, vc, bt, slots, ctx, 128 ** -0.5, 2)
    t_seq = (time.perf_counter() - t0) / 2
    budget = 100.0
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
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak" if args.gpus <= 1 else "strong", "vs_baseline": None,
        "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": f"{name}: {w['desc']}".replace("block_size 16", f"block_size {BLOCK}"), "block_size": BLOCK, "seed": args.seed,
                   "ms_per_step_is": f"the measured time of one sampled step (1 layer, {seqs} sequences); a whole decode step "
                                     f"of the workload is {w['L']} x {w['S'] / seqs:.2f} times that",
                   "gpus_used": 0, "note_n_gpus": "the CPU arm runs on rank 0's host cores only and does not scale with N"},
        "cpu_baseline": {"value": tokens_per_s, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tokens_per_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference ships no CPU (or CUDA) source for these ops; this arm is the oracle port",
    }
    emit(line)


# ----------------------------------------------------------------------------- native arm: shared machinery
class Env:
    def __init__(self, args):
        import torch.distributed as dist
        self.args = args
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py --impl native needs a CUDA device (there is no CPU fallback)")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.status = 0
        self.launches_timed = 0

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.world == 1:
            return list(values)
        t = torch.tensor(list(values), dtype=torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(x) for x in t]

    def capture(self, fn, what=""):
        """(callable that runs one step, kernels per step, mode).  A CUDA graph of one step unless --eager."""
        from muxserve_b200 import ops
        self.barrier()               # ranks enter together: kernels of the TP all-reduce wait for their peers
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        l0 = ops.launch_count
        fn()
        per_step = ops.launch_count - l0
        if self.args.eager:
            return fn, per_step, "eager (Python call per op)"
        try:
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            self.barrier()
            g.replay()
            torch.cuda.synchronize()
            return g.replay, per_step, "CUDA graph replay of one step"
        except Exception as exc:      # capture refused: time the Python-issued launches instead
            log(f"CUDA graph capture of {what} failed ({type(exc).__name__}: {exc}); timing eager launches")
            torch.cuda.synchronize()
            return fn, per_step, f"eager (graph capture failed: {type(exc).__name__})"

    def timed(self, run, steps, warmup=3, target_s=TARGET_REGION_S, max_regions=25, sampler=None):
        """Times regions of EXACTLY `steps` steps (barrier + synchronize on both sides, CUDA events on the
        launching stream, max over ranks), repeated until about `target_s` seconds are timed; returns the median
        region's ms per step and every region's."""
        for _ in range(max(3, warmup)):
            run()
        self.barrier()
        regions = []
        if sampler is not None:
            sampler.start()
        while True:
            self.barrier()
            self.e0.record()
            for _ in range(steps):
                run()
            self.e1.record()
            self.barrier()
            regions.append(self.e0.elapsed_time(self.e1))
            more = sum(regions) * 1e-3 < target_s and len(regions) < max_regions
            if self.world > 1:      # all ranks stop together
                t = torch.tensor([1.0 if more else 0.0], device=self.dev)
                self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
                more = bool(t.item() > 0)
            if not more:
                break
        regions = self.max_over_ranks(regions)
        per_step = sorted(r / steps for r in regions)
        return per_step[len(per_step) // 2], {"regions": len(regions), "steps_per_region": steps,
                                              "ms_per_step_min": per_step[0], "ms_per_step_max": per_step[-1],
                                              "timed_s": sum(regions) * 1e-3}


class Pool:
    """The FlexStore-sized KV pool, allocated once; `as_dtype` re-fills it when the element type changes (fp16 bit
    patterns read as bf16 would hold NaN and infinities)."""

    def __init__(self, env: Env):
        from muxserve_b200 import flexstore
        args = env.args
        total_mem = torch.cuda.get_device_properties(env.dev).total_memory
        self.num_blocks = flexstore.get_num_gpu_blocks(total_mem, args.pool_frac, BLOCK)
        self.kc, self.vc = flexstore.allocate_gpu_cache(self.num_blocks, BLOCK, torch.float16, env.dev)
        self.dtype = None
        self.env = env
        self.desc = (f"{self.num_blocks} blocks = {self.num_blocks * 8192 / 1e9:.1f} GB ({args.pool_frac:.0%} of HBM), "
                     "block lists scattered without replacement over the whole pool")

    def rebind(self, block_size: int):
        """The same memory as a pool of `block_size`-token blocks (random contents stay valid under any view)."""
        nb = self.kc.numel() // (128 * block_size)
        self.kc = self.kc.reshape(-1)[:nb * 128 * block_size].view(nb, 16, block_size, 8)
        self.vc = self.vc.reshape(-1)[:nb * 128 * block_size].view(nb, 128, block_size)
        self.num_blocks = nb

    def as_dtype(self, dt):
        from muxserve_b200 import workloads
        kc, vc = self.kc.view(dt), self.vc.view(dt)
        if self.dtype != dt:
            workloads.fill_pool_(kc, vc, self.env.args.seed + 17 * self.env.rank + (1 if dt == torch.bfloat16 else 0))
            self.dtype = dt
        return kc, vc


def sampled_parity(case, layer, out, kc, vc, NT, seed, count=3):
    """Oracle on a few sampled sequences (all their heads) of the launch that produced `out` (layer `layer` of
    `case`), and the appended K/V rows bit for bit.  Runs after the timed regions."""
    from oracle.sampled_check import check_decode_rows, pick_sequences
    seqs = pick_sequences(case.context_lens.tolist(), count, seed)
    li = layer % case.q.shape[0]
    return check_decode_rows(out, case.q[li], case.k[li], case.v[li], kc, vc, case.block_tables[layer],
                             case.context_lens, case.scale, BLOCK, seqs, new_tokens=NT)


def require_parity(name, pc):
    if pc is not None and (not pc["ok"] or pc["pool_bit_exact"] is False):
        raise SystemExit(f"bench: oracle check of {name} failed: {json.dumps(pc)}")


def run_decode(env: Env, pool: Pool, name: str, tp: int = 1, tp_rank: int = 0, headline: bool = False,
               comm=None, collective: str = "none"):
    """One decode workload (c2 / c4 / c5), optionally the shard of tensor-parallel rank `tp_rank` of `tp` with the
    output all-reduce after every layer (`collective`: "none", "peer" = the library's kernel, "nccl")."""
    from muxserve_b200 import ops, workloads
    from muxserve_b200 import parallel
    args = env.args
    w = dict(WORKLOADS[name])
    if args.layers > 0:
        w["L"] = args.layers
    if args.batch > 0:
        w["S"] = args.batch
    dt = DTYPES[w["dtype"]]
    kc, vc = pool.as_dtype(dt)
    dev = env.dev
    L, S, NT = w["L"], w["S"], w["new_tokens"]
    shard = parallel.shard_heads(w["Hq"], w["H"], tp, tp_rank)
    Hq, H = shard.q_count, shard.kv_count
    hidden = w["Hq"] * 128

    # every rank draws the same context lengths (a TP group serves ONE batch); pool contents, block scatter and
    # q/k/v differ by rank
    gen = torch.Generator().manual_seed(args.seed)
    ctx = workloads.uniform_context_lens(S, w["lo"], w["hi"], gen)
    per_layer = workloads.blocks_needed(ctx, 1, H, BLOCK)
    L_res = max(1, min(L, int(pool.num_blocks * 0.98) // per_layer))     # distinct resident layers
    shape = workloads.ModelShape(name, L_res, Hq, H, S)
    case = workloads.make_decode_case(shape, ctx, block_size=BLOCK, num_blocks=pool.num_blocks, dtype=dt, device=dev,
                                      seed=args.seed + 1000 * env.rank, new_tokens=NT, input_layers=min(L_res, 8))
    Lq = case.q.shape[0]
    ctx_list = ctx.tolist()
    attn_bytes = workloads.attention_bytes(ctx_list, Hq, H, BLOCK)
    cw_bytes = workloads.cache_write_bytes(S * NT, H)
    fused = NT <= ops.MAX_FUSED_NEW_TOKENS and not args.two_op
    early = fused and not args.no_early_kv

    # tensor parallel: the rank's heads land in its columns of a [S, hidden] buffer whose other columns stay zero;
    # the all-reduce (sum) of those buffers is the concatenation of the shards' outputs
    if tp > 1:
        full_in = torch.zeros((S, hidden), dtype=dt, device=dev)
        full_out = torch.empty_like(full_in)
        out = full_in.view(S, w["Hq"], 128)[:, shard.q_start:shard.q_start + Hq]
    else:
        out = torch.empty((S, Hq, 128), dtype=dt, device=dev)
    psize, nst = args.partition_size, args.num_stages
    # Work list from the context lengths the host scheduler holds (it uploads them every step): the real
    # (sequence, kv head, partition) triples, fullest first, padded to a fixed length for the captured graph.
    units = units_host = None
    if not args.no_units:
        import numpy as np
        if not psize:
            psize, nst_auto = ops.suggest_launch(ctx_list, Hq // H, dev, num_kv_heads=H)
            nst = nst or nst_auto
        real = ops.work_units(ctx_list, psize, num_kv_heads=H)
        cap = (real.size + 127) // 128 * 128
        units_np = np.full((cap,), -1, dtype=np.int32)
        units_np[:real.size] = real
        units_host = torch.from_numpy(units_np).pin_memory()
        units = units_host.to(dev)

    def collect():
        if collective == "peer":
            comm.all_reduce(full_in, full_out)
        elif collective == "nccl":
            full_out.copy_(full_in)
            env.dist.all_reduce(full_out)

    def layer(l, fuse=fused, attention=True, allreduce=True, cache_write=True):
        r = l % L_res
        if attention and fuse:      # one launch: append the new token(s) and attend
            ops.decode_attention(out, case.q[r % Lq], case.k[r % Lq], case.v[r % Lq], kc, vc, None, case.scale,
                                 case.block_tables[r], case.context_lens, BLOCK, case.max_context_len,
                                 partition_size=psize, num_stages=nst, units=units, early_kv=early)
        elif attention:
            if cache_write:
                ops.reshape_and_cache(case.k[r % Lq], case.v[r % Lq], kc, vc, case.slot_mapping[:, r, :])
            ops.paged_attention(out, case.q[r % Lq], kc, vc, None, case.scale, case.block_tables[r], case.context_lens,
                                BLOCK, case.max_context_len, partition_size=psize, num_stages=nst, units=units)
        if allreduce and tp > 1:
            collect()

    def step(**kw):
        for l in range(L):
            layer(l, **kw)

    # ---- device-resident leg ----
    sampler = ClockSampler(env.local_rank) if headline else None
    run, per_step_launches, mode = env.capture(step, name)
    ms_step, stats = env.timed(run, args.steps, args.warmup, sampler=sampler,
                               target_s=TARGET_REGION_S if headline else 0.5)
    clocks = sampler.stop() if sampler is not None else None
    res = {"ms_per_step": ms_step, "tokens_per_s": S / (ms_step * 1e-3), "timing": stats, "launch": mode,
           "kernels_per_step": per_step_launches, "resident_layers": L_res, "layers": L,
           "partition_size": psize or "library default", "num_stages": nst or "library default",
           "work_list": "none" if units is None else
           f"{int((units >= 0).sum())} (sequence, kv head, partition) units from the host's context lengths",
           "step": ("decode_attention per layer (cache write fused into the attention launch)" if fused else
                    "reshape_and_cache + paged_attention per layer"),
           "early_kv": early}
    env.launches_timed = per_step_launches * args.steps * stats["regions"]

    # ---- the attention launches alone, where a layer is more than the attention launch (separate cache write, all-reduce) ----
    if fused and tp == 1:
        attn_ms = ms_step / L
        span = "timed region / launches (graph replay, one attention launch per layer)"
    else:
        run_a, _, _ = env.capture(lambda: step(allreduce=False, cache_write=False), name + " attention only")
        ms_a, _ = env.timed(run_a, args.steps, 3, target_s=0.3)
        attn_ms = ms_a / L
        span = "a second timed region with only the attention launches of a step / launches"
        res["attention_only_ms_per_step"] = ms_a
    peak, peak_src = hbm_peak()
    launch_bytes = attn_bytes + (cw_bytes if fused else 0)
    achieved = launch_bytes / (attn_ms * 1e-3) / 1e9
    traffic, traffic_src = (ncu_traffic(name, launch_bytes) if tp == 1 and args.batch == 0 and BLOCK == 16
                            else (None, "not captured for this shape"))
    res["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                       "traffic": traffic, "traffic_source": traffic_src,
                       "kernel": ("paged_attn_kernel<fused cache write> (+ merge kernel)" if fused else
                                  "paged_attn_kernel (+ merge kernel)"),
                       "algorithmic_bytes_per_launch": launch_bytes, "avg_launch_ms": attn_ms,
                       "peak_source": peak_src, "span": span,
                       "whole_path_gbs": (attn_bytes + cw_bytes) * L / (ms_step * 1e-3) / 1e9}
    res["roofline"]["whole_path_frac"] = res["roofline"]["whole_path_gbs"] / peak
    if clocks is not None:
        res["clocks"] = clocks

    # ---- oracle on sampled rows of the last layer's launch (outside every timed region) ----
    if not args.no_parity:
        step()
        torch.cuda.synchronize()
        pc = sampled_parity(case, (L - 1) % L_res, out, kc, vc, NT, args.seed)
        res["parity_check"] = pc
        require_parity(name, pc)
    env.status |= ops.device_status()
    res["device_status"] = env.status
    res["_ctx"] = dict(case=case, out=out, units=units, units_host=units_host, psize=psize, nst=nst, L_res=L_res, w=w,
                       shard=shard, fused=fused, step=step, layer=layer, ctx=ctx, attn_bytes=attn_bytes, cw_bytes=cw_bytes,
                       full_in=full_in if tp > 1 else None, full_out=full_out if tp > 1 else None, kc=kc, vc=vc,
                       early=early)
    return res


def strip(res):
    return {k: v for k, v in res.items() if not k.startswith("_")}


def two_op_leg(env, res):
    """The same step with the two reference-signature ops (separate cache-write launch)."""
    c = res["_ctx"]
    w = c["w"]
    run2, _, _ = env.capture(lambda: c["step"](fuse=False), "two-op step")
    ms2, _ = env.timed(run2, env.args.steps, 3, target_s=0.5)
    return {"ms_per_step": ms2, "tokens_per_s": w["S"] / (ms2 * 1e-3),
            "whole_path_gbs": (c["attn_bytes"] + c["cw_bytes"]) * w["L"] / (ms2 * 1e-3) / 1e9,
            "note": "reshape_and_cache and paged_attention as two calls per layer"}


def e2e_leg(env, pool, res, name, comm=None):
    """End to end from HOST buffers: per layer q/k/v and the layer's block tables go up from pinned memory, the
    ops run, the layer's output comes back (for a TP rank: the all-reduced [S, hidden] output)."""
    from muxserve_b200 import workloads
    from muxserve_b200.host_step import HostDecodeStep
    c = res["_ctx"]
    w, case, shard = c["w"], c["case"], c["shard"]
    L, S, NT = w["L"], w["S"], w["new_tokens"]
    dt = DTYPES[w["dtype"]]
    Hq, H = shard.q_count, shard.kv_count
    depth = 4
    out_views = post = None
    if shard.tp > 1:
        hidden = w["Hq"] * 128
        ins = [torch.zeros((S, hidden), dtype=dt, device=env.dev) for _ in range(depth)]
        outs = [torch.empty((S, hidden), dtype=dt, device=env.dev) for _ in range(depth)]
        out_views = [t.view(S, w["Hq"], 128)[:, shard.q_start:shard.q_start + Hq] for t in ins]
        post = lambda b: comm.all_reduce(ins[b], outs[b])
    hs = HostDecodeStep(workloads.ModelShape(name, L, Hq, H, S), BLOCK, dt, c["kc"], c["vc"], case.block_tables.shape[-1],
                        new_tokens=NT, partition_size=c["psize"], num_stages=c["nst"],
                        units_capacity=0 if c["units_host"] is None else c["units_host"].numel(),
                        out_views=out_views, post=post, early_kv=c["early"])
    L_res, Lq = c["L_res"], case.q.shape[0]
    rep = [l % L_res for l in range(L)]
    repq = [(l % L_res) % Lq for l in range(L)]
    pin = lambda t: t.cpu().pin_memory()
    qh, kh, vh = pin(case.q[repq]), pin(case.k[repq]), pin(case.v[repq])
    bth = pin(case.block_tables[rep].clamp_min(0))
    smh = pin(case.slot_mapping[:, rep, :].contiguous())
    ch = pin(case.context_lens)
    oh = (torch.empty((L, S, w["Hq"] * 128), dtype=dt) if shard.tp > 1 else torch.empty((L, S, Hq, 128), dtype=dt)).pin_memory()
    run_once = lambda: hs.run(qh, kh, vh, bth, smh, ch, oh, case.max_context_len, units_host=c["units_host"])
    run, _, mode = env.capture(run_once, "host-driven step")
    ms, stats = env.timed(run, env.args.steps, 3, target_s=0.5)
    return {"value": S / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
            "h2d_bytes_per_step": hs.h2d_bytes, "d2h_bytes_per_step": hs.d2h_bytes, "launch": mode, "timing": stats,
            "how": "HostDecodeStep.run: pinned host q/k/v/block_tables/slot_mapping/context_lens -> device, ops"
                   + (", output all-reduce" if shard.tp > 1 else "") + ", out -> pinned host, per layer on copy "
                   "streams overlapped with the kernels"}


def serving_leg(env, pool, name="c2", steps=24):
    """Decode steps with the HOST rows of the path inside the timed loop, as a server runs them, one after the other
    (the next step's scheduling needs this step's sampled tokens): BatchScheduler.try_batch -> KVStorage.allocate_batch
    (only when a sequence crosses a block boundary) -> get_batch_info -> hand-over -> kernels -> output back.
    Variant "rebuild": the reference's hand-over (get_batch fills the whole [tokens, max_blocks, L, H] table, it is
    uploaded and permuted on the device: muxserve/flexserver/llm_runtime.py:277-339).  Variant "device_tables": the
    persistent device table takes only the newly granted block ids (DeviceBlockTables.stage_grant / flush)."""
    import numpy as np
    from muxserve_b200 import ops, workloads
    from muxserve_b200.batch_scheduler import BatchScheduler
    from muxserve_b200.device_tables import DeviceBlockTables
    from muxserve_b200.host_step import HostDecodeStep
    from muxserve_b200.memory_manager import KVStorage
    args = env.args
    w = WORKLOADS[name]
    dt = DTYPES[w["dtype"]]
    kc, vc = pool.as_dtype(dt)
    L, S, Hq, H = w["L"], w["S"], w["Hq"], w["H"]
    gen = torch.Generator().manual_seed(args.seed)
    ctx0 = workloads.uniform_context_lens(S, w["lo"], w["hi"], gen).tolist()
    max_seq = w["hi"] + steps + 16
    max_blocks = (max_seq + BLOCK - 1) // BLOCK
    out = {}
    pin = lambda t: t.pin_memory()
    qh = pin(torch.randn((L, S, Hq, 128), generator=gen).to(dt))
    kh = pin(torch.randn((L, S, H, 128), generator=gen).to(dt))
    vh = pin(torch.randn((L, S, H, 128), generator=gen).to(dt))
    oh = pin(torch.empty((L, S, Hq, 128), dtype=dt))
    for variant in ("rebuild", "device_tables"):
        kv, sched = KVStorage(pool.num_blocks), BatchScheduler(L, H, max_seq, BLOCK)
        ids = list(range(1000, 1000 + S))
        for rid, n in zip(ids, ctx0):
            sched.add_request(np.zeros(n - 1, dtype=np.int32), rid, steps + 8)
        info = sched.try_batch(ids, [])
        blocks = kv.allocate_batch(info[:-1], L, H)
        if blocks[0] != S:
            raise SystemExit("bench: the pool cannot hold the serving leg's prompts")
        dbt = None
        if variant == "device_tables":
            dbt = DeviceBlockTables(L, H, max_rows=S, max_blocks=max_blocks, device=env.dev)
            dbt.stage_grant(info[:-1], blocks)
            dbt.flush()
        sched.get_batch_info(info[:-1], blocks)
        hs = HostDecodeStep(workloads.ModelShape(name, L, Hq, H, S), BLOCK, dt, kc, vc, max_blocks)
        tok, pos = pin(torch.empty(((S + 7) // 8 * 8,), dtype=torch.int32)), pin(torch.empty(((S + 7) // 8 * 8,), dtype=torch.int32))
        ctx_h = pin(torch.empty((S,), dtype=torch.int32))
        slots_h = pin(torch.empty((S, L, H), dtype=torch.int64))
        host_ms, wall_ms, gpu_ms, idx_bytes, allocs = [], [], [], [], 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        bt_dev = None
        for it in range(steps + 3):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            info = sched.try_batch(ids, [1] * S)
            if info[-1] > 0:
                blocks = kv.allocate_batch(info[:-1], L, H)
                allocs += 1
            else:
                blocks = np.array([S], dtype=np.int32)
            if blocks[0] != S:
                raise SystemExit("bench: the serving leg ran out of blocks")
            ntok, nctx, maxctx, maxblk = sched.get_batch_info(info[:-1], blocks)[:4]
            if variant == "rebuild":
                bt_h = pin(torch.empty((S, maxblk, L, H), dtype=torch.int32))
                sched.get_batch(info[:-1], blocks, tok, pos, ctx_h, bt_h, slots_h)
                t1 = time.perf_counter()
                e0.record()
                bt_dev = bt_h.to(env.dev, non_blocking=True).permute(2, 0, 3, 1).contiguous()    # [L, S, H, maxblk]
                hs.run(qh, kh, vh, None, slots_h, ctx_h, oh, maxctx, device_tables=bt_dev)
                nbytes = bt_h.numel() * 4 + slots_h.numel() * 8 + ctx_h.numel() * 4
            else:
                dbt.stage_grant(info[:-1], blocks)
                # context lengths only: what the kernels need besides the table (positions = context - 1)
                st = [sched.request_state(r)["context_len"] for r in ids] if it == 0 else None
                if st is not None:
                    ctx_cur = torch.tensor(st, dtype=torch.int32)
                else:
                    ctx_cur = ctx_cur + 1
                ctx_h.copy_(ctx_cur)
                t1 = time.perf_counter()
                e0.record()
                before = dbt.uploaded_bytes
                dbt.flush()
                rows = dbt.rows_for(ids)
                hs.run(qh, kh, vh, None, None, ctx_h, oh, int(ctx_cur.max()), device_tables=dbt.tables, seq_rows=rows)
                nbytes = dbt.uploaded_bytes - before + ctx_h.numel() * 4
            e1.record()
            torch.cuda.synchronize()
            t2 = time.perf_counter()
            if it >= 3:
                host_ms.append((t1 - t0) * 1e3)
                wall_ms.append((t2 - t0) * 1e3)
                gpu_ms.append(e0.elapsed_time(e1))
                idx_bytes.append(nbytes)
        env.status |= ops.device_status()
        mean = lambda xs: sum(xs) / len(xs)
        out[variant] = {"tokens_per_s": S / (mean(wall_ms) * 1e-3), "ms_per_step": mean(wall_ms),
                        "host_ms_per_step": mean(host_ms), "gpu_ms_per_step": mean(gpu_ms),
                        "host_ms_max": max(host_ms), "index_bytes_per_step": int(mean(idx_bytes)),
                        "steps_with_allocation": allocs, "steps": steps}
        del kv, sched, hs, dbt, bt_dev
    out["how"] = ("wall clock per step around try_batch -> allocate_batch -> get_batch_info -> hand-over -> per-layer "
                  "q/k/v upload, fused decode launches, output download -> synchronize; host and GPU parts run one after "
                  "the other (a step's scheduling needs the previous step's tokens), so ms_per_step ~ host + gpu; block ids "
                  "come from the allocator (highest ids first), not scattered at random")
    out["cores"] = os.cpu_count()
    return out


# ----------------------------------------------------------------------------- config 3
def run_c3(env: Env, pool: Pool, tp_world: int = 1, comm=None):
    """Config 3: the per-GPU share of three colocated models, one fused attention launch per layer index
    (layers 0-31 serve all three models, 32-39 two, 40-59 one).  With `tp_world` = 4 the four ranks are the
    four tensor-parallel shards and every launch is followed by the all-reduce of the models' [batch, hidden] outputs."""
    from muxserve_b200 import mixed, ops, workloads
    args = env.args
    dev = env.dev
    dt = torch.float16
    kc, vc = pool.as_dtype(dt)
    tp_rank = env.rank if tp_world > 1 else 0
    gen = torch.Generator().manual_seed(args.seed)               # same batch on every rank (TP shares sequences)
    perm = torch.randperm(pool.num_blocks, generator=gen).to(dev)
    batches, cases, nxt = [], [], 0
    for name, L, heads, S in C3_MODELS:
        Hl = heads // C3_TP
        ctx = workloads.lognormal_context_lens(S, 256.0, 1.0, 16, 4096, gen)
        case = workloads.make_decode_case(workloads.ModelShape(name, L, Hl, Hl, S), ctx, block_size=BLOCK,
                                          num_blocks=pool.num_blocks, dtype=dt, device=dev,
                                          seed=args.seed + len(cases) + 100 * tp_rank,
                                          block_ids=perm, first_block=nxt, input_layers=4)
        nxt = case.extra["next_block"]
        cases.append(case)
        batches.append(mixed.ModelBatch(name, L, Hl, Hl, 128 ** -0.5, ctx, case.block_tables))
    full = tp_world > 1
    plan = mixed.build_mixed_plan(batches, dev, tp=C3_TP if full else 1, tp_rank=tp_rank)
    L_max = max(plan.layers)
    rows_total = plan.row_offset[-1]
    packed_q = [mixed.pack_rows(plan, [c.q[i % c.q.shape[0]] for c in cases]) for i in range(4)]
    packed_k = [mixed.pack_items(plan, [c.k[i % c.k.shape[0]] for c in cases]) for i in range(4)]
    packed_v = [mixed.pack_items(plan, [c.v[i % c.v.shape[0]] for c in cases]) for i in range(4)]
    out = torch.zeros((rows_total, 128), dtype=dt, device=dev)
    reduced = torch.empty_like(out) if full else None
    fused = not args.two_op
    early = fused and not args.no_early_kv
    attn_bytes, cw_bytes, launch_cfg = [], [], []
    for l in range(L_max):
        a = w = 0
        for b in batches:
            if b.num_layers > l:
                a += workloads.attention_bytes(b.context_lens.tolist(), b.num_q_heads, b.num_kv_heads, BLOCK)
                w += workloads.cache_write_bytes(b.num_seqs, b.num_kv_heads)
        attn_bytes.append(a)
        cw_bytes.append(w)
        n_items, _ = plan.active(l)
        if args.partition_size:
            launch_cfg.append((args.partition_size, args.num_stages))
        else:       # per layer index: the launches differ a lot in size (780 / 396 / 156 items)
            ps, ns = ops.suggest_launch(plan.item_context_len_host[:n_items], plan.max_group, dev)
            launch_cfg.append((ps, args.num_stages or ns))

    def step(attention=True, allreduce=True):
        for l in range(L_max):
            n_items, n_rows = plan.active(l)
            ps, ns = launch_cfg[l]
            new_kv = {}
            if attention:
                if fused:      # one launch per layer index: every model's cache write and attention
                    new_kv = dict(new_k=packed_k[l % 4][:n_items], new_v=packed_v[l % 4][:n_items])
                else:
                    for c in cases:
                        if c.shape.num_layers > l:
                            r = l % c.k.shape[0]
                            ops.reshape_and_cache(c.k[r], c.v[r], kc, vc, c.slot_mapping[:, l, :])
                ops.paged_attention_mixed(out[:n_rows], packed_q[l % 4][:n_rows], kc, vc, plan.block_tables[l, :n_items],
                                          plan.item_context_len[:n_items], plan.item_q_row[:n_items],
                                          plan.item_group[:n_items], plan.item_scale[:n_items], BLOCK,
                                          plan.max_context_len, plan.max_group, partition_size=ps, num_stages=ns,
                                          units=None if args.no_units else plan.units(l, ps), early_kv=early, **new_kv)
            if full and allreduce:
                comm.all_reduce(out[:n_rows], reduced[:n_rows])

    run, per_step_launches, mode = env.capture(step, "c3")
    ms_step, stats = env.timed(run, args.steps, args.warmup)
    S_total = sum(b.num_seqs for b in batches)
    peak, peak_src = hbm_peak()
    res = {"ms_per_step": ms_step, "tokens_per_s": S_total / (ms_step * 1e-3), "timing": stats, "launch": mode,
           "kernels_per_step": per_step_launches, "items_per_launch": plan.item_offset, "layers": plan.layers,
           "launch_config_per_layer_group": sorted({(plan.active(l)[0],) + launch_cfg[l] for l in range(L_max)}),
           "early_kv": early,
           "step": ("one fused launch per layer index (all models' cache writes + attention)" if fused else
                    "one reshape_and_cache per model and layer + one fused attention launch per layer index")}
    if full:
        run_a, _, _ = env.capture(lambda: step(allreduce=False), "c3 attention only")
        ms_a, _ = env.timed(run_a, args.steps, 3, target_s=0.5)
        res["attention_only_ms_per_step"] = ms_a
        res["allreduce_bytes_per_layer_group"] = sorted({plan.active(l)[1] * 256 for l in range(L_max)})
        span_ms = ms_a
    else:
        span_ms = ms_step
    total = sum(attn_bytes) + (sum(cw_bytes) if fused else 0)
    achieved = total / (span_ms * 1e-3) / 1e9
    traffic, traffic_src = ncu_traffic("c3", total) if not full else (None, "not captured for this shape")
    res["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                       "traffic": traffic, "traffic_source": traffic_src + ("; per STEP like algorithmic_bytes_per_step"
                                                                           if traffic is not None else ""),
                       "kernel": "paged_attn_kernel<mixed, fused cache write> (+ merge)",
                       "algorithmic_bytes_per_step": total, "attention_ms_per_step": span_ms, "peak_source": peak_src,
                       "span": "timed region of one step's attention launches (graph replay, one per layer index)"}
    if not args.no_parity:
        step()
        torch.cuda.synchronize()
        # the last launch served only the deepest model; check that one and, from layer 0's launch, the others
        from oracle.sampled_check import check_decode_rows, pick_sequences
        checks = {}
        for l in (L_max - 1, 0):
            n_items, n_rows = plan.active(l)
            ps, ns = launch_cfg[l]
            ops.paged_attention_mixed(out[:n_rows], packed_q[l % 4][:n_rows], kc, vc, plan.block_tables[l, :n_items],
                                      plan.item_context_len[:n_items], plan.item_q_row[:n_items],
                                      plan.item_group[:n_items], plan.item_scale[:n_items], BLOCK,
                                      plan.max_context_len, plan.max_group, partition_size=ps, num_stages=ns,
                                      units=None if args.no_units else plan.units(l, ps),
                                      new_k=packed_k[l % 4][:n_items], new_v=packed_v[l % 4][:n_items])
            torch.cuda.synchronize()
            outs = mixed.unpack_rows(plan, out, batches)
            for c, b, o in zip(cases, batches, outs):
                if b.num_layers <= l or b.name in checks:
                    continue
                li = l % c.q.shape[0]
                pc = check_decode_rows(o, c.q[li], c.k[li], c.v[li], kc, vc, c.block_tables[l], c.context_lens, c.scale,
                                       BLOCK, pick_sequences(c.context_lens.tolist(), 3, args.seed))
                checks[b.name] = pc
                require_parity("c3 " + b.name, pc)
        res["parity_check"] = {"rows": sum(p["rows"] for p in checks.values()),
                               "max_abs_err": max(p["max_abs_err"] for p in checks.values()),
                               "ok": all(p["ok"] for p in checks.values()),
                               "pool_bit_exact": all(p["pool_bit_exact"] for p in checks.values()),
                               "models": sorted(checks)}
    env.status |= ops.device_status()
    res["device_status"] = env.status
    return res


# ----------------------------------------------------------------------------- prompt phase (secondary workload)
PREFILL_METRIC = ("prompt-phase tokens/s (prompt attention + prompt cache write over all layers; achieved tensor TFLOP/s "
                  "of the attention kernel and fraction of peak in `roofline`)")


def run_prefill(env: Env, pool: Pool, full_detail: bool):
    from muxserve_b200 import ops, workloads
    args = env.args
    dev = env.dev
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
    kc, vc = pool.as_dtype(dt)
    L, Hq, H, S = w["L"], w["Hq"], w["H"], w["S"]
    gen = torch.Generator().manual_seed(args.seed)           # every replica draws the same prompts
    lens = workloads.uniform_context_lens(S, w["lo"], w["hi"], gen)
    T = int(lens.sum())
    max_len = int(lens.max())
    perm = torch.randperm(pool.num_blocks, generator=gen).to(dev)
    tables, _ = workloads.scatter_block_tables(lens, L, H, BLOCK, perm)
    del perm
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

    steps = max(3, min(args.steps, 10))
    l0 = ops.launch_count
    step()
    per_step_launches = ops.launch_count - l0
    ms, stats = env.timed(step, steps, 3, target_s=0.6)
    flops = workloads.prefill_flops(lens.tolist(), Hq)
    peak, peak_src = tensor_peak()
    achieved = flops * L / (ms * 1e-3) / 1e12        # one launch per layer: the step IS the kernel's launches
    res = {"metric": PREFILL_METRIC, "ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "timing": stats,
           "launch": "eager (Python call per op; launches of ~0.5 ms each)", "kernels_per_step": per_step_launches,
           "prompt_tokens": T, "prompts": S, "max_prompt_len": max_len, "layers": L,
           "workload": f"prefill: {w['desc']}",
           "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                        "traffic": None, "peak_source": peak_src,
                        "kernel": "prefill_attn_kernel (with the cache write inside)", "kernel_ms": ms / L,
                        "flops": "useful causal FLOPs: 4*128 per (query, visible key) and q head",
                        "span": "timed region / launches (one launch per layer)"}}
    if full_detail:
        ms2, _ = env.timed(step_two_op, steps, 3, target_s=0.5)
        res["two_op"] = {"ms_per_step": ms2, "note": "prefill_attention + reshape_and_cache per layer"}
    if not args.no_parity:
        # oracle on the two shortest prompts and one more (all heads), last layer's launch; their K/V rows in the pool
        from oracle.prefill_oracle import prefill_attention_ref
        step()
        torch.cuda.synchronize()
        i = (L - 1) % Lq
        order = sorted(range(S), key=lambda s: int(lens[s]))
        picks = order[:2] + [order[len(order) // 2]]
        err, ok, pool_ok, rows = 0.0, True, True, 0
        cu_h = cu.cpu().tolist()
        for s in picks:
            a, b = cu_h[s], cu_h[s + 1]
            ref = prefill_attention_ref(q[i][a:b].cpu(), k[i][a:b].cpu(), v[i][a:b].cpu(), [b - a], scale)
            got = out[a:b].float().cpu()
            e = (got - ref).abs()
            err = max(err, float(e.max()))
            ok = ok and bool((e <= 2e-3 + 1e-2 * ref.abs()).all())
            rows += (b - a) * Hq
            sl = slot_layers[L - 1][a:b]                                   # [n, H]
            blk, off = (sl // BLOCK).reshape(-1), (sl % BLOCK).reshape(-1)
            pool_ok = pool_ok and torch.equal(kc[blk, :, off, :].reshape(b - a, H, 128), k[i][a:b]) \
                and torch.equal(vc[blk, :, off].reshape(b - a, H, 128), v[i][a:b])
        pc = {"rows": rows, "prompts": picks, "max_abs_err": err, "ok": ok, "pool_bit_exact": bool(pool_ok),
              "tolerance": "2e-3 + 1e-2 * |ref|"}
        res["parity_check"] = pc
        require_parity("prefill", pc)
    if full_detail and not args.no_e2e:
        # e2e: what the host supplies per step in the reference (prompt lengths -> cu_seqlens, the [T, L, H] int64
        # slot mapping) goes up from pinned memory, the last-token rows the sampler reads come back
        cu_hh = cu.cpu().pin_memory()
        slots_h = slots.cpu().pin_memory()
        last_rows = (cu[1:].long() - 1)
        last_h = torch.empty((S, Hq, 128), dtype=dt).pin_memory()
        cu_d, slots_d = torch.empty_like(cu), torch.empty_like(slots)
        punits_h = None if punits is None else punits.cpu().pin_memory()
        punits_d = None if punits is None else torch.empty_like(punits)

        def e2e_step():
            if punits_h is not None:
                punits_d.copy_(punits_h, non_blocking=True)
            cu_d.copy_(cu_hh, non_blocking=True)
            slots_d.copy_(slots_h, non_blocking=True)
            for l in range(L):
                i = l % Lq
                ops.prefill_attention(out, q[i], k[i], v[i], cu_d, max_len, scale, key_cache=kc, value_cache=vc,
                                      slot_mapping=slots_d[:, l, :], units=punits_d)
            last_h.copy_(out[last_rows], non_blocking=True)

        e2e_ms, _ = env.timed(e2e_step, steps, 3, target_s=0.5)
        res["e2e"] = {"value": T / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                      "h2d_bytes_per_step": cu_hh.numel() * 4 + slots_h.numel() * 8,
                      "d2h_bytes_per_step": last_h.numel() * last_h.element_size()}
    if full_detail and not args.no_cpu_baseline and env.rank == 0:
        res["cpu_baseline"] = prefill_cpu_baseline(w, lens, args)
    env.status |= ops.device_status()
    res["device_status"] = env.status
    return res


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


# ----------------------------------------------------------------------------- tensor-parallel checks and sweep
def tp_checks(env: Env, comm):
    """(i) a small model sharded by KV head over the ranks: every rank attends over its heads of the SAME pool and
    batch, the all-reduce of the column-placed shard outputs must equal the unsharded launch bit for bit;
    (ii) the all-reduce of random 16-bit partials against the fp32 sum: the peer-memory kernel exactly (fp32 sums in
    rank order, one rounding), NCCL within the tolerance of tp roundings."""
    from muxserve_b200 import flexstore, ops, parallel, workloads
    dist, dev, tp, r = env.dist, env.dev, env.world, env.rank
    res = {}
    for dt_name, dt in (("bf16", torch.bfloat16), ("f16", torch.float16)):
        S, Hq, H, nb = 12, 16, 8 if tp <= 8 else tp, 4096
        Hq = max(Hq, H)
        gen = torch.Generator().manual_seed(4242)                 # identical on every rank
        ctx = workloads.uniform_context_lens(S, 16, 700, gen)
        case = workloads.make_decode_case(workloads.ModelShape("tp-check", 1, Hq, H, S), ctx, block_size=BLOCK,
                                          num_blocks=nb, dtype=dt, device=dev, seed=99)
        kc, vc = flexstore.allocate_gpu_cache(nb, BLOCK, dt, dev)
        workloads.fill_pool_(kc, vc, 7)
        kc2, vc2 = kc.clone(), vc.clone()
        whole = torch.empty((S, Hq, 128), dtype=dt, device=dev)
        ops.decode_attention(whole, case.q[0], case.k[0], case.v[0], kc, vc, None, case.scale, case.block_tables[0],
                             case.context_lens, BLOCK, case.max_context_len)
        sh = parallel.shard_heads(Hq, H, tp, r)
        q, k, v = parallel.shard_qkv(sh, case.q[0], case.k[0], case.v[0])
        bt, _ = parallel.shard_index_tensors(sh, case.block_tables, case.slot_mapping)
        partial = torch.zeros((S, Hq * 128), dtype=dt, device=dev)
        mine = partial.view(S, Hq, 128)[:, sh.q_start:sh.q_start + sh.q_count]
        ops.decode_attention(mine, q, k, v, kc2, vc2, None, case.scale, bt[0], case.context_lens, BLOCK,
                             case.max_context_len)
        total = torch.empty_like(partial)
        comm.all_reduce(partial, total)
        torch.cuda.synchronize()
        same = torch.equal(total.view(S, Hq, 128), whole)
        # the shard appended exactly its own heads' rows
        sl = slice(sh.kv_start, sh.kv_start + sh.kv_count)
        ids = case.block_tables[0][:, sl].reshape(-1).long()
        ids = ids[ids >= 0]
        pool_same = torch.equal(kc2[ids], kc[ids]) and torch.equal(vc2[ids], vc[ids])
        res[f"sharded_equals_unsharded_{dt_name}"] = bool(same and pool_same)
        # random partials
        g2 = torch.Generator().manual_seed(1000 + r)
        x = torch.randn((128, 8192), generator=g2).to(dt).to(dev)
        parts = [torch.empty_like(x) for _ in range(tp)]
        dist.all_gather(parts, x)
        acc = torch.zeros_like(x, dtype=torch.float32)
        for p_ in parts:
            acc += p_.float()
        ours = torch.empty_like(x)
        for algo in (1, 2):
            comm.all_reduce(x, ours, algo=algo)
            torch.cuda.synchronize()
            res[f"peer_allreduce_algo{algo}_exact_{dt_name}"] = bool(torch.equal(ours, acc.to(dt)))
        theirs = x.clone()
        dist.all_reduce(theirs)
        eps = 2.0 ** (-8 if dt == torch.bfloat16 else -11)
        tol = tp * eps * float(acc.abs().max())
        res[f"nccl_allreduce_max_err_{dt_name}"] = float((theirs.float() - acc).abs().max())
        res[f"nccl_allreduce_within_tp_roundings_{dt_name}"] = res[f"nccl_allreduce_max_err_{dt_name}"] <= tol
    res["device_status"] = ops.device_status()
    flags = [v for k_, v in res.items() if isinstance(v, bool)]
    ok = all(flags) and res["device_status"] == 0
    t = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    res["ok_on_all_ranks"] = bool(t.item() > 0)
    return res


def allreduce_sweep(env: Env, comm):
    """us per all-reduce for the message sizes of the path's TP configurations (the reference keeps such a sweep as
    its all-reduce template, muxserve/flexserver/dist_utils.py:80-118): the peer-memory kernel (auto, one-shot,
    two-shot) and NCCL, 40 back-to-back operations per CUDA graph."""
    dist, dev = env.dist, env.dev
    rows = []
    for nbytes in (64 << 10, 256 << 10, 512 << 10, 1 << 20, 2 << 20, 4 << 20):
        n = nbytes // 2
        x = torch.randn((n,), device=dev).to(torch.bfloat16)
        y = torch.empty_like(x)
        row = {"bytes": nbytes}
        for label, fn in (("peer_auto_us", lambda: comm.all_reduce(x, y)),
                          ("peer_one_shot_us", (lambda: comm.all_reduce(x, y, algo=1)) if nbytes * env.world <= comm.slot_bytes else None),
                          ("peer_two_shot_us", lambda: comm.all_reduce(x, y, algo=2)),
                          ("nccl_us", lambda: dist.all_reduce(y))):
            if fn is None:
                continue
            many = lambda fn=fn: [fn() for _ in range(40)]
            run, _, _ = env.capture(many, label)
            ms, _ = env.timed(run, 5, 3, target_s=0.05, max_regions=3)
            row[label] = ms * 1e3 / 40
        rows.append(row)
    return rows


def oproj_leg(env: Env, comm, name: str):
    """The step after attention on a TP rank: o_proj (row-parallel GEMM of the rank's heads' output with its weight
    slice) + the all-reduce of the [tokens, hidden] result, as ONE fused kernel per layer (tcgen05 GEMM whose epilogue
    exchanges the tiles), against the library's GEMM followed by its all-reduce and against torch.matmul (cuBLAS)
    followed by NCCL.  Weights of 16 layers are cycled (more than L2 holds); numerics: the fused result equals the
    rank-order sum of the ranks' rounded partial products exactly."""
    from muxserve_b200 import tp_comm
    dist, dev, world = env.dist, env.dev, env.world
    w = WORKLOADS[name]
    dt = DTYPES[w["dtype"]]
    hidden, L = w["Hq"] * 128, w["L"]
    k = hidden // world
    m = min(w["S"], 128)
    Lw = min(L, 16)
    gen = torch.Generator(device=dev).manual_seed(env.args.seed + env.rank)
    a = torch.randn((m, k), generator=gen, device=dev).to(dt)
    wt = (torch.randn((Lw, hidden, k), generator=gen, device=dev) / hidden ** 0.5).to(dt)
    out = torch.empty((m, hidden), dtype=dt, device=dev)
    tmp = torch.empty_like(out)
    op = tp_comm.TPOProj(m, hidden, dev)
    # numerics
    op.forward(a, wt[0], out)
    part = torch.empty_like(out)
    tp_comm.oproj(a, wt[0], part)
    parts = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    acc = torch.zeros_like(part, dtype=torch.float32)
    for p_ in parts:
        acc += p_.float()
    torch.cuda.synchronize()
    exact = bool(torch.equal(out, acc.to(dt)))
    ref = a.float() @ wt[0].float().T
    gemm_err = float((part.float() - ref).abs().max())
    res = {"m": m, "n": hidden, "k_local": k, "fused_equals_rank_order_sum_of_rounded_partials": exact,
           "gemm_max_abs_err_vs_fp32": gemm_err}

    def timed(fn, label):
        run, _, _ = env.capture(lambda: [fn(l % Lw) for l in range(L)], label)
        ms, _ = env.timed(run, env.args.steps, 3, target_s=0.3)
        return ms * 1e3 / L

    res["fused_us_per_layer"] = timed(lambda i: op.forward(a, wt[i], out, early_w=True), "fused o_proj")
    res["fused_no_early_w_us_per_layer"] = timed(lambda i: op.forward(a, wt[i], out), "fused o_proj, no early weights")
    res["fused_one_shot_us_per_layer"] = timed(lambda i: op.forward(a, wt[i], out, algo=1), "fused o_proj one-shot")
    res["fused_two_shot_us_per_layer"] = timed(lambda i: op.forward(a, wt[i], out, algo=2), "fused o_proj owners")
    res["gemm_then_allreduce_us_per_layer"] = timed(lambda i: (tp_comm.oproj(a, wt[i], tmp, early_w=True), comm.all_reduce(tmp, out)),
                                                    "o_proj then all-reduce")
    res["cublas_then_nccl_us_per_layer"] = timed(lambda i: (torch.matmul(a, wt[i].T, out=tmp), dist.all_reduce(tmp)),
                                                 "cuBLAS then NCCL")
    res["gemm_alone_us_per_layer"] = timed(lambda i: tp_comm.oproj(a, wt[i], tmp, early_w=True), "o_proj alone")
    flops, wbytes = 2.0 * m * hidden * k, hidden * k * 2
    link = 2.0 * (world - 1) / world * m * hidden * 2
    peak_t, _ = tensor_peak()
    peak_h, _ = hbm_peak()
    target = max(flops / (peak_t * 1e12), wbytes / (peak_h * 1e9), link / 770e9) * 1e6
    res["roofline"] = {"bound": "max(tensor, hbm weight read, nvlink)", "target_us": target,
                       "achieved_over_target": target / res["fused_us_per_layer"],
                       "flops": flops, "weight_bytes": wbytes, "nvlink_bytes_per_rank": link,
                       "nvlink_peak": "770 GB/s per direction per GPU (measured peer copy on this pool)"}
    return res


# ----------------------------------------------------------------------------- orchestration
def base_line(env, args, res, name, desc, dtype, scaling, placement, extra_cfg=None):
    cfg = {"workload": f"{name}: {desc}".replace("block_size 16", f"block_size {BLOCK}"), "block_size": BLOCK, "seed": args.seed,
           "l2": "no flush: every launch streams its own KV blocks, far more per step than the 126 MB L2 holds",
           "placement": placement}
    cfg.update(extra_cfg or {})
    for k in ("resident_layers", "layers", "partition_size", "num_stages", "work_list", "launch", "early_kv"):
        if k in res:
            cfg[k] = res[k]
    line = {"metric": METRIC, "value": res["tokens_per_s"], "unit": "tokens/s", "n_gpus": env.world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": res["ms_per_step"],
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": cfg, "roofline": res["roofline"], "timing": res["timing"], "step": res.get("step"),
            "parity_check": res.get("parity_check"), "clocks": res.get("clocks"), "device_status": env.status}
    return line


def block32_leg(env: Env, pool: Pool):
    """Configuration 2 over 32-token blocks (MuxServe's default block size, muxserve/arg_utils.py:22), on the same pool
    memory; everything that reads the module's block size sees 32 for the duration."""
    global BLOCK
    BLOCK = 32
    pool.rebind(32)
    try:
        keep = strip(run_decode(env, pool, "c2"))
        return dict(workload="c2 with block_size 32: " + WORKLOADS["c2"]["desc"].replace("block_size 16", "block_size 32"),
                    block_size=32, **keep)
    finally:
        BLOCK = 16
        pool.rebind(16)
        torch.cuda.empty_cache()


def run_native_single(env: Env):
    """1 GPU: headline config 2 + the other configurations as sub-results (or only the one --workload names)."""
    args = env.args
    pool = Pool(env)
    which = args.workload
    only = which != "all"
    if which in ("all", "c2", "c4", "c5"):
        name = "c2" if which == "all" else which
        w = WORKLOADS[name]
        res = run_decode(env, pool, name, headline=True)
        line = base_line(env, args, res, name, w["desc"], w["dtype"], "weak", "1 model on 1 GPU", {"pool": pool.desc})
        line["gpu_launches"] = env.launches_timed
        if res["_ctx"]["fused"] and not args.two_op:
            line["two_op"] = two_op_leg(env, res)
        line["e2e"] = None if args.no_e2e else e2e_leg(env, pool, res, name)
        if not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            rate, sample, _, _ = cpu_sample_rate(w, args.seed, args.cpu_seconds, cores)
            line["cpu_baseline"] = {"value": rate, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample}
        else:
            line["cpu_baseline"] = None
        del res
        torch.cuda.empty_cache()
        if not only:
            configs = {}
            if not args.no_serving:
                log("e2e_serving")
                line["e2e_serving"] = serving_leg(env, pool, "c2")
            log("c3")
            configs["c3"] = dict(workload="c3: " + C3_DESC, **run_c3(env, pool))
            torch.cuda.empty_cache()
            log("prefill")
            configs["prefill"] = run_prefill(env, pool, full_detail=False)
            torch.cuda.empty_cache()
            for n in ("c4", "c5"):
                log(n)
                r = run_decode(env, pool, n)
                configs[n] = dict(workload=f"{n}: {WORKLOADS[n]['desc']}", **strip(r))
                del r
                torch.cuda.empty_cache()
            if BLOCK == 16:
                log("c2 at block_size 32")
                configs["c2_block32"] = block32_leg(env, pool)
            line["configs"] = configs
        line["device_status"] = env.status
        emit(line)
    elif which == "c3":
        res = run_c3(env, pool)
        line = base_line(env, args, res, "c3", C3_DESC, "f16", "weak",
                         "one TP=4 rank's share on one GPU", {"pool": pool.desc, "items_per_launch": res["items_per_launch"]})
        line.update(gpu_launches=res["kernels_per_step"] * args.steps * res["timing"]["regions"], cpu_baseline=None, e2e=None)
        line["c3"] = {k: v for k, v in res.items() if k not in ("roofline", "timing", "parity_check")}
        emit(line)
    else:
        res = run_prefill(env, pool, full_detail=True)
        line = {"metric": PREFILL_METRIC, "value": res["tokens_per_s"], "unit": "tokens/s", "n_gpus": env.world,
                "steps": args.steps, "warmup": 3, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": res["workload"], "block_size": BLOCK, "seed": args.seed, "pool": pool.desc},
                "roofline": res["roofline"], "timing": res["timing"], "parity_check": res.get("parity_check"),
                "gpu_launches": res["kernels_per_step"] * res["timing"]["steps_per_region"] * res["timing"]["regions"],
                "e2e": res.get("e2e"), "cpu_baseline": res.get("cpu_baseline"), "two_op": res.get("two_op"),
                "device_status": env.status}
        emit(line)


def run_native_tp(env: Env):
    """N > 1 GPUs: the headline is config 4 sharded by KV head over the N ranks (strong scaling of ONE model's
    decode step), the all-reduce of the [batch, hidden] output after every layer done by the library's
    peer-memory kernel; the same step with NCCL, the attention and the collectives alone, the numeric checks, the
    all-reduce sweep, configs 2 and 5 at TP = N and (at N = 4) config 3 on its four ranks ride in `tp`."""
    from muxserve_b200 import ops
    from muxserve_b200.tp_comm import TPAllReduce
    args = env.args
    world = env.world
    name = args.workload if args.workload in WORKLOADS else "c4"
    w = WORKLOADS[name]
    if w["H"] % world != 0:
        raise SystemExit(f"bench: {w['H']} kv heads do not divide over {world} ranks")
    pool = Pool(env)
    comm = TPAllReduce(4 << 20, env.dev)
    tp = {"tp": world, "partition": "kv heads (and their q heads) sharded over the ranks, index tensors replicated; attention "
                                   "and the cache write need no cross-GPU traffic, the collective is the all-reduce (sum) of the "
                                   "[batch, hidden] output after every layer"}
    log("tp checks")
    tp["check"] = tp_checks(env, comm)
    if not tp["check"]["ok_on_all_ranks"]:
        if env.rank == 0:
            log("TP checks failed:", json.dumps(tp["check"]))
        raise SystemExit("bench: tensor-parallel numeric checks failed")
    log("headline", name)
    res = run_decode(env, pool, name, tp=world, tp_rank=env.rank, headline=True, comm=comm, collective="peer")
    c = res["_ctx"]
    hidden_bytes = w["S"] * w["Hq"] * 128 * 2
    line = base_line(env, args, res, name, w["desc"], w["dtype"], "strong",
                     f"ONE model sharded by kv head over {world} GPUs (tensor parallel), output all-reduce after every layer "
                     "by the library's peer-memory kernel",
                     {"pool": pool.desc + " (per rank: its own heads' blocks)", "allreduce_bytes": hidden_bytes,
                      "tp": world})
    line["gpu_launches"] = env.launches_timed
    tp["attention_only_ms_per_step"] = res.get("attention_only_ms_per_step")
    # the collectives alone, and the same step with NCCL
    L = w["L"] if args.layers <= 0 else args.layers
    run_ar, _, _ = env.capture(lambda: [comm.all_reduce(c["full_in"], c["full_out"]) for _ in range(L)], "peer all-reduce only")
    ms_ar, _ = env.timed(run_ar, args.steps, 3, target_s=0.3)
    run_nc, _, _ = env.capture(lambda: [env.dist.all_reduce(c["full_out"]) for _ in range(L)], "nccl all-reduce only")
    ms_nc, _ = env.timed(run_nc, args.steps, 3, target_s=0.3)
    tp["allreduce_only_ms_per_step"] = {"peer_memory_kernel": ms_ar, "nccl": ms_nc, "messages_per_step": L,
                                        "bytes": hidden_bytes}

    def nccl_step():
        for l in range(L):
            c["layer"](l, allreduce=False)
            c["full_out"].copy_(c["full_in"])
            env.dist.all_reduce(c["full_out"])
    run_n, _, _ = env.capture(nccl_step, "step with NCCL")
    ms_n, _ = env.timed(run_n, args.steps, 3, target_s=0.5)
    tp["with_nccl_allreduce"] = {"ms_per_step": ms_n, "tokens_per_s": w["S"] / (ms_n * 1e-3),
                                 "note": "the same step, the output copied and all-reduced by NCCL after every layer"}
    line["e2e"] = None if args.no_e2e else e2e_leg(env, pool, res, name, comm=comm)
    line["cpu_baseline"] = None
    del res, c
    torch.cuda.empty_cache()
    if not args.no_tp_extras:
        log("all-reduce sweep")
        tp["allreduce_sweep"] = allreduce_sweep(env, comm)
        log("fused o_proj")
        tp["oproj_fused"] = {n: oproj_leg(env, comm, n) for n in (name, "c2") if WORKLOADS[n]["Hq"] % world == 0}
        others = {}
        for n in ("c4", "c5", "c2"):          # bf16 workloads first: the pool is re-filled only once
            if n == name or WORKLOADS[n]["H"] % world != 0:
                continue
            log("tp", n)
            r = run_decode(env, pool, n, tp=world, tp_rank=env.rank, comm=comm, collective="peer")
            others[n] = dict(workload=f"{n}: {WORKLOADS[n]['desc']}", **strip(r))
            del r
            torch.cuda.empty_cache()
        if world == C3_TP:
            log("tp c3")
            others["c3"] = dict(workload="c3: " + C3_DESC + "; the four ranks are the four TP shards", **run_c3(env, pool, world, comm))
            torch.cuda.empty_cache()
        tp["configs"] = others
        # replicas (how MuxServe places models that fit one GPU): N independent copies of config 2, no collective
        log("replicas")
        r = run_decode(env, pool, "c2")
        tp["replicas_c2"] = {"tokens_per_s_all_gpus": world * r["tokens_per_s"], "ms_per_step": r["ms_per_step"],
                             "roofline_frac": r["roofline"]["frac"], "scaling": "weak",
                             "note": f"{world} independent model replicas of config 2, one per GPU, no data-path collective"}
        del r
    line["tp"] = tp
    line["device_status"] = env.status | ops.device_status()
    env.barrier()
    if env.rank == 0:
        emit(line)
    # The step graphs hold captured NCCL kernels and the peers' mapped buffers; tearing communicators down
    # under them has hung a run here for minutes.  Everything is measured and printed: leave without teardown.
    sys.stderr.flush()
    os._exit(0)


def main():
    global BLOCK
    args = parse_args()
    BLOCK = args.block_size
    claim_stdout()
    if args.impl == "reference":
        run_reference(args)
        return
    env = Env(args)
    if env.world > 1:
        run_native_tp(env)
    else:
        run_native_single(env)


if __name__ == "__main__":
    main()
