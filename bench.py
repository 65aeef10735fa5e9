"""Benchmark of the MTA forward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c4]

One "step" is one full MTA forward (QK^T/sqrt(D) -> conv -> head mix -> softmax -> conv -> head mix -> @V)
over one synthetic batch of the workload (default c4: B8 H16 S4096 D128 bf16, causal, conv 6x11, head
mixes 16x16, post-softmax conv 3x3).  Rank 0 prints ONE JSON line.

  value          tokens/s of the whole job with inputs resident in HBM (CUDA events, max over ranks)
  e2e            tokens/s through the module's forward_host with HOST buffers: pinned host -> device copies of
                 q,k,v and the device -> host copy of the output are inside the timed region (the library
                 overlaps them with the computation, batch chunk by batch chunk)
  roofline       the slowest kernel of the step (device time between the events the library records around
                 its kernels) against the measured peak that bounds it
  roofline_step  the whole step's algorithmic flops against the measured bf16 tensor peak of ONE GPU
  cpu_baseline   the reference's own PyTorch module (oracle/_ref, MTAAttention.forward) on this box's host
                 cores, one batch element per sample (rank 0, N=1 only); the C port of oracle/ if the
                 reference's files are not there
  standalone     the stand-alone conv (config 2), head mix (config 3) and conv attention (fusion tier F1)
                 entry points timed alone with CUDA events, each against its roofline
  reference_gpu  the reference's Triton path on the same GPU, run in a child process (N=1 only)
  strong         (N > 1) fixed batches split over the ranks by sharding.plan_shards - config 4, config 5 and a
                 batch smaller than the rank count (query-row blocks with recomputed halo rows) - with the NCCL
                 gather of the outputs timed separately and one foreign shard recomputed on rank 0 and
                 compared bit for bit with what the gather delivered
  h2d            bare pinned host <-> device copy rate per rank with all ranks copying at once: the ceiling of e2e

With N > 1 (torchrun, one rank per GPU) `value` is weak scaling: every rank runs the same-size workload on its
own seeded batch, no data-path collective; the only communication is the barrier and the max-reduction of the
measured time.

`--impl reference` times the reference's CPU implementation instead: each step is one forward of the reference's
MTAAttention over ONE batch element of the workload on all host cores (the line says how that sample scales to
the workload's tokens/s).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import statistics
import subprocess
import sys
import threading
import time
import types

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from multitokenatention_triton_b200.synthetic import (WORKLOADS, MTAWorkload, device_qkv, make_mta_inputs,  # noqa: E402
                                                      make_mta_weights)

METRIC = "MTA fwd tokens/s"
NOMINAL = {"hbm_gbs": 8000.0, "bf16_tflops": 2250.0}
FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
C23_BYTES = 805_437_440            # configs 2 and 3: the lower triangle read once, the whole (4,16,2048,2048) output written


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
    return dict(FALLBACK, bf16_tflops_sustained=1400.0), "fallback"


def dram_bytes_per_score():
    """DRAM traffic per lower-triangle score of each stage kernel, from the ncu captures under profiles/."""
    try:
        with open(os.path.join(ROOT, "profiles", "dram_bytes_per_score.json")) as f:
            return json.load(f)["bytes_per_lower_element"]
    except (OSError, KeyError, ValueError):
        return {}


def host_threads() -> int:
    """Every core this process may run on, whatever OMP_NUM_THREADS a launcher exported."""
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for n, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def workload_name(wl: MTAWorkload) -> str:
    return (f"{wl.name}: full MTA forward B{wl.B} H{wl.H} S{wl.S} D{wl.D} {str(wl.dtype).split('.')[-1]} causal, "
            f"conv {wl.cq}x{wl.ck} + head mix {wl.H}x{wl.H} + softmax + conv {wl.cq2}x{wl.ck2} + head mix, seed {wl.seed}")


def job_config(wl: MTAWorkload, world: int) -> dict:
    """The same dictionary in both arms: it names the job, not the implementation."""
    return {"workload": workload_name(wl), "global_batch": wl.B * world,
            "parallelism": f"batch-sharded x{world}, no collective",
            "l2": "working set per step (>= 4 GB of score planes at c4) exceeds the 126 MB L2; no explicit flush"}


# ---------------------------------------------------------------------------------------------------
# CPU legs: the reference's own PyTorch module when oracle/_ref holds it, else the C port.
class CpuSample:
    """One batch element of the workload through the reference's MTAAttention.forward (mta_attention_pytorch.py:58-83)
    on the host cores, at the workload's dtype.  If a full-length batch element does not fit `budget_s`, a shorter
    sequence is sampled; the reference's cost per batch element grows with S^2 (it evaluates whole S x S planes)."""

    def __init__(self, wl: MTAWorkload, budget_s: float):
        from oracle import ref_runner as rr
        self.rr, self.wl = rr, wl
        torch.set_num_threads(host_threads())
        self.cores = torch.get_num_threads()
        self.S = wl.S
        self._build()
        t = self.step()                                  # first forward: also sizes the sample
        while t > budget_s and self.S > 256:
            self.S = max(256, (int(self.S * (budget_s / t) ** 0.5) // 256) * 256)
            self._build()
            t = self.step()

    def _build(self):
        wl1 = dataclasses.replace(self.wl, B=1, S=self.S)
        inp = make_mta_inputs(wl1)
        self.model = self.rr.pytorch_mta(wl1, inp, torch.device("cpu"), self.wl.dtype)
        self.q, self.k, self.v = inp["q"], inp["k"], inp["v"]

    def step(self) -> float:
        t0 = time.perf_counter()
        self.rr.cpu_forward(self.model, self.q, self.k, self.v)
        return time.perf_counter() - t0

    def tokens_per_s(self, seconds_per_step: float) -> float:
        # one batch element of S_sample tokens; a full-length one costs (S / S_sample)^2 as much and holds S tokens
        return self.wl.S / (seconds_per_step * (self.wl.S / self.S) ** 2)

    def scaled(self) -> dict:
        return {"batch": f"each step is 1 of the workload's {self.wl.B} batch elements (tokens/s per batch element equals tokens/s of the batch)",
                "seq": None if self.S == self.wl.S else f"sampled at S={self.S}; time scaled by (S/{self.S})^2 = {(self.wl.S / self.S) ** 2:.2f}"}

    def describe(self, n: int, seconds: float) -> str:
        return (f"the reference's MTAAttention.forward (PyTorch {torch.__version__}, {str(self.wl.dtype).split('.')[-1]}) on batch "
                f"element 0, H{self.wl.H} S{self.S} D{self.wl.D}, {n} forward(s), {seconds:.1f} s")


_CPU_INPUTS = {}


def cpu_port_tokens_per_s(wl: MTAWorkload, budget_s: float, threads: int = 0):
    """Times the CPU port of the reference algorithm (oracle/mta_oracle.c, OpenMP) on a block of query rows
    of batch element 0 centred on S/2, where a row's cost equals the workload's mean cost per token.
    The block is grown until it needs about `budget_s` seconds.  Returns (tokens/s, cores, description, seconds)."""
    from oracle import mta_oracle as orc
    orc.set_threads(threads or host_threads())
    cores = orc.num_threads()
    if wl not in _CPU_INPUTS:
        inp = make_mta_inputs(wl, batch_slice=slice(0, 1))
        _CPU_INPUTS[wl] = [inp[k].float().numpy() for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    a = _CPU_INPUTS[wl]
    rmode = {torch.float32: orc.ROUND_NONE, torch.bfloat16: orc.ROUND_BF16, torch.float16: orc.ROUND_FP16}[wl.dtype]
    mid = wl.S // 2

    def run(n):
        r0, r1 = max(0, mid - n // 2), min(wl.S, mid - n // 2 + n)
        t0 = time.perf_counter()
        orc.mta_fwd_rows(*a, 0, r0, r1, True, rmode)
        return time.perf_counter() - t0, r1 - r0

    t, n = run(min(16, wl.S))
    target = int(min(wl.S, max(16, n * budget_s / max(t, 1e-3)))) // 16 * 16 or n
    if target > n:
        t, n = run(target)
    desc = (f"CPU port (C, OpenMP) of the reference algorithm on batch element 0, query rows "
            f"[{max(0, mid - n // 2)},{max(0, mid - n // 2) + n}) of {wl.S} (block centred on S/2 = mean cost per token), "
            f"all {wl.H} heads, {t:.1f} s")
    return n / t, cores, desc, t


def cpu_baseline(wl: MTAWorkload, budget_s: float) -> dict:
    """The bounded CPU sample of the main arm's line."""
    from oracle import ref_runner as rr
    if rr.available():
        s = CpuSample(wl, budget_s / 3)
        n = max(1, min(5, int(budget_s / max(s.step(), 1e-3)) - 1))
        t0 = time.perf_counter()
        for _ in range(n):
            s.step()
        t = time.perf_counter() - t0
        return {"value": s.tokens_per_s(t / n), "unit": "tokens/s", "cores": s.cores, "kind": "reference",
                "sample": s.describe(n, t), "scaled": s.scaled()}
    v, cores, desc, _ = cpu_port_tokens_per_s(wl, budget_s)
    return {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc}


def reference_arm(args, wl: MTAWorkload, rank: int, world: int):
    """`--impl reference`: K timed steps (after W warm-up steps) of the reference's CPU implementation, each step one
    batch element, sized so that the run ends within a few minutes.  Rank 0 alone works."""
    if rank != 0:
        return
    from oracle import ref_runner as rr
    total = max(1, args.steps + args.warmup)
    per_step = max(1.0, min(20.0, 150.0 / total))
    if rr.available():
        s = CpuSample(wl, per_step)
        for _ in range(max(0, args.warmup - 1)):         # sizing the sample was the first warm-up step
            s.step()
        times = [s.step() for _ in range(args.steps)]
        sec = statistics.mean(times)
        value, cores, kind = s.tokens_per_s(sec), s.cores, "reference"
        desc, scaled = s.describe(args.steps, sum(times)), s.scaled()
    else:
        vals, secs = [], []
        for i in range(total):
            v, cores, desc, t = cpu_port_tokens_per_s(wl, per_step)
            if i >= args.warmup:
                vals.append(v)
                secs.append(t)
        value, sec, kind = statistics.mean(vals), statistics.mean(secs), "port"
        scaled = {"batch": "each step is a block of query rows of batch element 0 centred on S/2 (mean cost per token)", "seq": None}
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": str(wl.dtype).split(".")[-1] if kind == "reference" else "f64 accumulate on %s inputs" % str(wl.dtype).split(".")[-1],
        "data": "synthetic", "config": job_config(wl, world), "scaled": scaled,
        "ms_per_step_is": "the time of one sampled step (one batch element), not of a whole batch; `value` applies `scaled`",
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": desc},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
def event_time_ms(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    e.synchronize()
    return s.elapsed_time(e) / iters


def stage_table(wl: MTAWorkload, samples, peaks):
    """Per-stage device times of the forward as it runs in the step (CUDA events the library records on the launching
    stream between its kernels: `samples` = list of [(stage, ms)] per traced step) -> one row per kernel with its
    roofline.  A score-plane stage reads the lower triangle of its input planes once and writes the lower triangle of
    its output planes once (nothing above the diagonal is touched inside the forward): HBM-bound.  The score + conv
    kernel and P.V are contractions; the former is bound by the tensor pipe (its ncu profile: tensor pipe the busiest
    unit, DRAM under 20 %), so its row is in TFLOP/s, with the bytes it moves beside it."""
    es = torch.empty(0, dtype=wl.dtype).element_size()
    lower = wl.lower_elements()
    qkv_bytes = float(es) * wl.B * wl.H * wl.S * wl.D
    acc = {}
    for step in samples:
        for name, ms in step:
            acc.setdefault(name, []).append(ms)
    out = []
    for name, vals in acc.items():
        ms = sum(vals) / len(vals)
        row = {"kernel": name, "ms": ms, "samples": len(vals)}
        if name in ("qk_scores", "pv", "qk_scores+conv1"):
            nbytes = float(es) * lower + 2 * qkv_bytes        # one score triangle written (read) + two operands
            flops = (2.0 * wl.D + (2.0 * wl.cq * wl.ck if name == "qk_scores+conv1" else 0.0)) * lower
            row.update(tflops=flops / (ms * 1e-3) / 1e12, gbs=nbytes / (ms * 1e-3) / 1e9)
        else:
            nbytes = 2.0 * es * lower
        if name == "qk_scores+conv1":
            ach = row["tflops"]
            row.update(bound="tensor", flops_algorithmic=flops, achieved=ach, peak=peaks["bf16_tflops"], unit="TFLOP/s",
                       frac=ach / peaks["bf16_tflops"])
        else:
            ach = nbytes / (ms * 1e-3) / 1e9
            row.update(bound="hbm", bytes_algorithmic=nbytes, achieved=ach, peak=peaks["hbm_gbs"], unit="GB/s",
                       frac=ach / peaks["hbm_gbs"])
        out.append(row)
    return out


def standalone_table(wl: MTAWorkload, d, dev, peaks):
    """Configs 2 and 3 (stand-alone conv and head mix on a (4,16,2048,2048) bf16 plane; 805 437 440 algorithmic bytes
    each, inputs of 512 MiB > L2) and fusion tier F1 (the conv attention at the workload's shape), timed alone."""
    from multitokenatention_triton_b200 import _lib, ops
    out = {}
    g = torch.Generator(device=dev).manual_seed(21)
    x = torch.randn(4, 16, 2048, 2048, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(16, 6, 11, device=dev, generator=g) * 66 ** -0.5).to(torch.bfloat16)
    ms = event_time_ms(lambda: ops.conv2d_fwd(x, w, True), 20)
    out["c2_conv"] = {"kernel": "mta_conv2d_fwd 6x11 causal (4,16,2048,2048) bf16", "ms": ms, "bound": "hbm",
                      "bytes_algorithmic": C23_BYTES, "achieved": C23_BYTES / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                      "unit": "GB/s", "frac": C23_BYTES / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                      "frac_of_nominal_8000": C23_BYTES / (ms * 1e-3) / 1e9 / NOMINAL["hbm_gbs"]}
    x = torch.softmax(torch.tril(x.float()) + torch.triu(torch.full((2048, 2048), float("-inf"), device=dev), 1), -1).to(torch.bfloat16)
    W = (torch.eye(16, device=dev) + 0.02 ** 0.5 * torch.randn(16, 16, device=dev, generator=g)).to(torch.bfloat16)
    ms = event_time_ms(lambda: ops.head_linear_fwd(x, W, True, 0.0), 20)
    out["c3_head_mix"] = {"kernel": "mta_head_linear_fwd 16x16 causal (4,16,2048,2048) bf16", "ms": ms, "bound": "hbm",
                          "bytes_algorithmic": C23_BYTES, "achieved": C23_BYTES / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                          "unit": "GB/s", "frac": C23_BYTES / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                          "frac_of_nominal_8000": C23_BYTES / (ms * 1e-3) / 1e9 / NOMINAL["hbm_gbs"]}
    del x
    torch.cuda.empty_cache()
    ms = event_time_ms(lambda: ops.conv_attn_fwd(d["q"], d["k"], d["v"], d["w1"], True, wl.D ** -0.5), 10)
    flops = (4.0 * wl.D + 2.0 * wl.cq * wl.ck) * wl.lower_elements()
    out["f1_conv_attn"] = {"kernel": f"mta_conv_attn_fwd {wl.cq}x{wl.ck} causal B{wl.B} H{wl.H} S{wl.S} D{wl.D} (one kernel, no score plane)",
                           "ms": ms, "bound": "tensor", "flops_algorithmic": flops, "achieved": flops / (ms * 1e-3) / 1e12,
                           "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": flops / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
                           "tokens_per_s": wl.tokens / (ms * 1e-3),
                           "workspace_bytes": int(_lib.lib().mta_conv_attn_workspace_bytes(wl.B, wl.H, wl.S, wl.D, wl.cq, wl.ck, 1,
                                                                                           _lib.DTYPE_CODE[wl.dtype], _lib.DTYPE_CODE[wl.dtype]))}
    return out


def reference_gpu_numbers(wl: MTAWorkload, limit_s: float = 240.0) -> dict:
    """The reference's Triton modules timed on this GPU by oracle/ref_gpu_bench.py in a child process."""
    script = os.path.join(ROOT, "oracle", "ref_gpu_bench.py")
    try:
        r = subprocess.run([sys.executable, script, "--batch", str(wl.B), "--seq", str(wl.S), "--heads", str(wl.H)],
                           capture_output=True, text=True, timeout=limit_s)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"the reference's GPU path did not finish within {limit_s:.0f} s"}
    for line in reversed(r.stdout.strip().splitlines()):
        try:
            return json.loads(line)
        except ValueError:
            continue
    return {"unavailable": f"no result (exit code {r.returncode}): {r.stderr.strip()[-300:]}"}


def copy_rates(dev, nbytes_h2d: int, nbytes_d2h: int, barrier) -> dict:
    """Bare pinned host -> device and device -> host copies of one step's bytes, all ranks at once."""
    h = torch.empty(nbytes_h2d, dtype=torch.uint8).pin_memory()
    g = torch.empty(nbytes_h2d, dtype=torch.uint8, device=dev)
    ho = torch.empty(nbytes_d2h, dtype=torch.uint8).pin_memory()
    go = torch.empty(nbytes_d2h, dtype=torch.uint8, device=dev)
    out = {}
    for name, fn, n in (("h2d", lambda: g.copy_(h, non_blocking=True), nbytes_h2d),
                        ("d2h", lambda: ho.copy_(go, non_blocking=True), nbytes_d2h)):
        fn()
        barrier()
        ms = event_time_ms(fn, 5, warmup=1)
        barrier()
        out[name + "_gbs"] = n / (ms * 1e-3) / 1e9
    # both directions at once, as the pipelined forward does
    s2 = torch.cuda.Stream(device=dev)
    barrier()
    t0 = time.perf_counter()
    for _ in range(5):
        g.copy_(h, non_blocking=True)
        with torch.cuda.stream(s2):
            ho.copy_(go, non_blocking=True)
    torch.cuda.synchronize()
    out["both_gbs"] = 5 * (nbytes_h2d + nbytes_d2h) / (time.perf_counter() - t0) / 1e9
    return out


def strong_record(tag: str, wl: MTAWorkload, world: int, rank: int, dev, dist, steps: int = 5) -> dict:
    """A FIXED batch split over the ranks by sharding.plan_shards: every rank draws only its own batch elements (seeded
    by batch element), computes its shard, and the shards are gathered with NCCL (timed separately).  Rank 0 then
    recomputes one foreign shard from a fresh draw of its inputs and compares it bit for bit with the gathered one."""
    from multitokenatention_triton_b200 import sharding
    plan = sharding.plan_shards(wl.B, wl.S, world, row_align=128)
    b0, b1, r0, r1 = plan[rank]
    weights = [t.to(dev) for t in (make_mta_weights(wl)[n] for n in ("w1", "W1", "w2", "W2"))]

    def draw(bb0, bb1):
        parts = [device_qkv(wl, b, dev) for b in range(bb0, bb1)]
        return [torch.cat([p[n] for p in parts]) for n in ("q", "k", "v")]

    q, k, v = draw(b0, b1)

    def sync():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    local = None
    for _ in range(2):
        local = sharding.local_forward(q, k, v, weights, plan[rank])
    sync()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        local = sharding.local_forward(q, k, v, weights, plan[rank])
    e.record()
    sync()
    t = torch.tensor([s.elapsed_time(e) / steps], device=dev, dtype=torch.float64)
    tmin = t.clone()
    rec = {"workload": f"{tag}: B{wl.B} H{wl.H} S{wl.S} D{wl.D}", "plan": [list(p) for p in plan]}
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tmin, op=dist.ReduceOp.MIN)
        full = sharding.gather_outputs(local, plan, wl.B, wl.S)          # warm-up of the collective
        sync()
        s.record()
        full = sharding.gather_outputs(local, plan, wl.B, wl.S)
        e.record()
        sync()
        tg = torch.tensor([s.elapsed_time(e)], device=dev, dtype=torch.float64)
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        rec["gather_ms"] = float(tg.item())
        rec["gather_bytes_per_rank"] = int(local.numel() * local.element_size())
        if rank == 0:
            fb0, fb1, fr0, fr1 = plan[world - 1]                           # the last rank's shard
            del q, k, v
            fq, fk, fv = draw(fb0, fb1)
            again = sharding.local_forward(fq, fk, fv, weights, plan[world - 1])
            rec["foreign_shard_bit_identical"] = bool(torch.equal(again, full[fb0:fb1, :, fr0:fr1]))
            rec["own_shard_bit_identical"] = bool(torch.equal(local, full[b0:b1, :, r0:r1]))
        del full
    ms = float(t.item())
    rec.update(ms_per_step=ms, ms_fastest_rank=float(tmin.item()), tokens_per_s=wl.tokens / (ms * 1e-3), n_gpus=world,
               scaling="strong", timing="CUDA events per rank, max over ranks")
    if "gather_ms" in rec:
        rec["tokens_per_s_with_gather"] = wl.tokens / ((ms + rec["gather_ms"]) * 1e-3)
        rec["gather_share"] = rec["gather_ms"] / (ms + rec["gather_ms"])
    del local
    torch.cuda.empty_cache()
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch size (smaller captures)")
    ap.add_argument("--seq", type=int, default=0, help="override the workload's sequence length (smaller captures)")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip e2e, the CPU baseline, the stand-alone kernels, the reference's GPU path and the strong-scaling records")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    wl = WORKLOADS[args.workload]
    if args.batch or args.seq:
        wl = dataclasses.replace(wl, B=args.batch or wl.B, S=args.seq or wl.S, name=wl.name + "-reduced")

    if args.impl == "reference":
        reference_arm(args, wl, rank, world)
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device: this package has no CPU path"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from multitokenatention_triton_b200 import MTAAttentionTriton, _lib

    peaks, peak_kind = measured_peaks()
    my_wl = dataclasses.replace(wl, seed=wl.seed + 1000 * rank)          # every rank its own batch (weak scaling)
    inp = make_mta_inputs(my_wl)
    host = {k: inp[k].pin_memory() for k in ("q", "k", "v")}
    d = {k: t.to(dev) for k, t in inp.items()}
    cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=wl.cq, key_kernel_size=wl.ck,
                                after_sm_query_kernel_size=wl.cq2, after_sm_key_kernel_size=wl.ck2,
                                pre_sm_linear_head=True, post_sm_linear_head=True, pad_key="both",
                                init_method="identity", dim=wl.H * wl.D)
    model = MTAAttentionTriton(wl.H, cfg, dropout=0.0, causal=True).to(dev).to(wl.dtype).eval()
    with torch.no_grad():
        model.mta_conv_triton.weight.copy_(d["w1"])
        model.wpsm_triton.weight.copy_(d["W1"])
        model.mta_conv_after_sm_triton.weight.copy_(d["w2"])
        model.wposm_triton.weight.copy_(d["W2"])

    def step():
        with torch.no_grad():
            return model(d["q"], d["k"], d["v"], None, None)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput --------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    _lib.device_status()
    _lib.reset_launch_count()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    _lib.set_stage_trace(True)                     # the library brackets its kernels with events on this stream
    s.record()
    for _ in range(args.steps):
        step()
    e.record()
    barrier()
    launches = _lib.launch_count()
    # A device-side wait that gave up makes every later kernel return at once: no number may come out of such a run.
    _lib.device_status()
    stage_samples = [_lib.stage_times_ms()]        # the last step of the timed region ...
    for _ in range(4):                             # ... and four more steps, read one by one
        step()
        stage_samples.append(_lib.stage_times_ms())
    _lib.set_stage_trace(False)
    _lib.device_status()
    ms_total = torch.tensor([s.elapsed_time(e)], device=dev, dtype=torch.float64)
    clocks = sampler.stop() if rank == 0 else None
    if dist is not None:
        dist.all_reduce(ms_total, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms_total.item()) / args.steps
    tokens = wl.tokens * world
    value = tokens / (ms_per_step * 1e-3)

    # ---- end to end with host buffers ------------------------------------------------------------
    e2e, h2d = None, None
    if not args.no_extras:
        out_host = torch.empty((wl.B, wl.H, wl.S, wl.D), dtype=wl.dtype).pin_memory()

        def e2e_step():
            with torch.no_grad():                            # blocks until out_host is complete
                model.forward_host(host["q"], host["k"], host["v"], out=out_host)

        for _ in range(2):
            e2e_step()
        barrier()
        n_e2e = max(2, min(args.steps, 5))
        t0 = time.perf_counter()                             # the call runs on the library's own streams and blocks:
        for _ in range(n_e2e):                               # the host clock around it is the end-to-end time
            e2e_step()
        torch.cuda.synchronize()
        t = torch.tensor([(time.perf_counter() - t0) * 1e3], device=dev, dtype=torch.float64)
        barrier()
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        _lib.device_status()
        h2d_rank = sum(host[k].numel() * host[k].element_size() for k in host)
        d2h_rank = out_host.numel() * out_host.element_size()
        e2e = {"value": tokens / (float(t.item()) / n_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": world * h2d_rank,
               "d2h_bytes_per_step": world * d2h_rank, "steps": n_e2e,
               "path": "MTAAttentionTriton.forward_host -> mta_fused_fwd_host: batch chunks on three streams, host clock around the blocking call"}
        # the ceiling of that number: what the host <-> device links carry when every rank copies at once
        from multitokenatention_triton_b200 import ops
        ops.host_pipeline_release(dev)
        r = copy_rates(dev, h2d_rank, d2h_rank, barrier)
        rt = torch.tensor([r["h2d_gbs"], r["d2h_gbs"], r["both_gbs"]], device=dev, dtype=torch.float64)
        rmin = rt.clone()
        if dist is not None:
            dist.all_reduce(rt, op=dist.ReduceOp.MAX)
            dist.all_reduce(rmin, op=dist.ReduceOp.MIN)
        step_bytes = h2d_rank + d2h_rank
        h2d = {"per_rank_gbs": {"h2d_min": float(rmin[0]), "h2d_max": float(rt[0]), "d2h_min": float(rmin[1]), "d2h_max": float(rt[1]),
                                "both_directions_min": float(rmin[2]), "both_directions_max": float(rt[2])},
               "bytes_per_rank_per_step": step_bytes,
               "e2e_ceiling_tokens_per_s": tokens / (step_bytes / (float(rmin[2]) * 1e9)),
               "what": "pinned buffers of one step's q,k,v (host to device) and output (device to host), copied by every rank at the "
                       "same time; the ceiling is the step's bytes over the slowest rank's two-directional rate",
               "cpu_affinity_cores": host_threads()}
        del out_host

    # ---- per-kernel breakdown and rooflines (rank 0) ---------------------------------------------
    roofline, roofline_step, stages, cpu, standalone, reference_gpu = None, None, None, None, None, None
    step_tflops = wl.algorithmic_flops() / (ms_per_step * 1e-3) / 1e12            # per GPU: every rank runs the same step
    if rank == 0:
        stages = stage_table(wl, stage_samples, peaks)
        top = max(stages, key=lambda r: r["ms"])
        per_lower = dram_bytes_per_score().get(top["kernel"])
        roofline = {"kernel": top["kernel"], "ms": top["ms"], "bound": top["bound"], "achieved": top["achieved"], "peak": top["peak"],
                    "unit": top["unit"], "frac": top["frac"],
                    "traffic": per_lower * wl.lower_elements() if per_lower is not None else None, "peak_kind": peak_kind}
        roofline_step = {"bound": "tensor", "achieved": step_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": step_tflops / peaks["bf16_tflops"], "per": "GPU", "flops_algorithmic_per_gpu": wl.algorithmic_flops(),
                         "frac_of_nominal_2250": step_tflops / NOMINAL["bf16_tflops"], "peak_kind": peak_kind}
    if not args.no_extras:
        if rank == 0 and world == 1:
            standalone = standalone_table(wl, d, dev, peaks)
            _lib.device_status()
            cpu = cpu_baseline(wl, 15.0)
    del d, host, model
    torch.cuda.empty_cache()
    strong = None
    if not args.no_extras and args.workload == "c4" and not (args.batch or args.seq):
        strong = {}
        strong["c4"] = strong_record("c4", WORKLOADS["c4"], world, rank, dev, dist)
        free, _ = torch.cuda.mem_get_info(dev)
        c5 = WORKLOADS["c5"]
        per_rank_b = -(-c5.B // world)
        need = _lib.lib().mta_workspace_bytes(per_rank_b, c5.H, c5.S, c5.D, c5.cq, c5.ck, c5.cq2, c5.ck2, 0, c5.S,
                                              _lib.DTYPE_CODE[c5.dtype]) + 6 * per_rank_b * c5.H * c5.S * c5.D * 2
        if need < free * 0.9:
            strong["c5"] = strong_record("c5", c5, world, rank, dev, dist, steps=3)
        else:
            strong["c5"] = {"unavailable": f"needs {need / 2**30:.0f} GiB per rank, {free / 2**30:.0f} GiB free"}
        if world > 1:                                     # fewer batch elements than ranks: query-row blocks, halo rows recomputed
            rows_wl = dataclasses.replace(WORKLOADS["c4"], B=max(1, world // 4), name="c4-rows")
            strong["rows"] = strong_record("c4 shape, batch smaller than the rank count", rows_wl, world, rank, dev, dist)
        _lib.device_status()
    if not args.no_extras and rank == 0 and world == 1:
        reference_gpu = reference_gpu_numbers(wl)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": str(wl.dtype).split(".")[-1], "data": "synthetic",
            "config": job_config(wl, world),
            "gpu_launches": launches, "clocks": clocks, "e2e": e2e, "roofline": roofline, "roofline_step": roofline_step,
            "cpu_baseline": cpu,
            "step_tflops_algorithmic_per_gpu": step_tflops,
            "step_frac_of_bf16_peak": step_tflops / peaks["bf16_tflops"],
            "peaks": dict(peaks, kind=peak_kind, nominal=NOMINAL), "kernels": stages, "standalone": standalone,
            "reference_gpu": reference_gpu, "strong": strong, "h2d": h2d,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
