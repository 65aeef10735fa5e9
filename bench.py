"""Benchmark of the MTA forward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload c4]

One "step" is one full MTA forward (QK^T/sqrt(D) -> conv -> head mix -> softmax -> conv -> head mix -> @V)
over one synthetic batch of the workload (default c4: B8 H16 S4096 D128 bf16, causal, conv 6x11, head
mixes 16x16, post-softmax conv 3x3).  Rank 0 prints ONE JSON line.

  value     tokens/s of the whole job with inputs resident in HBM (CUDA events, max over ranks)
  e2e       tokens/s through the module's forward_host with HOST buffers: pinned host -> device copies of
            q,k,v and the device -> host copy of the output are inside the timed region (the library
            overlaps them with the computation, batch chunk by batch chunk)
  roofline  the dominant kernel of the step, timed alone with CUDA events, against the measured peak
  cpu_baseline  the CPU port of the reference's algorithm (oracle/, C + OpenMP) on a bounded sample of
            the same workload, on this box's host cores (rank 0, N=1 only)

With N > 1 (torchrun, one rank per GPU) every rank runs the same-size workload on its own seeded batch
(weak scaling, no data-path collective); the only communication is the barrier and the max-reduction
of the measured time.

`--impl reference` times the CPU port of the reference algorithm instead (all host threads).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from multitokenatention_triton_b200.synthetic import WORKLOADS, MTAWorkload, make_mta_inputs  # noqa: E402

METRIC = "MTA fwd tokens/s"
NOMINAL = {"hbm_gbs": 8000.0, "bf16_tflops": 2250.0}
FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"]))}, "measured"
    return dict(FALLBACK, bf16_tflops_sustained=1400.0), "fallback"


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


# ---------------------------------------------------------------------------------------------------
_CPU_INPUTS = {}


def cpu_port_tokens_per_s(wl: MTAWorkload, budget_s: float, threads: int = 0):
    """Times the CPU port of the reference algorithm (oracle/mta_oracle.c, OpenMP) on a block of query rows
    of batch element 0 centred on S/2, where a row's cost equals the workload's mean cost per token.
    The block is grown until it needs about `budget_s` seconds.  Returns (tokens/s, cores, description)."""
    from oracle import mta_oracle as orc
    if not threads:      # all the cores this process may run on, whatever OMP_NUM_THREADS a launcher exported
        threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    orc.set_threads(threads)
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
    reps = 1
    if n == wl.S and t < budget_s:             # a whole batch element is too short a sample: time several (same cost each)
        reps = int(min(wl.B, max(1, budget_s // max(t, 1e-3))))
        t0 = time.perf_counter()
        for _ in range(reps):
            run(n)
        t = time.perf_counter() - t0
    desc = (f"CPU port (C, OpenMP) of the reference algorithm on batch element 0, query rows "
            f"[{max(0, mid - n // 2)},{max(0, mid - n // 2) + n}) of {wl.S} (block centred on S/2 = mean cost per token), "
            f"all {wl.H} heads, {reps} time(s), {t:.1f} s")
    return reps * n / t, cores, desc


def reference_arm(args, wl: MTAWorkload, rank: int):
    if rank != 0:
        return
    per_step_budget = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    vals, cores, desc = [], 1, ""
    # every host core this process may use: torchrun exports OMP_NUM_THREADS=1 to its workers, and the other ranks of
    # this arm exit without work, so the cores are free
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    for i in range(args.warmup + args.steps):
        v, cores, desc = cpu_port_tokens_per_s(wl, per_step_budget, threads=threads)
        if i >= args.warmup:
            vals.append(v)
    value = statistics.mean(vals) if vals else 0.0
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": (wl.tokens / value * 1e3) if value else None,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64 accumulate on %s inputs" % str(wl.dtype).split(".")[-1],
        "data": "synthetic", "config": {"workload": workload_name(wl)},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_name(wl: MTAWorkload) -> str:
    return (f"{wl.name}: full MTA forward B{wl.B} H{wl.H} S{wl.S} D{wl.D} {str(wl.dtype).split('.')[-1]} causal, "
            f"conv {wl.cq}x{wl.ck} + head mix {wl.H}x{wl.H} + softmax + conv {wl.cq2}x{wl.ck2} + head mix, seed {wl.seed}")


# ---------------------------------------------------------------------------------------------------
def event_time_ms(fn, iters: int) -> float:
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    e.synchronize()
    return s.elapsed_time(e) / iters


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per lower-triangle score element of one launch, from ncu
# captures of smaller cases of the same kernels (the summaries under profiles/ give the commands); a launch's traffic
# grows in proportion to the triangle it processes.
NCU_DRAM_BYTES_PER_LOWER_ELEMENT = {       # profiles/mta_forward_kernels_b1_s4096.md (B1 H16 S4096: 134.25 M scores)
    "qk_scores+conv1": 2.03, "qk_scores": 2.01, "conv1": 4.07, "head_mix1+softmax": 3.62, "conv2": 3.99, "head_mix2": 3.71,
    "pv": 2.28,
}


def stage_table(wl: MTAWorkload, samples, peaks):
    """Per-stage device times of the forward as it runs in the step (CUDA events the library records on the launching
    stream between its kernels: `samples` = list of [(stage, ms)] per traced step) -> one row per kernel with its
    roofline.  Algorithmic work of a launch: a score-plane stage reads the lower triangle of its input planes once and
    writes the lower triangle of its output planes once (nothing above the diagonal is touched inside the forward);
    the two contractions are counted by their flops and by the triangle they write / read."""
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
        if name in ("qk_scores", "pv"):
            nbytes = float(es) * lower + 2 * qkv_bytes        # the score triangle written (read) + two operands
            row.update(bound="hbm", tflops=2.0 * wl.D * lower / (ms * 1e-3) / 1e12)
        elif name == "qk_scores+conv1":
            nbytes = float(es) * lower + 2 * qkv_bytes        # Q and K read, the conv's triangle written; no score plane
            row.update(bound="hbm", tflops=(2.0 * wl.D + 2.0 * wl.cq * wl.ck) * lower / (ms * 1e-3) / 1e12)
        else:
            nbytes = 2.0 * es * lower
            row.update(bound="hbm")
        ach = nbytes / (ms * 1e-3) / 1e9
        row.update(bytes_algorithmic=nbytes, achieved=ach, peak=peaks["hbm_gbs"], unit="GB/s", frac=ach / peaks["hbm_gbs"])
        out.append(row)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="override the workload's batch size (smaller captures)")
    ap.add_argument("--seq", type=int, default=0, help="override the workload's sequence length (smaller captures)")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-kernel breakdown, e2e and CPU baseline")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    wl = WORKLOADS[args.workload]
    if args.batch or args.seq:
        import dataclasses
        wl = dataclasses.replace(wl, B=args.batch or wl.B, S=args.seq or wl.S, name=wl.name + "-reduced")

    if args.impl == "reference":
        reference_arm(args, wl, rank)
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
    import types
    import dataclasses

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
    stage_samples = [_lib.stage_times_ms()]        # the last step of the timed region ...
    for _ in range(4):                             # ... and four more steps, read one by one
        step()
        stage_samples.append(_lib.stage_times_ms())
    _lib.set_stage_trace(False)
    ms_total = torch.tensor([s.elapsed_time(e)], device=dev, dtype=torch.float64)
    clocks = sampler.stop() if rank == 0 else None
    if dist is not None:
        dist.all_reduce(ms_total, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms_total.item()) / args.steps
    tokens = wl.tokens * world
    value = tokens / (ms_per_step * 1e-3)

    # ---- end to end with host buffers ------------------------------------------------------------
    e2e = None
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
        h2d = world * sum(host[k].numel() * host[k].element_size() for k in host)      # whole job, like the value
        d2h = world * out_host.numel() * out_host.element_size()
        e2e = {"value": tokens / (float(t.item()) / n_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "steps": n_e2e,
               "path": "MTAAttentionTriton.forward_host -> mta_fused_fwd_host: batch chunks on three streams, host clock around the blocking call"}

    # ---- per-kernel breakdown and roofline (rank 0) ----------------------------------------------
    roofline, stages, cpu = None, None, None
    if rank == 0:
        stages = stage_table(wl, stage_samples, peaks)
        top = max(stages, key=lambda r: r["ms"])
        per_lower = NCU_DRAM_BYTES_PER_LOWER_ELEMENT.get(top["kernel"])
        roofline = {"kernel": top["kernel"], "bound": top["bound"], "achieved": top["achieved"], "peak": top["peak"],
                    "unit": top["unit"], "frac": top["frac"],
                    "traffic": per_lower * wl.lower_elements() if per_lower is not None else None, "peak_kind": peak_kind}
    if rank == 0 and world == 1 and not args.no_extras:
        v, cores, desc = cpu_port_tokens_per_s(wl, 15.0)
        cpu = {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc}

    if rank == 0:
        flops = wl.algorithmic_flops() * world
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": str(wl.dtype).split(".")[-1], "data": "synthetic",
            "config": {"workload": workload_name(wl), "global_batch": wl.B * world, "parallelism": f"batch-sharded x{world}, no collective",
                       "l2": "working set per step (>= 4 GB of score planes at c4) exceeds the 126 MB L2; no explicit flush"},
            "gpu_launches": launches, "clocks": clocks, "e2e": e2e, "roofline": roofline, "cpu_baseline": cpu,
            "step_tflops_algorithmic": flops / (ms_per_step * 1e-3) / 1e12,
            "step_frac_of_bf16_peak": flops / (ms_per_step * 1e-3) / 1e12 / peaks["bf16_tflops"],
            "peaks": dict(peaks, kind=peak_kind, nominal=NOMINAL), "kernels": stages,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
