"""Times the reference's own Triton path on the GPU this process sees: the "kernel to beat" numbers of bench.py.

    python oracle/ref_gpu_bench.py [--items c2_conv,c3_head_mix,f1_conv_attn,f3_mta] [--batch 8] [--seq 4096]

Runs as a child process of bench.py (a fault inside a reference kernel then cannot take the benchmark's own CUDA
context with it) and prints ONE JSON object: item -> {"ms": ..., "shape": ...} or {"unavailable": "<why>"}.
Modules come unmodified from oracle/_ref/ (make_ref.py).  Timing follows the reference's benchmark_forward
(benchmark_mta_attention.py:40-64): 3 warm-up runs, 10 timed runs under torch.no_grad(), here bracketed by CUDA events.
Inputs are seeded normal tensors drawn on the device with the shapes of the benchmark configurations.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from oracle import ref_runner as rr  # noqa: E402

WARMUP_RUNS, BENCHMARK_RUNS = 3, 10


def timed(fn):
    with torch.no_grad():
        for _ in range(WARMUP_RUNS):
            fn()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(BENCHMARK_RUNS):
            fn()
        e.record()
        e.synchronize()
    return s.elapsed_time(e) / BENCHMARK_RUNS


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--items", default="c2_conv,c3_head_mix,f1_conv_attn,f3_mta")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=16)
    args = ap.parse_args()
    out = {}
    if not rr.available():
        print(json.dumps({"unavailable": "oracle/_ref is empty (python oracle/make_ref.py <reference checkout>)"}))
        return
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(1234)
    dt = torch.bfloat16
    H, D = args.heads, 128
    for item in args.items.split(","):
        try:
            if item == "c2_conv":
                x = (torch.randn(4, H, 2048, 2048, device=dev, generator=g) * 1.0).to(dt)
                m = rr.module("convolution_2d_trit").Conv2dTriton(H, (6, 11), causal=True).to(dev).to(dt)
                with torch.no_grad():
                    m.weight.copy_(torch.randn(H, 6, 11, device=dev, generator=g) * 66 ** -0.5)
                out[item] = {"ms": timed(lambda: m(x)), "shape": f"Conv2dTriton 6x11 causal on (4,{H},2048,2048) bf16"}
                del x, m
            elif item == "c3_head_mix":
                x = torch.softmax(torch.randn(4, H, 2048, 2048, device=dev, generator=g), -1).to(dt)
                m = rr.module("triton_linear_head").TritonLinearHead(H, causal=True, output_value=0.0).to(dev).to(dt)
                out[item] = {"ms": timed(lambda: m(x)), "shape": f"TritonLinearHead {H}x{H} causal on (4,{H},2048,2048) bf16"}
                del x, m
            elif item in ("f1_conv_attn", "f3_mta"):
                B, S = args.batch, args.seq
                q, k, v = (torch.randn(B, H, S, D, device=dev, generator=g).to(dt) for _ in range(3))
                if item == "f1_conv_attn":
                    m = rr.module("conv_attention_triton").TritonConvAttention(H, (6, 11), causal=True).to(dev).to(dt)
                    with torch.no_grad():
                        m.weight.copy_(torch.randn(H, 6, 11, device=dev, generator=g) * 66 ** -0.5)
                        m.weight[:, 5, 5] += 1.0
                    ms = timed(lambda: m(q, k, v, True, D ** -0.5))
                    out[item] = {"ms": ms, "tokens_per_s": B * S / (ms * 1e-3),
                                 "shape": f"TritonConvAttention 6x11 causal, B{B} H{H} S{S} D{D} bf16"}
                else:
                    from multitokenatention_triton_b200.synthetic import MTAWorkload
                    wl = MTAWorkload("ref", B, H, S, D, 6, 11, dtype=dt)
                    w = {"w1": torch.randn(H, 6, 11, device=dev, generator=g) * 66 ** -0.5,
                         "W1": torch.eye(H, device=dev) + 0.02 ** 0.5 * torch.randn(H, H, device=dev, generator=g),
                         "w2": torch.zeros(H, 3, 3, device=dev),
                         "W2": torch.eye(H, device=dev) + 0.02 ** 0.5 * torch.randn(H, H, device=dev, generator=g)}
                    w["w1"][:, 5, 5] += 1.0
                    w["w2"][:, 2, 1] = 1.0
                    m = rr.triton_mta(wl, w, dev, dt)
                    ms = timed(lambda: m(q, k, v, None, None))
                    out[item] = {"ms": ms, "tokens_per_s": B * S / (ms * 1e-3),
                                 "shape": f"MTAAttentionTriton.forward, B{B} H{H} S{S} D{D} bf16, conv 6x11 + 3x3, head mixes {H}x{H}"}
                del q, k, v, m
            else:
                out[item] = {"unavailable": "unknown item"}
        except Exception as exc:  # noqa: BLE001 - reported, not hidden
            out[item] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
        torch.cuda.empty_cache()
    out["method"] = f"{WARMUP_RUNS} warm-up + {BENCHMARK_RUNS} timed runs, CUDA events, torch.no_grad()"
    print(json.dumps(out))


if __name__ == "__main__":
    main()
