"""Micro-benchmarks of the stand-alone kernels on the configurations their roofline targets are quoted on.

    python -m multitokenatention_triton_b200.microbench [conv2d|head_linear|softmax|mix_softmax|qk|pv|backward|conv_attn|graph|all] [--variant V]
                                                        [--batch N] [--seq S] [--iters K]

  conv2d       causal depthwise conv 6x11 on a (B=4, H=16, S=2048, S) bf16 score plane
  head_linear  16x16 head mix on post-softmax probabilities of the same shape
  graph        the whole forward (five launches) at --batch/--heads/--seq/--dim, launched call by call and replayed
               from a CUDA graph: what stream capture saves where the forward is launch-bound (not part of "all")

Each kernel is timed alone with CUDA events on the launching stream (3 warm-up launches, then K timed ones;
input + output of one launch exceed the 126 MB L2).  One JSON line per kernel:
algorithmic bytes = read the lower triangle once + write the whole output (zero / fill included), divided by
the mean launch time, against the measured copy bandwidth in MEASURED_PEAKS.json when present.
--variant selects 0 auto, 1 CUDA-core, 2 tensor-core (see mta_set_variant).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import _lib, ops
from .synthetic import make_conv_inputs, make_head_linear_inputs

ROOT = os.path.abspath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def _time(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    e.synchronize()
    return s.elapsed_time(e) / iters


def _line(name, ms, nbytes=None, flops=None, **extra):
    hbm, tf, kind = _peaks()
    out = {"kernel": name, "ms": ms, "peak_kind": kind}
    if nbytes is not None:
        out.update(bound="hbm", bytes_algorithmic=nbytes, achieved=nbytes / ms / 1e6, peak=hbm, unit="GB/s",
                   frac=nbytes / ms / 1e6 / hbm, frac_of_nominal_8000=nbytes / ms / 1e6 / 8000.0)
    else:
        out.update(bound="tensor", flops_algorithmic=flops, achieved=flops / ms / 1e9, peak=tf, unit="TFLOP/s",
                   frac=flops / ms / 1e9 / tf, frac_of_nominal_2250=flops / ms / 1e9 / 2250.0)
    out.update(extra)
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("which", nargs="?", default="all", choices=["conv2d", "head_linear", "softmax", "mix_softmax", "qk", "pv", "backward", "conv_attn", "graph", "all"])
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16", "float32"])
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    dtype = getattr(torch, a.dtype)
    es = torch.empty(0, dtype=dtype).element_size()
    N, C, S, D = a.batch, a.heads, a.seq, a.dim
    tri = S * (S + 1) // 2
    shape = f"B{N} H{C} S{S} {a.dtype}"
    for key in ("conv2d", "head_linear", "gemm"):
        _lib.set_variant(key, a.variant)

    if a.which in ("conv2d", "all"):
        inp = make_conv_inputs(N, C, S, D, 6, 11, dtype, seed=1)
        x, w = inp["x"].to(dev), inp["w"].to(dev)
        y = torch.empty_like(x)

        def run():
            _lib.check(_lib.lib().mta_conv2d_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), N, C, S, S, 6, 11, 1,
                                                 _lib.dtype_code(x), _lib.dtype_code(w), _lib.stream_ptr(dev)), "conv2d")
        ms = _time(run, a.iters)
        _line("conv2d 6x11 causal", ms, nbytes=es * N * C * (tri + S * S), shape=shape, variant=a.variant,
              lower_only_bytes=2 * es * N * C * tri)
        del x, y
    if a.which in ("head_linear", "softmax", "mix_softmax", "all"):
        inp = make_head_linear_inputs(N, C, S, dtype, seed=2)
        x, W = inp["x"].to(dev), inp["W"].to(dev)
        y = torch.empty_like(x)
        if a.which in ("head_linear", "all"):
            for fill in (0.0, float("-inf")):
                def run():
                    _lib.check(_lib.lib().mta_head_linear_fwd(x.data_ptr(), W.data_ptr(), y.data_ptr(), N, C, S, S, 1, fill,
                                                              _lib.dtype_code(x), _lib.dtype_code(W), _lib.stream_ptr(dev)),
                               "head_linear")
                ms = _time(run, a.iters)
                _line(f"head_linear {C}x{C} causal fill={fill}", ms, nbytes=es * N * C * (tri + S * S), shape=shape,
                      variant=a.variant)
        if a.which in ("softmax", "all"):
            ms = _time(lambda: ops.softmax_fwd(x, True, out=y), a.iters)
            _line("softmax causal rows", ms, nbytes=es * N * C * (tri + S * S), shape=shape)
        if a.which in ("mix_softmax", "all"):
            def run():
                _lib.check(_lib.lib().mta_head_linear_softmax_fwd(x.data_ptr(), W.data_ptr(), y.data_ptr(), N, C, S, S,
                                                                  _lib.dtype_code(x), _lib.dtype_code(W), _lib.stream_ptr(dev)),
                           "head_linear_softmax")
            ms = _time(run, a.iters)
            _line(f"head mix {C}x{C} + softmax, one pass", ms, nbytes=es * N * C * (tri + S * S), shape=shape)
        del x, y
    if a.which in ("backward", "all"):
        # gradients of the two stand-alone ops: dx moves read-lower + write-full like the forward; a weight gradient
        # reads the lower triangle of x and of dy
        from .synthetic import make_upstream_grad
        inp = make_conv_inputs(N, C, S, D, 6, 11, dtype, seed=1)
        x, w = inp["x"].to(dev), inp["w"].to(dev)
        g = make_upstream_grad((N, C, S, S), dtype, 1001).to(dev)
        ms = _time(lambda: ops.conv2d_bwd_input(g, w, True), a.iters)
        _line("conv2d 6x11 causal, input gradient", ms, nbytes=es * N * C * (tri + S * S), shape=shape, variant=a.variant)
        ms = _time(lambda: ops.conv2d_bwd_weight(x, g, (6, 11), True), a.iters)
        _line("conv2d 6x11 causal, weight gradient", ms, nbytes=2 * es * N * C * tri, shape=shape)
        hl = make_head_linear_inputs(N, C, S, dtype, seed=2)
        W = hl["W"].to(dev)
        x = hl["x"].to(dev)
        ms = _time(lambda: ops.head_linear_bwd_input(g, W, True), a.iters)
        _line(f"head_linear {C}x{C} causal, input gradient", ms, nbytes=es * N * C * (tri + S * S), shape=shape, variant=a.variant)
        ms = _time(lambda: ops.head_linear_bwd_weight(x, g, True), a.iters)
        _line(f"head_linear {C}x{C} causal, weight gradient", ms, nbytes=2 * es * N * C * tri, shape=shape)
        del x, g
    if a.which in ("qk", "pv", "all"):
        g = torch.Generator().manual_seed(3)
        q, k, v = (torch.randn(N, C, S, D, generator=g).to(dtype).to(dev) for _ in range(3))
        s = torch.zeros(N, C, S, S, dtype=dtype, device=dev)
        if a.which in ("qk", "all"):
            ms = _time(lambda: ops.qk_scores_fwd(q, k, D ** -0.5, True, out=s), a.iters)
            _line("qk_scores causal", ms, flops=2.0 * D * N * C * tri, shape=shape + f" D{D}", variant=a.variant,
                  write_gbs=es * N * C * tri / ms / 1e6)
        if a.which in ("pv", "all"):
            ms = _time(lambda: ops.pv_fwd(s, v, True), a.iters)
            _line("pv causal", ms, flops=2.0 * D * N * C * tri, shape=shape + f" D{D}", variant=a.variant,
                  read_gbs=es * N * C * tri / ms / 1e6)
    if a.which in ("conv_attn", "all"):
        # the conv attention softmax(scale * conv(Q K^T)) V (TritonConvAttention): one kernel for 16-bit causal problems
        g = torch.Generator().manual_seed(5)
        q, k, v = (torch.randn(N, C, S, D, generator=g).to(dtype).to(dev) for _ in range(3))
        w = (torch.randn(C, 6, 11, generator=g) / 66 ** 0.5).to(dtype).to(dev)
        ms = _time(lambda: ops.conv_attn_fwd(q, k, v, w, True, D ** -0.5), a.iters)
        _line("conv attention 6x11 causal", ms, flops=(4.0 * D + 2.0 * 66) * N * C * tri, shape=shape + f" D{D}",
              tokens_per_s=N * S / (ms * 1e-3))
    if a.which == "graph":
        from .synthetic import MTAWorkload, make_mta_inputs
        wl = MTAWorkload("graph", N, C, S, D, 6, 11, 3, 3, dtype, 3, random_post_conv=True)
        t = {k: v.to(dev) for k, v in make_mta_inputs(wl).items()}
        out = torch.empty_like(t["q"])
        nbytes = _lib.lib().mta_workspace_bytes(N, C, S, D, 6, 11, 3, 3, 0, S, _lib.dtype_code(t["q"]))
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)

        def run():
            ops.mta_fused_fwd(t["q"], t["k"], t["v"], t["w1"], t["W1"], t["w2"], t["W2"], True, out=out, workspace=ws)
        run()                                                  # first call: per-device setup, before any capture
        _lib.device_status()
        eager = _time(run, a.iters)
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            run()
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                run()
        torch.cuda.synchronize()
        ref = out.clone()
        out.zero_()
        replay = _time(graph.replay, a.iters)
        print(json.dumps({"kernel": "full forward, call by call against CUDA-graph replay", "shape": shape + f" D{D}",
                          "ms_eager": eager, "ms_graph": replay, "bit_identical": bool(torch.equal(out, ref)),
                          "tokens_per_s_graph": N * S / (replay * 1e-3)}), flush=True)
    _lib.device_status()


if __name__ == "__main__":
    main()
