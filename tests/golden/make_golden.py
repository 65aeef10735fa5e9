"""Generate the golden vectors in this directory from the reference project's own PyTorch code.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's modules unmodified (mta_attention_pytorch.MTAAttention,
convolution_2d_trit.pytorch_conv, conv_attention_pytorch.ConvAttention), feeds them the seeded
inputs of multitokenatention_triton_b200.synthetic and stores the outputs as float32 arrays in
golden_*.npz.  Inputs are not stored: the tests regenerate them from the same seeds.

Two shims, neither of which edits the reference: `torch.tensor(..., device="cuda")` in
MTAAttention.forward is redirected to the CPU, and the four MTA weights are assigned directly
instead of through reset_mta_parameters (which calls .cuda()).  If Triton's interpreter can run the
reference's conv and head-linear kernels on the CPU their outputs are stored as well; they pin the
fill values written above the diagonal.
"""
import os
import sys
import types

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))

from multitokenatention_triton_b200.synthetic import (  # noqa: E402
    WORKLOADS, MTAWorkload, make_conv_inputs, make_head_linear_inputs, make_mta_inputs)

# Small cases shared with the tests (tests/cases.py imports these tables).
sys.path.insert(0, HERE)
from cases import CONV_CASES, HEAD_CASES, MTA_CASES, CONV_ATTN_CASES  # noqa: E402


def _patch_torch_tensor():
    real = torch.tensor

    def tensor(*a, **kw):
        if kw.get("device") == "cuda":
            kw["device"] = "cpu"
        return real(*a, **kw)

    torch.tensor = tensor


def f32(t):
    """Outputs are stored in the run dtype: float32 as is, 16-bit dtypes as their bit patterns
    (uint16) under a key that ends in the dtype name; tests/golden/cases.py:load_golden undoes it."""
    return t.detach().contiguous()


def store(out, key, t):
    t = t.detach().contiguous()
    if t.dtype == torch.float32:
        out[key] = t.numpy()
    else:
        name = {torch.bfloat16: "bf16", torch.float16: "f16"}[t.dtype]
        out[f"{key}@{name}"] = t.view(torch.int16).numpy().view(np.uint16)


KERNEL_GOLDEN_MAX_S = 65   # reference Triton kernels (CPU interpreter) are stored for small planes only


def run_mta(ref_mod, wl: MTAWorkload):
    inp = make_mta_inputs(wl)
    cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=wl.cq, key_kernel_size=wl.ck,
                                after_sm_query_kernel_size=wl.cq2, after_sm_key_kernel_size=wl.ck2,
                                pre_sm_linear_head=True, post_sm_linear_head=True, pad_key="both",
                                init_method="identity", dim=wl.H * wl.D)
    m = ref_mod.MTAAttention(wl.H, cfg, dropout=0.0).eval().to(wl.dtype)
    with torch.no_grad():
        m.mta_kernel.copy_(inp["w1"].unsqueeze(1))
        m.wpsm.weight.copy_(inp["W1"])
        m.mta_kernel_after_sm.copy_(inp["w2"].unsqueeze(1))
        m.wposm.weight.copy_(inp["W2"])
        out = m(inp["q"], inp["k"], inp["v"], None, None)   # (B,S,H,D) view
    return out.transpose(1, 2).contiguous()                  # stored as (B,H,S,D)


def main(ref_path: str):
    sys.path.insert(0, ref_path)
    _patch_torch_tensor()
    torch.manual_seed(0)
    import mta_attention_pytorch as ref_mta
    import conv_attention_pytorch as ref_ca
    import convolution_2d_trit as ref_conv
    import triton_linear_head as ref_lin

    out = {}
    for name, wl in MTA_CASES.items():
        y = run_mta(ref_mta, wl)
        store(out, f"mta/{name}", y)
        print("mta", name, tuple(y.shape))

    for name, (N, C, S, D, R, Sk, dtype, seed, causal) in CONV_CASES.items():
        inp = make_conv_inputs(N, C, S, D, R, Sk, dtype, seed)
        x = torch.tril(inp["x"]) if causal else inp["x"]
        with torch.no_grad():
            y = ref_conv.pytorch_conv(x, inp["w"].unsqueeze(1), causal=causal)
        store(out, f"conv/{name}", y)
        if S <= KERNEL_GOLDEN_MAX_S:  # the reference's own kernel under Triton's CPU interpreter: upper triangle stays 0
            # the reference's own kernel under Triton's CPU interpreter, fp32 in/out, raw (untrilled) input:
            # pins "input above the diagonal is ignored" and "output above the diagonal is 0"
            yt = ref_conv.Conv2dTritonFunction.apply(inp["x"].float().contiguous(), inp["w"].float().contiguous(), causal)
            store(out, f"conv_kernel/{name}", yt)
        print("conv", name, y.shape)

    for name, (N, C, S, dtype, seed, causal, fill) in HEAD_CASES.items():
        inp = make_head_linear_inputs(N, C, S, dtype, seed)
        with torch.no_grad():
            y = F.linear(inp["x"].transpose(1, -1), inp["W"]).transpose(1, -1)   # mta_attention_pytorch.py:68
            if causal:
                upper = torch.triu(torch.ones(S, S, dtype=torch.bool), diagonal=1)
                y = y.masked_fill(upper, fill)
        store(out, f"head/{name}", y)
        if S <= KERNEL_GOLDEN_MAX_S:
            yt = ref_lin.TritonLinearHeadFunction.apply(inp["x"].float().contiguous(), inp["W"].float().contiguous(),
                                                        causal, fill)
            store(out, f"head_kernel/{name}", yt)
        print("head", name, y.shape)

    for name, (wl, causal) in CONV_ATTN_CASES.items():
        inp = make_mta_inputs(wl)
        m = ref_ca.ConvAttention(wl.H, wl.cq, wl.ck).to(wl.dtype)
        with torch.no_grad():
            m.conv_weight.copy_(inp["w1"])
            y = m(inp["q"], inp["k"], inp["v"], causal=causal)
        store(out, f"conv_attn/{name}", y)
        print("conv_attn", name, y.shape)

    np.savez_compressed(os.path.join(HERE, "golden_mta.npz"), **{k: v for k, v in out.items()})
    print("wrote", os.path.join(HERE, "golden_mta.npz"), sum(v.nbytes for v in out.values()) / 1e6, "MB raw")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} /path/to/reference")
    main(sys.argv[1])
