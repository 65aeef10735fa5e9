"""Generate golden gradients for the two stand-alone ops from the reference project's own PyTorch code.

    python tests/golden/make_golden_backward.py /path/to/reference

For every case of CONV_BWD_CASES / HEAD_BWD_CASES (tests/golden/cases.py) the reference's PyTorch restatement of the
op (convolution_2d_trit.pytorch_conv; F.linear on the transposed view as in mta_attention_pytorch.py:68) is run in
float32 on the seeded inputs of multitokenatention_triton_b200.synthetic (16-bit cases: on the 16-bit-rounded values),
differentiated by autograd against the seeded upstream gradient, and the gradients are stored in golden_backward.npz.
Where Triton's CPU interpreter can run them, the gradients of the reference's own autograd functions
(Conv2dTritonFunction / TritonLinearHeadFunction, i.e. its backward kernels) are stored as well for the small float32
cases; they pin the masks of the backward kernels.  Full-module gradients (MTA_BWD_CASES): autograd through the reference's
MTAAttention (mta_attention_pytorch.py) in float32.
"""
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))
sys.path.insert(0, HERE)

from multitokenatention_triton_b200.synthetic import make_conv_inputs, make_head_linear_inputs, make_upstream_grad  # noqa: E402
from cases import BACKWARD_GOLDEN, CONV_BWD_CASES, CONV_CASES, HEAD_BWD_CASES, HEAD_CASES  # noqa: E402

KERNEL_GOLDEN_MAX_S = 65


def main(ref_path: str):
    sys.path.insert(0, ref_path)
    import convolution_2d_trit as ref_conv
    import triton_linear_head as ref_lin

    out = {}
    for name in CONV_BWD_CASES:
        N, C, S, D, R, Sk, dtype, seed, causal = CONV_CASES[name]
        inp = make_conv_inputs(N, C, S, D, R, Sk, dtype, seed)
        g = make_upstream_grad((N, C, S, S), dtype, seed + 1000).float()
        x = inp["x"].float().clone().requires_grad_()
        w = inp["w"].float().clone().requires_grad_()
        y = ref_conv.pytorch_conv(torch.tril(x) if causal else x, w.unsqueeze(1), causal=causal)
        y.backward(g)
        out[f"conv_dx/{name}"] = x.grad.numpy().copy()
        out[f"conv_dw/{name}"] = w.grad.numpy().copy()
        if S <= KERNEL_GOLDEN_MAX_S and dtype == torch.float32:
            try:
                xt = inp["x"].float().clone().contiguous().requires_grad_()
                wt = inp["w"].float().clone().contiguous().requires_grad_()
                yt = ref_conv.Conv2dTritonFunction.apply(xt, wt, causal)
                yt.backward(g.contiguous())
                out[f"conv_kernel_dx/{name}"] = xt.grad.float().numpy()
                out[f"conv_kernel_dw/{name}"] = wt.grad.float().numpy()
            except Exception as ex:  # the interpreter cannot run every construct of the backward kernels
                print("  reference Triton conv backward not stored for", name, "-", type(ex).__name__, str(ex)[:120])
        print("conv backward", name)

    for name in HEAD_BWD_CASES:
        N, C, S, dtype, seed, causal, fill = HEAD_CASES[name]
        inp = make_head_linear_inputs(N, C, S, dtype, seed)
        g = make_upstream_grad((N, C, S, S), dtype, seed + 1000).float()
        x = inp["x"].float().clone().requires_grad_()
        W = inp["W"].float().clone().requires_grad_()
        y = F.linear(x.transpose(1, -1), W).transpose(1, -1)
        if causal:
            y = y * torch.tril(torch.ones(S, S))          # entries above the diagonal are a constant fill: no gradient
        y.backward(g)
        out[f"head_dx/{name}"] = x.grad.numpy().copy()
        out[f"head_dW/{name}"] = W.grad.numpy().copy()
        if S <= KERNEL_GOLDEN_MAX_S and dtype == torch.float32:
            try:
                xt = inp["x"].float().clone().contiguous().requires_grad_()
                Wt = inp["W"].float().clone().contiguous().requires_grad_()
                yt = ref_lin.TritonLinearHeadFunction.apply(xt, Wt, causal, 0.0)
                yt.backward(g.contiguous())
                dx = xt.grad.float()
                if causal:                                 # the reference leaves these entries uninitialised
                    dx = torch.where(torch.tril(torch.ones(S, S, dtype=torch.bool)), dx, torch.zeros(()))
                out[f"head_kernel_dx/{name}"] = dx.numpy()
                out[f"head_kernel_dW/{name}"] = Wt.grad.float().numpy()
            except Exception as ex:
                print("  reference Triton head-mix backward not stored for", name, "-", type(ex).__name__, str(ex)[:120])
        print("head backward", name)

    import types
    import mta_attention_pytorch as ref_mta
    from make_golden import _patch_torch_tensor
    from multitokenatention_triton_b200.synthetic import make_mta_inputs
    from cases import MTA_BWD_CASES, MTA_CASES
    _patch_torch_tensor()
    for name in MTA_BWD_CASES:
        wl = MTA_CASES[name]
        inp = make_mta_inputs(wl)
        cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=wl.cq, key_kernel_size=wl.ck,
                                    after_sm_query_kernel_size=wl.cq2, after_sm_key_kernel_size=wl.ck2,
                                    pre_sm_linear_head=True, post_sm_linear_head=True, pad_key="both",
                                    init_method="identity", dim=wl.H * wl.D)
        m = ref_mta.MTAAttention(wl.H, cfg, dropout=0.0).eval().float()
        with torch.no_grad():
            m.mta_kernel.copy_(inp["w1"].float().unsqueeze(1))
            m.wpsm.weight.copy_(inp["W1"].float())
            m.mta_kernel_after_sm.copy_(inp["w2"].float().unsqueeze(1))
            m.wposm.weight.copy_(inp["W2"].float())
        q, k, v = (inp[x].float().clone().requires_grad_() for x in ("q", "k", "v"))
        g = make_upstream_grad((wl.B, wl.S, wl.H, wl.D), wl.dtype, wl.seed + 2000).float()
        m(q, k, v, None, None).backward(g)
        for key, t in (("dq", q.grad), ("dk", k.grad), ("dv", v.grad), ("dw1", m.mta_kernel.grad.squeeze(1)),
                       ("dW1", m.wpsm.weight.grad), ("dw2", m.mta_kernel_after_sm.grad.squeeze(1)), ("dW2", m.wposm.weight.grad)):
            out[f"mta_{key}/{name}"] = t.detach().numpy().copy()
        print("mta backward", name)

    path = os.path.join(HERE, BACKWARD_GOLDEN)
    np.savez_compressed(path, **out)
    print("wrote", path, sum(v.nbytes for v in out.values()) / 1e6, "MB raw,", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} /path/to/reference")
    main(sys.argv[1])
