"""Generate golden outputs and gradients for pad_key = "left" / "right" from the reference's PyTorch module.

    python tests/golden/make_golden_padkey.py /path/to/reference

For every case of PADKEY_CASES (tests/golden/cases.py) the reference's MTAAttention (mta_attention_pytorch.py; the only
implementation of the reference that places the key window of the convs to the left or to the right, :91-98) is run on
the seeded inputs of the named workload, with the mask the case names, and the output is stored in golden_padkey.npz as
(B,H,S,D).  For the float32 cases without a mask the module is also differentiated against the seeded upstream
gradient and dq, dk, dv and the four weight gradients are stored.  Same two shims as make_golden.py.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))
sys.path.insert(0, HERE)

from multitokenatention_triton_b200.synthetic import make_mta_inputs, make_upstream_grad  # noqa: E402
from cases import PADKEY_CASES, PADKEY_GOLDEN, PADKEY_WORKLOADS, make_mask  # noqa: E402
from make_golden import _patch_torch_tensor, store  # noqa: E402


def build_module(ref_mta, wl, pad_key, inp, dtype):
    cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=wl.cq, key_kernel_size=wl.ck,
                                after_sm_query_kernel_size=wl.cq2, after_sm_key_kernel_size=wl.ck2,
                                pre_sm_linear_head=True, post_sm_linear_head=True, pad_key=pad_key,
                                init_method="const", dim=wl.H * wl.D)
    m = ref_mta.MTAAttention(wl.H, cfg, dropout=0.0).eval().to(dtype)
    with torch.no_grad():
        m.mta_kernel.copy_(inp["w1"].to(dtype).unsqueeze(1))
        m.wpsm.weight.copy_(inp["W1"].to(dtype))
        m.mta_kernel_after_sm.copy_(inp["w2"].to(dtype).unsqueeze(1))
        m.wposm.weight.copy_(inp["W2"].to(dtype))
    return m


def main(ref_path: str):
    sys.path.insert(0, ref_path)
    _patch_torch_tensor()
    import mta_attention_pytorch as ref_mta
    out = {}
    for name, (wl_name, pad_key, kind) in PADKEY_CASES.items():
        wl = PADKEY_WORKLOADS[wl_name]
        inp = make_mta_inputs(wl)
        m = build_module(ref_mta, wl, pad_key, inp, wl.dtype)
        mask = make_mask(kind, wl.S, wl.dtype)
        with torch.no_grad():
            y = m(inp["q"], inp["k"], inp["v"], mask, None)
        store(out, f"padkey/{name}", y.transpose(1, 2).contiguous())
        print("padkey forward", name, tuple(y.shape))
        if wl.dtype == torch.float32 and kind == "none":
            m = build_module(ref_mta, wl, pad_key, inp, torch.float32)
            q, k, v = (inp[x].float().clone().requires_grad_() for x in ("q", "k", "v"))
            g = make_upstream_grad((wl.B, wl.S, wl.H, wl.D), wl.dtype, wl.seed + 2000).float()
            m(q, k, v, None, None).backward(g)
            for key, t in (("dq", q.grad), ("dk", k.grad), ("dv", v.grad), ("dw1", m.mta_kernel.grad.squeeze(1)),
                           ("dW1", m.wpsm.weight.grad), ("dw2", m.mta_kernel_after_sm.grad.squeeze(1)),
                           ("dW2", m.wposm.weight.grad)):
                out[f"padkey_{key}/{name}"] = t.detach().numpy().copy()
            print("padkey backward", name)
    path = os.path.join(HERE, PADKEY_GOLDEN)
    np.savez_compressed(path, **out)
    print("wrote", path, len(out), "arrays", os.path.getsize(path) / 1e3, "KB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} /path/to/reference")
    main(sys.argv[1])
