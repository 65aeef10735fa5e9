"""GPU parity of pad_key = "left" / "right": the module (one fused call, stage by stage, and the explicit-mask path)
against golden outputs and gradients of the reference's PyTorch module, and the conv entry point with the
zero-extended kernel against the oracle's direct form."""
import os

import numpy as np
import pytest
import torch

from cases import PADKEY_CASES, PADKEY_GOLDEN, PADKEY_WORKLOADS, load_golden, make_mask
from multitokenatention_triton_b200 import Conv2dTriton, _lib
from multitokenatention_triton_b200.synthetic import make_conv_inputs, make_mta_inputs, make_upstream_grad
from oracle import mta_oracle as orc
from test_padkey_cpu import module_for
from util import ROUND, assert_parity, max_abs, npf

pytestmark = pytest.mark.gpu
DEV = "cuda"
HERE = os.path.dirname(os.path.abspath(__file__))
ULP = {torch.float32: 2.0 ** -17, torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}


@pytest.fixture(scope="module")
def golden_padkey():
    return load_golden(os.path.join(HERE, "golden", PADKEY_GOLDEN))


def load_weights(m, inp):
    with torch.no_grad():
        m.mta_conv_triton.weight.copy_(inp["w1"])
        m.wpsm_triton.weight.copy_(inp["W1"])
        m.mta_conv_after_sm_triton.weight.copy_(inp["w2"])
        m.wposm_triton.weight.copy_(inp["W2"])
    return m


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("name", list(PADKEY_CASES))
def test_padkey_forward_against_the_reference(name, fused, golden_padkey):
    wl_name, pad_key, kind = PADKEY_CASES[name]
    wl = PADKEY_WORKLOADS[wl_name]
    inp = make_mta_inputs(wl)
    m = load_weights(module_for(wl, pad_key, use_mask=kind != "none", fused=fused).to(DEV).to(wl.dtype).eval(), inp)
    mask = make_mask(kind, wl.S, wl.dtype)
    with torch.no_grad():
        y = m(inp["q"].to(DEV), inp["k"].to(DEV), inp["v"].to(DEV), None if mask is None else mask.to(DEV), None)
    _lib.device_status()
    assert y.shape == (wl.B, wl.S, wl.H, wl.D)
    assert_parity(npf(y.transpose(1, 2)), golden_padkey[f"padkey/{name}"], wl.dtype, f"{name} fused={fused}")


@pytest.mark.parametrize("name", [n for n, (w, _, kind) in PADKEY_CASES.items()
                                  if kind == "none" and PADKEY_WORKLOADS[w].dtype == torch.float32])
def test_padkey_gradients_against_the_reference(name, golden_padkey):
    wl_name, pad_key, _ = PADKEY_CASES[name]
    wl = PADKEY_WORKLOADS[wl_name]
    inp = make_mta_inputs(wl)
    m = load_weights(module_for(wl, pad_key).to(DEV).to(wl.dtype).eval(), inp)
    q, k, v = (inp[x].to(DEV).requires_grad_() for x in ("q", "k", "v"))
    g = make_upstream_grad((wl.B, wl.S, wl.H, wl.D), wl.dtype, wl.seed + 2000).to(DEV)
    m(q, k, v, None, None).backward(g)
    _lib.device_status()
    got = {"dq": q.grad, "dk": k.grad, "dv": v.grad, "dw1": m.mta_conv_triton.weight.grad, "dW1": m.wpsm_triton.weight.grad,
           "dw2": m.mta_conv_after_sm_triton.weight.grad, "dW2": m.wposm_triton.weight.grad}
    assert got["dw1"].shape == (wl.H, wl.cq, wl.ck) and got["dw2"].shape == (wl.H, wl.cq2, wl.ck2)
    for key, t in got.items():
        ref = golden_padkey[f"padkey_{key}/{name}"]
        err = float(np.max(np.abs(npf(t) - ref)))
        scale = max(1.0, float(np.max(np.abs(ref))))
        assert err <= 1e-3 * scale, f"{name} {key}: max abs {err:.3e} against scale {scale:.3e}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pad_key", ["left", "right"])
@pytest.mark.parametrize("S,R,Sk", [(72, 6, 11), (130, 3, 4), (264, 2, 9), (40, 1, 1)])
def test_padkey_conv_against_the_oracle(S, R, Sk, pad_key, dtype):
    inp = make_conv_inputs(2, 4, S, 16, R, Sk, dtype, seed=S + Sk)
    conv = Conv2dTriton(4, (R, Sk), causal=True, pad_key=pad_key).to(DEV).to(dtype)
    with torch.no_grad():
        conv.weight.copy_(inp["w"])
        y = conv(inp["x"].to(DEV))
    _lib.device_status()
    ref = orc.conv2d(npf(inp["x"]), npf(inp["w"]), True, ROUND[dtype], pad_key=pad_key)
    tol = 2.0 * ULP[dtype] * max(1.0, float(np.max(np.abs(ref))))
    assert max_abs(npf(y), ref) <= tol
