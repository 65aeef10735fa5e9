"""The explicit-mask forward (use_mask=True) on the GPU against the masked oracle and the golden outputs of the
reference's MTAAttention run with the same masks."""
import os

import numpy as np
import pytest
import torch

from cases import MASK_CASES, MASK_GOLDEN, MTA_CASES, load_golden, make_mask
from multitokenatention_triton_b200 import _lib
from multitokenatention_triton_b200.synthetic import make_mta_inputs
from oracle import mta_oracle as orc
from test_masked_cpu import module_for
from util import assert_parity, npf

pytestmark = pytest.mark.gpu
DEV = "cuda"
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def golden_masked():
    return load_golden(os.path.join(HERE, "golden", MASK_GOLDEN))


def build(wl, inp, use_mask):
    m = module_for(wl, use_mask).to(DEV).to(wl.dtype).eval()
    with torch.no_grad():
        m.mta_conv_triton.weight.copy_(inp["w1"])
        m.wpsm_triton.weight.copy_(inp["W1"])
        m.mta_conv_after_sm_triton.weight.copy_(inp["w2"])
        m.wposm_triton.weight.copy_(inp["W2"])
    return m


@pytest.mark.parametrize("name", list(MASK_CASES))
def test_masked_forward(name, golden_masked):
    mta_case, kind = MASK_CASES[name]
    wl = MTA_CASES[mta_case]
    inp = make_mta_inputs(wl)
    B = 1 if kind == "padding" else wl.B
    m = build(wl, inp, True)
    mask = make_mask(kind, wl.S, wl.dtype)
    q, k, v = (inp[x][:B].to(DEV) for x in ("q", "k", "v"))
    with torch.no_grad():
        out = m(q, k, v, mask.to(DEV) if mask is not None else None, None)
    _lib.device_status()
    assert out.shape == (B, wl.S, wl.H, wl.D)
    got = npf(out.transpose(1, 2))
    full = m._update_mask(mask, B, inp["q"][:B], wl.S)
    ref = orc.mta_fwd_masked(*(npf(inp[x][:B]) for x in ("q", "k", "v")), *(npf(inp[x]) for x in ("w1", "W1", "w2", "W2")),
                             npf(full), True)
    assert_parity(got, ref, wl.dtype, f"{name} vs oracle")
    assert_parity(got, golden_masked[f"masked/{name}"], wl.dtype, f"{name} vs golden")


@pytest.mark.parametrize("name", ["c1", "s130_6x11_bf16"])
def test_no_mask_equals_the_fused_causal_forward(name):
    wl = MTA_CASES[name]
    inp = make_mta_inputs(wl)
    q, k, v = (inp[x].to(DEV) for x in ("q", "k", "v"))
    with torch.no_grad():
        masked = build(wl, inp, True)(q, k, v, None, None)
        fused = build(wl, inp, False)(q, k, v, None, None)
    _lib.device_status()
    assert_parity(npf(masked), npf(fused), wl.dtype, name)
