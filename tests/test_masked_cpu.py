"""The explicit-mask forward on the CPU: the module's mask normalisation (host logic) and the numpy/C restatement of
the masked pipeline against golden outputs of the reference's MTAAttention run with the same masks."""
import os
import types

import numpy as np
import pytest
import torch

from cases import MASK_CASES, MASK_GOLDEN, MTA_CASES, load_golden, make_mask
from multitokenatention_triton_b200 import MTAAttentionTriton
from multitokenatention_triton_b200.synthetic import make_mta_inputs
from oracle import mta_oracle as orc
from util import assert_parity, npf

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def golden_masked():
    return load_golden(os.path.join(HERE, "golden", MASK_GOLDEN))


def module_for(wl, use_mask=True):
    cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=wl.cq, key_kernel_size=wl.ck,
                                after_sm_query_kernel_size=wl.cq2, after_sm_key_kernel_size=wl.ck2,
                                pre_sm_linear_head=True, post_sm_linear_head=True, pad_key="both", init_method="identity",
                                dim=wl.H * wl.D)
    return MTAAttentionTriton(wl.H, cfg, dropout=0.0, causal=True, use_mask=use_mask)


@pytest.mark.parametrize("name", list(MASK_CASES))
def test_masked_oracle_matches_the_reference(name, golden_masked):
    mta_case, kind = MASK_CASES[name]
    wl = MTA_CASES[mta_case]
    inp = make_mta_inputs(wl)
    B = 1 if kind == "padding" else wl.B
    m = module_for(wl)
    full = m._update_mask(make_mask(kind, wl.S, wl.dtype), B, inp["q"][:B], wl.S)
    assert full.shape == (B, wl.H, wl.S, wl.S) and full.dtype == wl.dtype
    assert set(np.unique(npf(full))) <= {0.0, -np.inf}
    assert torch.all(torch.isneginf(full[..., torch.triu_indices(wl.S, wl.S, 1)[0], torch.triu_indices(wl.S, wl.S, 1)[1]]))
    out = orc.mta_fwd_masked(*(npf(inp[k][:B]) for k in ("q", "k", "v")), *(npf(inp[k]) for k in ("w1", "W1", "w2", "W2")),
                             npf(full), True)
    assert_parity(out, golden_masked[f"masked/{name}"], wl.dtype, name)


def test_no_mask_is_the_causal_forward():
    """use_mask=True with mask=None builds the causal mask: same result as the oracle's causal forward."""
    wl = MTA_CASES["ragged_f32"]
    inp = make_mta_inputs(wl)
    m = module_for(wl)
    full = m._update_mask(None, wl.B, inp["q"], wl.S)
    args = [npf(inp[k]) for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    np.testing.assert_allclose(orc.mta_fwd_masked(*args, npf(full), True), orc.mta_fwd(*args, True), atol=2e-5)


def test_boolean_and_additive_masks_agree():
    wl = MTA_CASES["tiny_f32"]
    inp = make_mta_inputs(wl)
    m = module_for(wl)
    add = make_mask("documents", wl.S, wl.dtype)
    a = m._update_mask(add, wl.B, inp["q"], wl.S)
    b = m._update_mask(add == 0, wl.B, inp["q"], wl.S)
    assert torch.equal(a, b)
