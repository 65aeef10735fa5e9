"""pad_key = "left" / "right" on the CPU: the oracle against golden outputs of the reference's PyTorch module (the only
implementation of the reference that places the key window there), the zero-extended kernel the CUDA path uses against
the direct form, and the module's host logic."""
import os
import types

import numpy as np
import pytest
import torch

from cases import PADKEY_CASES, PADKEY_GOLDEN, PADKEY_WORKLOADS, load_golden, make_mask
from multitokenatention_triton_b200 import Conv2dTriton, MTAAttentionTriton
from multitokenatention_triton_b200.synthetic import make_mta_inputs
from oracle import mta_oracle as orc
from util import ROUND, assert_parity, npf

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def golden_padkey():
    return load_golden(os.path.join(HERE, "golden", PADKEY_GOLDEN))


def module_for(wl, pad_key, **kw):
    cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=wl.cq, key_kernel_size=wl.ck,
                                after_sm_query_kernel_size=wl.cq2, after_sm_key_kernel_size=wl.ck2,
                                pre_sm_linear_head=True, post_sm_linear_head=True, pad_key=pad_key, init_method="const",
                                dim=wl.H * wl.D)
    return MTAAttentionTriton(wl.H, cfg, dropout=0.0, causal=True, **kw)


@pytest.mark.parametrize("name", list(PADKEY_CASES))
def test_padkey_oracle_matches_the_reference(name, golden_padkey):
    wl_name, pad_key, kind = PADKEY_CASES[name]
    wl = PADKEY_WORKLOADS[wl_name]
    inp = make_mta_inputs(wl)
    args = [npf(inp[k]) for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    if kind == "none":
        out = orc.mta_fwd(*args, True, ROUND[wl.dtype], pad_key=pad_key)
    else:
        full = module_for(wl, pad_key, use_mask=True)._update_mask(make_mask(kind, wl.S, wl.dtype), wl.B, inp["q"], wl.S)
        out = orc.mta_fwd_masked(*args, npf(full), True, pad_key=pad_key)
    assert_parity(out, golden_padkey[f"padkey/{name}"], wl.dtype, name)


@pytest.mark.parametrize("S", [1, 2, 3, 4, 11])
@pytest.mark.parametrize("pad_key", ["left", "right", "both"])
@pytest.mark.parametrize("causal", [True, False])
def test_zero_extended_kernel_is_the_same_conv(S, pad_key, causal):
    rng = np.random.default_rng(S)
    x = rng.standard_normal((2, 3, 23, 23)).astype(np.float32)
    w = rng.standard_normal((3, 4, S)).astype(np.float32)
    direct = orc.conv2d(x, w, causal, pad_key=pad_key)
    assert np.array_equal(direct, orc.conv2d(x, orc.embed_pad_key(w, pad_key), causal))
    # against torch's conv2d on the padded plane, as the reference writes it (mta_attention_pytorch.py:91-112)
    lead = orc.key_lead(pad_key, S)
    xt = torch.from_numpy(x).double()
    if causal:
        xt = torch.tril(xt)
    yt = torch.nn.functional.conv2d(torch.nn.functional.pad(xt, (lead, S - 1 - lead, 3, 0)),
                                    torch.from_numpy(w).double().unsqueeze(1), groups=3)
    if causal:
        yt = torch.tril(yt)
    np.testing.assert_allclose(direct, yt.numpy(), atol=1e-5)


@pytest.mark.parametrize("pad_key", ["left", "right", "both"])
def test_effective_weight_and_its_gradient(pad_key):
    conv = Conv2dTriton(3, (2, 4), causal=True, pad_key=pad_key)
    with torch.no_grad():
        conv.weight.copy_(torch.arange(24.0).reshape(3, 2, 4) + 1)
    eff = conv.effective_weight()
    assert np.array_equal(eff.detach().numpy(), orc.embed_pad_key(conv.weight.detach().numpy(), pad_key))
    g = torch.randn(eff.shape, generator=torch.Generator().manual_seed(0))
    (eff * g).sum().backward()
    lo = {"left": 0, "right": 3, "both": 0}[pad_key]
    assert torch.equal(conv.weight.grad, g[..., lo:lo + 4])


def test_unknown_pad_key_is_refused():
    with pytest.raises(ValueError):
        Conv2dTriton(3, (2, 3), pad_key="centre")
    wl = PADKEY_WORKLOADS["even_f32"]
    with pytest.raises(ValueError):
        module_for(wl, "middle")
