"""The CPU oracle against the golden vectors made by the reference's own PyTorch code.

These pins are what lets the GPU parity tests trust the oracle.  float32 cases must agree to
accumulation noise.  16-bit cases are checked twice: the oracle with the reference's rounding points
emulated must land within a few ulps of the 16-bit dtype, and the unrounded oracle within the
parity contract's 2e-2.
"""
import numpy as np
import pytest
import torch

from cases import CONV_ATTN_CASES, CONV_CASES, HEAD_CASES, MTA_CASES
from multitokenatention_triton_b200.synthetic import make_conv_inputs, make_head_linear_inputs, make_mta_inputs
from oracle import mta_oracle as orc
from util import ROUND, max_abs, npf, rel_fro, rel_max

ULP = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}


def check(out, ref, dtype, exact_rounding: bool, scale_ulps: float = 4.0):
    if dtype == torch.float32:
        tol = 2e-5 * max(1.0, float(np.max(np.abs(ref[np.isfinite(ref)]))))
        assert max_abs(out, ref) <= tol, (max_abs(out, ref), tol)
        rel_fro(out, ref)
    elif exact_rounding:
        assert rel_fro(out, ref) <= scale_ulps * ULP[dtype], rel_fro(out, ref)
        assert rel_max(out, ref) <= 4 * scale_ulps * ULP[dtype], rel_max(out, ref)
    else:
        assert rel_fro(out, ref) <= 2e-2 and rel_max(out, ref) <= 2e-2, (rel_fro(out, ref), rel_max(out, ref))


@pytest.mark.parametrize("name", list(CONV_CASES))
def test_conv2d(name, golden):
    N, C, S, D, R, Sk, dtype, seed, causal = CONV_CASES[name]
    inp = make_conv_inputs(N, C, S, D, R, Sk, dtype, seed)
    ref = golden[f"conv/{name}"]
    out = orc.conv2d(npf(inp["x"]), npf(inp["w"]), causal, ROUND[dtype])
    check(out, ref, dtype, True, scale_ulps=1.0)
    if causal:
        assert np.all(out[..., np.triu_indices(S, 1)[0], np.triu_indices(S, 1)[1]] == 0.0)
    if f"conv_kernel/{name}" in golden:   # the reference's Triton kernel, fp32 arithmetic on the same values
        k = golden[f"conv_kernel/{name}"]
        o32 = orc.conv2d(npf(inp["x"]), npf(inp["w"]), causal, orc.ROUND_NONE)
        assert max_abs(o32, k) <= 2e-5 * max(1.0, float(np.abs(k).max()))
        if causal:
            iu = np.triu_indices(S, 1)
            assert np.all(k[..., iu[0], iu[1]] == 0.0)


@pytest.mark.parametrize("name", list(HEAD_CASES))
def test_head_linear(name, golden):
    N, C, S, dtype, seed, causal, fill = HEAD_CASES[name]
    inp = make_head_linear_inputs(N, C, S, dtype, seed)
    ref = golden[f"head/{name}"]
    out = orc.head_linear(npf(inp["x"]), npf(inp["W"]), causal, fill, ROUND[dtype])
    check(out, ref, dtype, True, scale_ulps=1.0)
    if f"head_kernel/{name}" in golden:
        k = golden[f"head_kernel/{name}"]
        o32 = orc.head_linear(npf(inp["x"]), npf(inp["W"]), causal, fill, orc.ROUND_NONE)
        # the reference kernel's dot runs in TF32 on fp32 inputs; the interpreter evaluates it in fp32
        assert rel_fro(o32, k) <= 1e-3
        if causal:
            iu = np.triu_indices(S, 1)
            up = k[..., iu[0], iu[1]]
            assert np.all(up == fill) if np.isfinite(fill) else np.all(np.isneginf(up))


@pytest.mark.parametrize("name", list(MTA_CASES))
def test_mta_forward(name, golden):
    wl = MTA_CASES[name]
    inp = {k: npf(v) for k, v in make_mta_inputs(wl).items()}
    ref = golden[f"mta/{name}"]
    out = orc.mta_fwd(inp["q"], inp["k"], inp["v"], inp["w1"], inp["W1"], inp["w2"], inp["W2"], True, ROUND[wl.dtype])
    check(out, ref, wl.dtype, True)
    if wl.dtype != torch.float32:
        exact = orc.mta_fwd(inp["q"], inp["k"], inp["v"], inp["w1"], inp["W1"], inp["w2"], inp["W2"], True,
                            orc.ROUND_NONE)
        check(exact, ref, wl.dtype, False)


def test_mta_forward_row_ranges_agree():
    wl = MTA_CASES["ragged_f32"]
    inp = {k: npf(v) for k, v in make_mta_inputs(wl).items()}
    args = [inp[k] for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    full = orc.mta_fwd(*args)
    for r0, r1 in ((0, 1), (0, 7), (3, 20), (17, 65), (64, 65)):
        part = orc.mta_fwd_rows(*args, 0, r0, r1)
        assert np.array_equal(part, full[0][:, r0:r1])


@pytest.mark.parametrize("name", list(CONV_ATTN_CASES))
def test_conv_attention(name, golden):
    wl, causal = CONV_ATTN_CASES[name]
    inp = {k: npf(v) for k, v in make_mta_inputs(wl).items()}
    ref = golden[f"conv_attn/{name}"]
    out = orc.conv_attn_fwd(inp["q"], inp["k"], inp["v"], inp["w1"], causal, None, ROUND[wl.dtype])
    check(out, ref, wl.dtype, True)
