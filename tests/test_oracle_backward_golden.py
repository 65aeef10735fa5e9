"""The CPU oracle's gradients of the two stand-alone ops against golden gradients from the reference.

golden_backward.npz holds, per case, (a) autograd through the reference's PyTorch restatement of the op (float32) and,
for the small float32 cases, (b) the gradients produced by the reference's own backward kernels under Triton's CPU
interpreter.  Both must agree with the oracle to float32 accumulation noise.
"""
import numpy as np
import pytest
import torch

from cases import CONV_BWD_CASES, CONV_CASES, HEAD_BWD_CASES, HEAD_CASES
from multitokenatention_triton_b200.synthetic import make_conv_inputs, make_head_linear_inputs, make_upstream_grad
from oracle import mta_oracle as orc
from util import npf


def close(out, ref, what):
    tol = 2e-5 * max(1.0, float(np.max(np.abs(ref))))
    err = float(np.max(np.abs(np.asarray(out, dtype=np.float64) - ref)))
    assert err <= tol, f"{what}: max abs {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("name", CONV_BWD_CASES)
def test_conv2d_backward(name, golden_bwd):
    N, C, S, D, R, Sk, dtype, seed, causal = CONV_CASES[name]
    inp = make_conv_inputs(N, C, S, D, R, Sk, dtype, seed)
    g = npf(make_upstream_grad((N, C, S, S), dtype, seed + 1000))
    dx = orc.conv2d_bwd_input(g, npf(inp["w"]), causal)
    dw = orc.conv2d_bwd_weight(npf(inp["x"]), g, (R, Sk), causal)
    close(dx, golden_bwd[f"conv_dx/{name}"], f"{name} dx")
    close(dw, golden_bwd[f"conv_dw/{name}"], f"{name} dw")
    if f"conv_kernel_dx/{name}" in golden_bwd:          # the reference's own backward kernels
        close(dx, golden_bwd[f"conv_kernel_dx/{name}"], f"{name} dx vs reference kernel")
        close(dw, golden_bwd[f"conv_kernel_dw/{name}"], f"{name} dw vs reference kernel")
    if causal:
        iu = np.triu_indices(S, 1)
        assert np.all(dx[..., iu[0], iu[1]] == 0.0)
        xn = npf(inp["x"]).copy()                        # what sits above the diagonal of x or dy carries no gradient
        gn = g.copy()
        xn[..., iu[0], iu[1]] = 1e9
        gn[..., iu[0], iu[1]] = -1e9
        assert np.array_equal(orc.conv2d_bwd_weight(xn, gn, (R, Sk), causal), dw)
        assert np.array_equal(orc.conv2d_bwd_input(gn, npf(inp["w"]), causal), dx)


@pytest.mark.parametrize("name", HEAD_BWD_CASES)
def test_head_linear_backward(name, golden_bwd):
    N, C, S, dtype, seed, causal, fill = HEAD_CASES[name]
    inp = make_head_linear_inputs(N, C, S, dtype, seed)
    g = npf(make_upstream_grad((N, C, S, S), dtype, seed + 1000))
    dx = orc.head_linear_bwd_input(g, npf(inp["W"]), causal)
    dW = orc.head_linear_bwd_weight(npf(inp["x"]), g, causal)
    close(dx, golden_bwd[f"head_dx/{name}"], f"{name} dx")
    close(dW, golden_bwd[f"head_dW/{name}"], f"{name} dW")
    if f"head_kernel_dx/{name}" in golden_bwd:
        close(dx, golden_bwd[f"head_kernel_dx/{name}"], f"{name} dx vs reference kernel")
        close(dW, golden_bwd[f"head_kernel_dW/{name}"], f"{name} dW vs reference kernel")
    if causal:
        iu = np.triu_indices(S, 1)
        assert np.all(dx[..., iu[0], iu[1]] == 0.0)


def test_gradients_are_the_adjoint_of_the_forward():
    """<conv(x; w), g> is linear in x and in w: its exact derivatives are what the backward functions return."""
    rng = np.random.default_rng(7)
    x = rng.standard_normal((2, 3, 21, 21)).astype(np.float32)
    w = rng.standard_normal((3, 4, 5)).astype(np.float32)
    g = rng.standard_normal((2, 3, 21, 21)).astype(np.float32)
    for causal in (True, False):
        lhs = float(np.sum(orc.conv2d(x, w, causal).astype(np.float64) * g))
        assert abs(lhs - float(np.sum(orc.conv2d_bwd_input(g, w, causal).astype(np.float64) * x))) <= 1e-3 * max(1.0, abs(lhs))
        assert abs(lhs - float(np.sum(orc.conv2d_bwd_weight(x, g, (4, 5), causal) * w))) <= 1e-3 * max(1.0, abs(lhs))
    W = rng.standard_normal((3, 3)).astype(np.float32)
    lhs = float(np.sum(orc.head_linear(x, W, True, 0.0).astype(np.float64) * g))
    assert abs(lhs - float(np.sum(orc.head_linear_bwd_input(g, W, True).astype(np.float64) * x))) <= 1e-3 * max(1.0, abs(lhs))
    assert abs(lhs - float(np.sum(orc.head_linear_bwd_weight(x, g, True) * W))) <= 1e-3 * max(1.0, abs(lhs))
