"""GPU parity of the gradients of the two stand-alone ops (through the C ABI) against the CPU oracle, the golden
gradients from the reference, and size-independent properties at the score-plane size of configs 2/3.

Tolerances: an input gradient is one fp32 accumulation followed by one rounding to the dtype (~1 ulp of the dtype
relative to the largest magnitude in play).  A weight gradient is a float32 sum over every position of every plane
(partial sums per tile in float32, added in double): its error is bounded by float32 epsilon times the sum of the
absolute values of its terms, which the oracle evaluates on |x| and |dy|.
"""
import numpy as np
import pytest
import torch

from cases import CONV_BWD_CASES, CONV_CASES, HEAD_BWD_CASES, HEAD_CASES
from multitokenatention_triton_b200 import Conv2dTriton, TritonLinearHead, _lib, ops
from multitokenatention_triton_b200.synthetic import make_conv_inputs, make_head_linear_inputs, make_upstream_grad
from oracle import mta_oracle as orc
from util import ROUND, max_abs, npf

pytestmark = pytest.mark.gpu
DEV = "cuda"
ULP = {torch.float32: 2.0 ** -17, torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}


def input_grad_close(out, ref, dtype, what):
    tol = 2.0 * ULP[dtype] * max(1.0, float(np.max(np.abs(ref))))
    assert max_abs(out, ref) <= tol, f"{what}: max abs {max_abs(out, ref):.3e} > {tol:.3e}"


def weight_grad_close(out, ref, sum_abs, what):
    tol = 4e-6 * sum_abs + 1e-6
    err = np.abs(np.asarray(out, dtype=np.float64) - ref)
    assert np.all(err <= tol), f"{what}: max excess {float(np.max(err - tol)):.3e}"


@pytest.mark.parametrize("name", CONV_BWD_CASES)
def test_conv2d_backward_cases(name, golden_bwd):
    N, C, S, D, R, Sk, dtype, seed, causal = CONV_CASES[name]
    inp = make_conv_inputs(N, C, S, D, R, Sk, dtype, seed)
    g = make_upstream_grad((N, C, S, S), dtype, seed + 1000)
    dx = ops.conv2d_bwd_input(g.to(DEV), inp["w"].to(DEV), causal)
    dw = ops.conv2d_bwd_weight(inp["x"].to(DEV), g.to(DEV), (R, Sk), causal)
    _lib.device_status()
    ref_dx = orc.conv2d_bwd_input(npf(g), npf(inp["w"]), causal, ROUND[dtype])
    ref_dw = orc.conv2d_bwd_weight(npf(inp["x"]), npf(g), (R, Sk), causal)
    sum_abs = orc.conv2d_bwd_weight(np.abs(npf(inp["x"])), np.abs(npf(g)), (R, Sk), causal)
    input_grad_close(npf(dx), ref_dx, dtype, f"{name} dx")
    weight_grad_close(npf(dw), ref_dw, sum_abs, f"{name} dw")
    input_grad_close(npf(dx), golden_bwd[f"conv_dx/{name}"], dtype, f"{name} dx vs golden")
    weight_grad_close(npf(dw), golden_bwd[f"conv_dw/{name}"], sum_abs + 1e-4 * np.abs(ref_dw), f"{name} dw vs golden")
    assert dw.dtype == torch.float32 and dx.dtype == dtype
    if causal:
        iu = np.triu_indices(S, 1)
        assert np.all(npf(dx)[..., iu[0], iu[1]] == 0.0)


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("S,R,Sk,causal", [(7, 3, 3, True), (96, 2, 7, True), (129, 6, 11, True), (200, 11, 15, True),
                                           (70, 20, 21, True), (131, 4, 6, True), (66, 5, 9, False), (264, 3, 3, True),
                                           (512, 6, 11, True), (136, 1, 1, True), (320, 5, 9, False)])
def test_conv2d_backward_shapes(S, R, Sk, causal, dtype, variant):
    """variant 0: the tensor-core kernel where the shape allows it (16-bit, S % 8 == 0, odd key extent <= 17);
    variant 1: CUDA cores."""
    if variant == 1 and (dtype == torch.float32 or S % 8 or Sk % 2 == 0 or Sk > 17):
        pytest.skip("same kernel as variant 0 for this shape")
    _lib.set_variant("conv2d", variant)
    try:
        _conv2d_backward_shape(S, R, Sk, causal, dtype)
    finally:
        _lib.set_variant("conv2d", 0)


def _conv2d_backward_shape(S, R, Sk, causal, dtype):
    inp = make_conv_inputs(2, 3, S, 16, R, Sk, dtype, seed=500 + S)
    w32 = inp["w"].float() + 1e-3 * torch.randn(3, R, Sk, generator=torch.Generator().manual_seed(S))
    g = make_upstream_grad((2, 3, S, S), dtype, 1500 + S)
    xn, gn = inp["x"].clone(), g.clone()
    if causal:                                           # garbage above the diagonal of x and dy must be ignored
        iu = torch.triu_indices(S, S, 1)
        xn[..., iu[0], iu[1]] = float("nan")
        gn[..., iu[0], iu[1]] = float("nan")
    dx = ops.conv2d_bwd_input(gn.to(DEV), w32.to(DEV), causal)
    dw = ops.conv2d_bwd_weight(xn.to(DEV), gn.to(DEV), (R, Sk), causal)
    _lib.device_status()
    input_grad_close(npf(dx), orc.conv2d_bwd_input(npf(g), npf(w32), causal, ROUND[dtype]), dtype, "dx")
    ref_dw = orc.conv2d_bwd_weight(npf(inp["x"]), npf(g), (R, Sk), causal)
    weight_grad_close(npf(dw), ref_dw, orc.conv2d_bwd_weight(np.abs(npf(inp["x"])), np.abs(npf(g)), (R, Sk), causal), "dw")


@pytest.mark.parametrize("name", HEAD_BWD_CASES)
def test_head_linear_backward_cases(name, golden_bwd):
    N, C, S, dtype, seed, causal, fill = HEAD_CASES[name]
    inp = make_head_linear_inputs(N, C, S, dtype, seed)
    g = make_upstream_grad((N, C, S, S), dtype, seed + 1000)
    dx = ops.head_linear_bwd_input(g.to(DEV), inp["W"].to(DEV), causal)
    dW = ops.head_linear_bwd_weight(inp["x"].to(DEV), g.to(DEV), causal)
    _lib.device_status()
    input_grad_close(npf(dx), orc.head_linear_bwd_input(npf(g), npf(inp["W"]), causal, ROUND[dtype]), dtype, f"{name} dx")
    sum_abs = orc.head_linear_bwd_weight(np.abs(npf(inp["x"])), np.abs(npf(g)), causal)
    weight_grad_close(npf(dW), orc.head_linear_bwd_weight(npf(inp["x"]), npf(g), causal), sum_abs, f"{name} dW")
    input_grad_close(npf(dx), golden_bwd[f"head_dx/{name}"], dtype, f"{name} dx vs golden")
    weight_grad_close(npf(dW), golden_bwd[f"head_dW/{name}"], sum_abs + 1e-4 * np.abs(golden_bwd[f"head_dW/{name}"]), f"{name} dW vs golden")
    if causal:
        iu = np.triu_indices(S, 1)
        assert np.all(npf(dx)[..., iu[0], iu[1]] == 0.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("C", [1, 2, 7, 16, 24, 32, 48, 128])
def test_head_linear_backward_head_counts(C, dtype):
    S = 72
    inp = make_head_linear_inputs(2, C, S, dtype, seed=700 + C, mix_var=0.2)
    W32 = inp["W"].float() + 1e-3 * torch.randn(C, C, generator=torch.Generator().manual_seed(C))
    g = make_upstream_grad((2, C, S, S), dtype, 1700 + C)
    xn, gn = inp["x"].clone(), g.clone()                 # garbage above the diagonal of x and dy must be ignored
    iu = torch.triu_indices(S, S, 1)
    xn[..., iu[0], iu[1]] = float("nan")
    gn[..., iu[0], iu[1]] = float("nan")
    dx = ops.head_linear_bwd_input(gn.to(DEV), W32.to(DEV), True)
    dW = ops.head_linear_bwd_weight(xn.to(DEV), gn.to(DEV), True)
    _lib.set_variant("head_linear", 1)                   # CUDA-core kernels
    try:
        dW1 = ops.head_linear_bwd_weight(xn.to(DEV), gn.to(DEV), True)
    finally:
        _lib.set_variant("head_linear", 0)
    weight_grad_close(npf(dW1), orc.head_linear_bwd_weight(npf(inp["x"]), npf(g), True),
                      orc.head_linear_bwd_weight(np.abs(npf(inp["x"])), np.abs(npf(g)), True), f"C={C} dW (CUDA cores)")
    _lib.device_status()
    input_grad_close(npf(dx), orc.head_linear_bwd_input(npf(g), npf(W32), True, ROUND[dtype]), dtype, f"C={C} dx")
    weight_grad_close(npf(dW), orc.head_linear_bwd_weight(npf(inp["x"]), npf(g), True),
                      orc.head_linear_bwd_weight(np.abs(npf(inp["x"])), np.abs(npf(g)), True), f"C={C} dW")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_autograd_through_the_modules(dtype):
    """loss.backward() through Conv2dTriton and TritonLinearHead, as a training step of the reference would run it."""
    S, C = 96, 8
    inp = make_conv_inputs(2, C, S, 16, 3, 5, dtype, seed=88)
    hl = make_head_linear_inputs(2, C, S, dtype, seed=89, mix_var=0.1)
    conv = Conv2dTriton(C, (3, 5), causal=True).to(DEV)
    mix = TritonLinearHead(C, causal=True, output_value=0.0).to(DEV)
    with torch.no_grad():
        conv.weight.copy_(inp["w"].float())
        mix.weight.copy_(hl["W"].float())
    x = inp["x"].to(DEV).requires_grad_()
    g = make_upstream_grad((2, C, S, S), dtype, 90)
    y = mix(conv(x))
    y.backward(g.to(DEV))
    _lib.device_status()
    w, W = npf(conv.weight.detach()), npf(mix.weight.detach())
    mid = orc.conv2d(npf(inp["x"]), w, True, ROUND[dtype])
    g_mid = orc.head_linear_bwd_input(npf(g), W, True, ROUND[dtype])
    input_grad_close(npf(x.grad), orc.conv2d_bwd_input(g_mid, w, True, ROUND[dtype]), dtype, "dx through both modules")
    weight_grad_close(npf(mix.weight.grad), orc.head_linear_bwd_weight(mid, npf(g), True),
                      orc.head_linear_bwd_weight(np.abs(mid), np.abs(npf(g)), True) + 1e-2, "mix.weight.grad")
    weight_grad_close(npf(conv.weight.grad), orc.conv2d_bwd_weight(npf(inp["x"]), g_mid, (3, 5), True),
                      orc.conv2d_bwd_weight(np.abs(npf(inp["x"])), np.abs(g_mid), (3, 5), True) + 1e-2, "conv.weight.grad")
    assert conv.weight.grad.dtype == conv.weight.dtype and x.grad.dtype == dtype


def test_backward_at_score_plane_size():
    """B2 H16 S2048 bf16 (half of configs 2/3): the gradients are the adjoints of the forward, <conv(x), g> = <x, dx> =
    <w, dw>, they are reproducible bit for bit, and nothing above the diagonal is read or written."""
    N, C, S, R, Sk = 2, 16, 2048, 6, 11
    inp = make_conv_inputs(N, C, S, 128, R, Sk, torch.bfloat16, seed=1)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    g = make_upstream_grad((N, C, S, S), torch.bfloat16, 1001).to(DEV)
    y = ops.conv2d_fwd(x, w, True)
    dx = ops.conv2d_bwd_input(g, w, True)
    dw = ops.conv2d_bwd_weight(x, g, (R, Sk), True)
    _lib.device_status()
    assert torch.count_nonzero(torch.triu(dx, diagonal=1)) == 0
    gl, xl = torch.tril(g).double(), torch.tril(x).double()
    lhs = float((y.double() * gl).sum())
    scale = float((y.double().abs() * gl.abs()).sum())
    assert abs(lhs - float((dx.double() * xl).sum())) <= 4e-3 * scale        # y and dx carry one bf16 rounding each
    assert abs(lhs - float((dw.double() * w.double()).sum())) <= 4e-3 * scale
    assert torch.equal(ops.conv2d_bwd_weight(x, g, (R, Sk), True), dw) and torch.equal(ops.conv2d_bwd_input(g, w, True), dx)
    hl = make_head_linear_inputs(N, C, S, torch.bfloat16, seed=2)
    p, W = hl["x"].to(DEV), hl["W"].to(DEV)
    z = ops.head_linear_fwd(p, W, True, 0.0)
    dp = ops.head_linear_bwd_input(g, W, True)
    dW = ops.head_linear_bwd_weight(p, g, True)
    _lib.device_status()
    assert torch.count_nonzero(torch.triu(dp, diagonal=1)) == 0
    lhs = float((z.double() * gl).sum())
    scale = float((z.double().abs() * gl.abs()).sum())
    assert abs(lhs - float((dp.double() * torch.tril(p).double()).sum())) <= 4e-3 * scale
    assert abs(lhs - float((dW.double() * W.double()).sum())) <= 4e-3 * scale
    assert torch.equal(ops.head_linear_bwd_weight(p, g, True), dW)


@pytest.mark.parametrize("name", ["tiny_f32", "ragged_f32", "c1b"])
def test_module_gradients_against_the_reference(name, golden_bwd):
    """loss.backward() through MTAAttentionTriton (the stage-by-stage path a training step takes) against autograd
    through the reference's MTAAttention: gradients of q, k, v and of the four weights."""
    import types
    from cases import MTA_CASES
    from multitokenatention_triton_b200 import MTAAttentionTriton
    from multitokenatention_triton_b200.synthetic import make_mta_inputs
    wl = MTA_CASES[name]
    inp = make_mta_inputs(wl)
    cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=wl.cq, key_kernel_size=wl.ck,
                                after_sm_query_kernel_size=wl.cq2, after_sm_key_kernel_size=wl.ck2,
                                pre_sm_linear_head=True, post_sm_linear_head=True, pad_key="both", init_method="identity",
                                dim=wl.H * wl.D)
    m = MTAAttentionTriton(wl.H, cfg, dropout=0.0, causal=True).to(DEV).to(wl.dtype).eval()
    with torch.no_grad():
        m.mta_conv_triton.weight.copy_(inp["w1"])
        m.wpsm_triton.weight.copy_(inp["W1"])
        m.mta_conv_after_sm_triton.weight.copy_(inp["w2"])
        m.wposm_triton.weight.copy_(inp["W2"])
    q, k, v = (inp[x].to(DEV).requires_grad_() for x in ("q", "k", "v"))
    g = make_upstream_grad((wl.B, wl.S, wl.H, wl.D), wl.dtype, wl.seed + 2000).to(DEV)
    m(q, k, v, None, None).backward(g)
    _lib.device_status()
    got = {"dq": q.grad, "dk": k.grad, "dv": v.grad, "dw1": m.mta_conv_triton.weight.grad, "dW1": m.wpsm_triton.weight.grad,
           "dw2": m.mta_conv_after_sm_triton.weight.grad, "dW2": m.wposm_triton.weight.grad}
    for key, t in got.items():
        ref = golden_bwd[f"mta_{key}/{name}"]
        err = float(np.max(np.abs(npf(t) - ref)))
        scale = max(1.0, float(np.max(np.abs(ref))))
        assert err <= 1e-3 * scale, f"{name} {key}: max abs {err:.3e} against scale {scale:.3e}"


def test_dropout_in_training_mode():
    """dropout > 0 in training mode is applied to the attention weights before the product with V, as the reference does
    (mta_attention_triton.py:87): p = 0 in training mode equals eval, p > 0 is unbiased."""
    import types
    from cases import MTA_CASES
    from multitokenatention_triton_b200 import MTAAttentionTriton
    from multitokenatention_triton_b200.synthetic import make_mta_inputs
    wl = MTA_CASES["c1"]
    inp = make_mta_inputs(wl)
    cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=wl.cq, key_kernel_size=wl.ck,
                                after_sm_query_kernel_size=wl.cq2, after_sm_key_kernel_size=wl.ck2,
                                pre_sm_linear_head=True, post_sm_linear_head=True, pad_key="both", init_method="identity",
                                dim=wl.H * wl.D)
    q, k, v = (inp[x].to(DEV) for x in ("q", "k", "v"))
    outs = {}
    for p in (0.0, 0.5):
        m = MTAAttentionTriton(wl.H, cfg, dropout=p, causal=True).to(DEV)
        with torch.no_grad():
            m.mta_conv_triton.weight.copy_(inp["w1"])
            m.wpsm_triton.weight.copy_(inp["W1"])
            m.mta_conv_after_sm_triton.weight.copy_(inp["w2"])
            m.wposm_triton.weight.copy_(inp["W2"])
            ref = m.eval()(q, k, v, None, None)
            m.train()
            torch.manual_seed(0)
            outs[p] = torch.stack([m(q, k, v, None, None) for _ in range(64 if p else 1)]).mean(0)
        if p == 0.0:
            assert torch.allclose(outs[p], ref, atol=1e-5)
        else:
            assert not torch.allclose(outs[p], ref, atol=1e-3)
            assert float((outs[p] - ref).abs().mean()) < 0.25 * float(ref.abs().mean())
    _lib.device_status()
