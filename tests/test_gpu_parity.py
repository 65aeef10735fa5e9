"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle and the golden
vectors made by the reference's PyTorch code, on the same seeded inputs.

Tolerances are those of the parity contract (tests/util.py): float32 max abs error <= 1e-3; 16-bit
dtypes <= 2e-2 relative, norm-wise.  Stand-alone ops are held to a much tighter bound because a single
stage only differs from the oracle by summation order and one rounding.
"""
import dataclasses

import numpy as np
import pytest
import torch

from cases import CONV_ATTN_CASES, CONV_CASES, HEAD_CASES, MTA_CASES
from multitokenatention_triton_b200 import (Conv2dTriton, MTAAttentionTriton, TritonConvAttention, TritonLinearHead,
                                            _lib, ops)
from multitokenatention_triton_b200.synthetic import MTAWorkload, make_conv_inputs, make_head_linear_inputs, make_mta_inputs
from oracle import mta_oracle as orc
from util import ROUND, assert_parity, max_abs, npf, rel_fro, rel_max

pytestmark = pytest.mark.gpu
DEV = "cuda"
ULP = {torch.float32: 2.0 ** -17, torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}


def one_stage_close(out, ref, dtype, what):
    """A single stage: fp32 accumulation then one rounding to the dtype -> at most ~1 ulp of the dtype
    relative to the largest magnitude in play."""
    tol = 2.0 * ULP[dtype] * max(1.0, float(np.max(np.abs(ref[np.isfinite(ref)]), initial=0.0)))
    rel_fro(out, ref)   # non-finite pattern must match exactly
    assert max_abs(out, ref) <= tol, f"{what}: max abs {max_abs(out, ref):.3e} > {tol:.3e}"


# ---------------------------------------------------------------------------------------------
def conv_mma_able(dtype, S, Sk):
    return dtype != torch.float32 and Sk <= 17 and S % 8 == 0


@pytest.mark.parametrize("variant", [1, 2, 3])
@pytest.mark.parametrize("name", list(CONV_CASES))
def test_conv2d(name, variant, golden):
    """variant 1 = CUDA-core kernel, 2 = mma.sync Toeplitz kernel, 3 = tcgen05 Toeplitz kernel."""
    N, C, S, D, R, Sk, dtype, seed, causal = CONV_CASES[name]
    if variant >= 2 and not conv_mma_able(dtype, S, Sk):
        pytest.skip("outside the tensor-core kernel's domain")
    inp = make_conv_inputs(N, C, S, D, R, Sk, dtype, seed)          # upper triangle left as computed
    m = Conv2dTriton(C, (R, Sk), causal=causal).to(DEV).to(dtype)
    _lib.set_variant("conv2d", variant)
    try:
        with torch.no_grad():
            m.weight.copy_(inp["w"])
            y = m(inp["x"].to(DEV))
        _lib.device_status()
    finally:
        _lib.set_variant("conv2d", 0)
    assert y.shape == inp["x"].shape and y.dtype == dtype
    out = npf(y)
    ref = orc.conv2d(npf(inp["x"]), npf(inp["w"]), causal, ROUND[dtype])
    one_stage_close(out, ref, dtype, name)
    one_stage_close(out, golden[f"conv/{name}"], dtype, name + " vs golden")
    if causal:
        iu = np.triu_indices(S, 1)
        assert np.all(out[..., iu[0], iu[1]] == 0.0), "output above the diagonal must be exactly 0"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,R,Sk", [(7, 3, 3), (33, 1, 1), (96, 2, 7), (129, 6, 11), (200, 11, 15), (70, 20, 21)])
def test_conv2d_fp32_weights_and_odd_shapes(S, R, Sk, dtype):
    inp = make_conv_inputs(2, 3, S, 16, R, Sk, dtype, seed=1000 + S)
    w32 = torch.randn(3, R, Sk, generator=torch.Generator().manual_seed(S)) * (R * Sk) ** -0.5   # weight kept in fp32
    y = ops.conv2d_fwd(inp["x"].to(DEV), w32.to(DEV), True)
    ref = orc.conv2d(npf(inp["x"]), npf(w32), True, ROUND[dtype])
    one_stage_close(npf(y), ref, dtype, f"S={S} {R}x{Sk}")


@pytest.mark.parametrize("variant", [2, 3])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("S,R,Sk,causal", [(512, 6, 11, True), (264, 3, 3, True), (136, 1, 1, True), (320, 11, 15, True),
                                             (200, 2, 17, True), (128, 4, 4, True), (384, 6, 11, False), (8, 3, 3, True)])
def test_conv2d_tensor_core(S, R, Sk, causal, dtype, variant):
    """The Toeplitz tensor-core kernels on larger planes, with NaN planted above the diagonal (must never be read)."""
    if variant == 3 and R > 8:
        pytest.skip("the tcgen05 kernel's shared-memory rings take fewer row taps")
    inp = make_conv_inputs(2, 3, S, 32, R, Sk, dtype, seed=2000 + S + R)
    x = inp["x"].clone()
    if causal:
        iu = torch.triu_indices(S, S, 1)
        x[..., iu[0], iu[1]] = float("nan")
    _lib.set_variant("conv2d", variant)
    try:
        y = ops.conv2d_fwd(x.to(DEV), inp["w"].to(DEV), causal)      # weights in the activation dtype
        _lib.device_status()
    finally:
        _lib.set_variant("conv2d", 0)
    ref = orc.conv2d(npf(torch.tril(inp["x"]) if causal else inp["x"]), npf(inp["w"]), causal, ROUND[dtype])
    one_stage_close(npf(y), ref, dtype, f"S={S} {R}x{Sk}")


def test_conv2d_rectangular_noncausal():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(2, 3, 37, 150, generator=g)
    w = torch.randn(3, 4, 9, generator=g) / 6
    y = ops.conv2d_fwd(x.to(DEV), w.to(DEV), False)
    ref = orc.conv2d(npf(x), npf(w), False)
    one_stage_close(npf(y), ref, torch.float32, "rectangular")


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("variant", [1, 2, 3])
@pytest.mark.parametrize("name", list(HEAD_CASES))
def test_head_linear(name, variant, golden):
    N, C, S, dtype, seed, causal, fill = HEAD_CASES[name]
    mma_able = dtype != torch.float32 and C <= 32 and S % 8 == 0
    if variant == 2 and not mma_able:
        pytest.skip("tensor-core variant needs a 16-bit dtype, C <= 32 and S % 8 == 0")
    if variant == 3 and not (dtype != torch.float32 and C in (8, 16, 32, 64, 128) and S % 8 == 0):
        pytest.skip("the tcgen05 variant needs a 16-bit dtype, 8, 16, 32, 64 or 128 heads and S % 8 == 0")
    inp = make_head_linear_inputs(N, C, S, dtype, seed)
    m = TritonLinearHead(C, causal=causal, output_value=fill).to(DEV).to(dtype)
    _lib.set_variant("head_linear", variant)
    try:
        with torch.no_grad():
            m.weight.copy_(inp["W"])
            y = m(inp["x"].to(DEV))
    finally:
        _lib.set_variant("head_linear", 0)
    out = npf(y)
    ref = orc.head_linear(npf(inp["x"]), npf(inp["W"]), causal, fill, ROUND[dtype])
    one_stage_close(out, ref, dtype, name)
    one_stage_close(out, golden[f"head/{name}"], dtype, name + " vs golden")
    if causal:
        iu = np.triu_indices(S, 1)
        up = out[..., iu[0], iu[1]]
        assert np.all(up == fill) if np.isfinite(fill) else np.all(np.isneginf(up))


@pytest.mark.parametrize("C", [1, 2, 7, 12, 16, 24, 32, 48, 128])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_head_linear_head_counts(C, dtype):
    S = 72
    inp = make_head_linear_inputs(1, C, S, dtype, seed=300 + C, mix_var=0.2)
    W32 = inp["W"].float() + 1e-3 * torch.randn(C, C, generator=torch.Generator().manual_seed(C))   # not bf16-representable
    y = ops.head_linear_fwd(inp["x"].to(DEV), W32.to(DEV), True, float("-inf"))
    ref = orc.head_linear(npf(inp["x"]), npf(W32), True, float("-inf"), ROUND[dtype])
    one_stage_close(npf(y), ref, dtype, f"C={C}")


@pytest.mark.parametrize("variant", [2, 3])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("C,S,causal,fill", [(16, 520, True, 0.0), (16, 1304, True, float("-inf")), (8, 264, True, 0.0),
                                             (32, 1032, True, 0.0), (64, 200, True, float("-inf")), (128, 136, True, 0.0),
                                             (16, 264, False, 0.0), (32, 136, False, 0.0)])
def test_head_linear_16bit_weights(C, S, causal, fill, dtype, variant):
    """Weights in the activations' dtype, rows of several key tiles: the tcgen05 kernel (3) and the mma.sync kernel (2)
    against the oracle; NaN above the diagonal of the input must change nothing; the part above the diagonal is `fill`."""
    if variant == 2 and C > 32:
        pytest.skip("the mma.sync kernel takes up to 32 heads")
    g = torch.Generator().manual_seed(2900 + C + S)
    x = torch.randn(2, C, S, S, generator=g).to(dtype)
    W = (torch.eye(C) + 0.3 * torch.randn(C, C, generator=g)).to(dtype)
    _lib.set_variant("head_linear", variant)
    try:
        _lib.reset_launch_count()
        y = ops.head_linear_fwd(x.to(DEV), W.to(DEV), causal, fill)
        assert _lib.launch_count() == 1
        if causal:
            xn = x.clone()
            iu = torch.triu_indices(S, S, 1)
            xn[..., iu[0], iu[1]] = float("nan")
            yn = ops.head_linear_fwd(xn.to(DEV), W.to(DEV), causal, fill)
            assert torch.equal(y, yn)
    finally:
        _lib.set_variant("head_linear", 0)
    _lib.device_status()
    ref = orc.head_linear(npf(x), npf(W), causal, fill, ROUND[dtype])
    one_stage_close(npf(y), ref, dtype, f"C={C} S={S} causal={causal}")
    if causal:
        iu = np.triu_indices(S, 1)
        up = npf(y)[..., iu[0], iu[1]]
        assert np.all(up == fill) if np.isfinite(fill) else np.all(np.isneginf(up))


@pytest.mark.parametrize("P,Q,causal", [(200, 136, True), (100, 264, True), (37, 152, False), (300, 64, False)])
def test_head_linear_rectangular_on_tcgen05(P, Q, causal):
    """Planes with more rows than keys and the other way round, on the tcgen05 kernels: the plain head mix and, for the
    causal shapes, head mix + softmax (rows past the last key see every key)."""
    g = torch.Generator().manual_seed(31 * P + Q)
    x = (2 * torch.randn(2, 16, P, Q, generator=g)).to(torch.bfloat16)
    W = (torch.eye(16) + 0.3 * torch.randn(16, 16, generator=g)).to(torch.bfloat16)
    _lib.set_variant("head_linear", 3)
    _lib.set_variant("mix_softmax", 2)
    try:
        y = ops.head_linear_fwd(x.to(DEV), W.to(DEV), causal, 0.0)
        ys = ops.head_linear_softmax_fwd(x.to(DEV), W.to(DEV)) if causal else None
    finally:
        _lib.set_variant("head_linear", 0)
        _lib.set_variant("mix_softmax", 0)
    _lib.device_status()
    one_stage_close(npf(y), orc.head_linear(npf(x), npf(W), causal, 0.0, orc.ROUND_BF16), torch.bfloat16, f"{P}x{Q}")
    if causal:
        mixed = orc.head_linear(npf(x), npf(W), True, float("-inf"), orc.ROUND_BF16)
        ref = orc.softmax(mixed, True, orc.ROUND_BF16)
        tol = 2.0 * ULP[torch.bfloat16] * max(1.0, float(np.max(np.abs(mixed[np.isfinite(mixed)]))))
        assert max_abs(npf(ys), ref) <= tol


def test_head_linear_ignores_input_above_diagonal():
    inp = make_head_linear_inputs(1, 16, 128, torch.bfloat16, seed=77)
    x = inp["x"].clone()
    iu = torch.triu_indices(128, 128, 1)
    x[..., iu[0], iu[1]] = float("nan")
    y = ops.head_linear_fwd(x.to(DEV), inp["W"].to(DEV), True, 0.0)
    ref = orc.head_linear(npf(inp["x"]), npf(inp["W"]), True, 0.0, orc.ROUND_BF16)
    one_stage_close(npf(y), ref, torch.bfloat16, "nan above the diagonal")


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("S", [1, 5, 64, 130, 1000])
def test_softmax(S, dtype):
    g = torch.Generator().manual_seed(S)
    x = (3 * torch.randn(2, 3, S, S, generator=g)).to(dtype)
    y = ops.softmax_fwd(x.to(DEV), True)
    ref = orc.softmax(npf(x), True, ROUND[dtype])
    one_stage_close(npf(y), ref, dtype, f"softmax S={S}")
    xm = x.clone()
    xm[..., torch.triu_indices(S, S, 1)[0], torch.triu_indices(S, S, 1)[1]] = float("-inf")
    y2 = ops.softmax_fwd(xm.to(DEV), False)      # the -inf filled tensor of the reference, full rows
    one_stage_close(npf(y2), ref, dtype, f"softmax of -inf filled S={S}")


@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("C,S", [(16, 72), (16, 520), (7, 64), (32, 136), (4, 8), (16, 1304), (48, 40), (16, 67)])
def test_head_linear_softmax(C, S, dtype, variant):
    """Head mix + softmax in one pass (variant 0 where the shape allows it) against the oracle's two stages."""
    g = torch.Generator().manual_seed(900 + C + S)
    x = (3 * torch.randn(2, C, S, S, generator=g)).to(dtype)          # conv-output-like logits, peaked softmax
    W32 = torch.eye(C) + 0.5 * torch.randn(C, C, generator=g)          # not representable in 16 bits
    W = W32 if variant == 0 else W32.to(dtype)
    _lib.set_variant("fused", variant)
    try:
        y = ops.head_linear_softmax_fwd(x.to(DEV), W.to(DEV))
    finally:
        _lib.set_variant("fused", 0)
    _lib.device_status()
    mixed = orc.head_linear(npf(x), npf(W), True, float("-inf"), ROUND[dtype])
    ref = orc.softmax(mixed, True, ROUND[dtype])
    # a logit that rounds the other way (fp32 against the oracle's double accumulation) moves its probability by up to
    # one ulp of the LOGIT, relative
    tol = 2.0 * ULP[dtype] * max(1.0, float(np.max(np.abs(mixed[np.isfinite(mixed)]))))
    assert max_abs(npf(y), ref) <= tol, f"head mix + softmax C={C} S={S}: {max_abs(npf(y), ref):.3e} > {tol:.3e}"
    iu = np.triu_indices(S, 1)
    assert np.all(npf(y)[..., iu[0], iu[1]] == 0)
    np.testing.assert_allclose(npf(y).sum(-1), 1.0, atol=4 * ULP[dtype] * np.sqrt(S) + 1e-6)


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("C,S", [(16, 72), (16, 128), (16, 520), (16, 1304), (8, 264), (32, 136), (32, 1032), (64, 200), (128, 136)])
def test_head_linear_softmax_16bit_weights(C, S, dtype, variant):
    """Weights in the activations' dtype: the tcgen05 kernel (variant 2: two passes over key tiles, the mix recomputed)
    and the mma.sync kernel (variant 1, up to 32 heads) against the oracle's two stages; NaN above the diagonal of the
    input must change nothing."""
    if variant == 1 and C > 32:
        pytest.skip("the mma.sync kernel takes up to 32 heads")
    g = torch.Generator().manual_seed(1900 + C + S)
    x = (3 * torch.randn(2, C, S, S, generator=g)).to(dtype)
    W = (torch.eye(C) + 0.5 * torch.randn(C, C, generator=g)).to(dtype)
    xn = x.clone()
    iu = torch.triu_indices(S, S, 1)
    xn[..., iu[0], iu[1]] = float("nan")
    _lib.set_variant("mix_softmax", variant)
    try:
        _lib.reset_launch_count()
        y = ops.head_linear_softmax_fwd(x.to(DEV), W.to(DEV))
        assert _lib.launch_count() == 1
        yn = ops.head_linear_softmax_fwd(xn.to(DEV), W.to(DEV))
    finally:
        _lib.set_variant("mix_softmax", 0)
    _lib.device_status()
    assert torch.equal(y, yn)
    mixed = orc.head_linear(npf(x), npf(W), True, float("-inf"), ROUND[dtype])
    ref = orc.softmax(mixed, True, ROUND[dtype])
    tol = 2.0 * ULP[dtype] * max(1.0, float(np.max(np.abs(mixed[np.isfinite(mixed)]))))
    assert max_abs(npf(y), ref) <= tol, f"head mix + softmax C={C} S={S}: {max_abs(npf(y), ref):.3e} > {tol:.3e}"
    assert np.all(npf(y)[..., iu[0], iu[1]] == 0)
    np.testing.assert_allclose(npf(y).sum(-1), 1.0, atol=4 * ULP[dtype] * np.sqrt(S) + 1e-6)


def test_head_linear_softmax_is_reproducible_and_ignores_upper_input():
    inp = make_head_linear_inputs(1, 16, 264, torch.bfloat16, seed=41)
    x = (inp["x"].float() * 40).to(torch.bfloat16).to(DEV)
    y = ops.head_linear_softmax_fwd(x, inp["W"].to(DEV))
    xn = x.clone()
    iu = torch.triu_indices(264, 264, 1)
    xn[..., iu[0], iu[1]] = float("nan")
    assert torch.equal(ops.head_linear_softmax_fwd(xn, inp["W"].to(DEV)), y)
    two = ops.softmax_fwd(ops.head_linear_fwd(x, inp["W"].to(DEV), True, float("-inf")), True)
    assert rel_max(npf(y), npf(two)) <= 2 * ULP[torch.bfloat16]


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("S,D", [(5, 8), (65, 16), (130, 64), (256, 128), (128, 64), (200, 128), (8, 64), (1000, 128)])
def test_contractions(S, D, dtype, variant):
    """variant 1 = CUDA-core kernels, 2 = tcgen05 kernels (16-bit dtypes, D in {64,128}, S % 8 == 0)."""
    if variant >= 2 and (dtype == torch.float32 or D not in (64, 128) or S % 8):
        pytest.skip("outside the tensor-core kernels' domain")
    _lib.set_variant("gemm", variant)
    try:
        _contractions(S, D, dtype)
        _lib.device_status()
    finally:
        _lib.set_variant("gemm", 0)


def _contractions(S, D, dtype):
    g = torch.Generator().manual_seed(S + D)
    q, k, v = (torch.randn(2, 3, S, D, generator=g).to(dtype) for _ in range(3))
    s = ops.qk_scores_fwd(q.to(DEV), k.to(DEV), D ** -0.5, True)
    ref = torch.tril(torch.matmul(q.double(), k.double().transpose(2, 3)))
    if dtype == torch.float32:
        ref = ref * D ** -0.5
    else:   # matmul rounded, times the rounded scale, rounded (mta_attention_pytorch.py:63-65)
        ref = (ref.to(dtype).double() * torch.tensor(D ** -0.5).to(dtype).double()).to(dtype).double()
    one_stage_close(npf(s), ref.float().numpy(), dtype, "scores")
    p = torch.tril(torch.softmax(torch.randn(2, 3, S, S, generator=g), -1)).to(dtype)
    pg = p.clone()
    iu = torch.triu_indices(S, S, 1)
    pg[..., iu[0], iu[1]] = float("nan")           # whatever sits above the diagonal must not be read
    o = ops.pv_fwd(pg.to(DEV), v.to(DEV), True)
    oref = torch.matmul(p.double(), v.double())
    one_stage_close(npf(o), oref.float().numpy(), dtype, "pv")
    # non-causal: full rows
    pf = torch.softmax(torch.randn(2, 3, S, S, generator=g), -1).to(dtype)
    o2 = ops.pv_fwd(pf.to(DEV), v.to(DEV), False)
    one_stage_close(npf(o2), torch.matmul(pf.double(), v.double()).float().numpy(), dtype, "pv non-causal")
    s2 = ops.qk_scores_fwd(q.to(DEV), k.to(DEV), 1.0, False, round_like_reference=False)
    one_stage_close(npf(s2), torch.matmul(q.double(), k.double().transpose(2, 3)).float().numpy(), dtype, "scores non-causal")


# ---------------------------------------------------------------------------------------------
def build_mta(wl, inp, fused):
    import types
    cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=wl.cq, key_kernel_size=wl.ck,
                                after_sm_query_kernel_size=wl.cq2, after_sm_key_kernel_size=wl.ck2,
                                pre_sm_linear_head=True, post_sm_linear_head=True, pad_key="both",
                                init_method="identity", dim=wl.H * wl.D)
    m = MTAAttentionTriton(wl.H, cfg, dropout=0.0, causal=True, fused=fused).to(DEV).to(wl.dtype).eval()
    with torch.no_grad():
        m.mta_conv_triton.weight.copy_(inp["w1"])
        m.wpsm_triton.weight.copy_(inp["W1"])
        m.mta_conv_after_sm_triton.weight.copy_(inp["w2"])
        m.wposm_triton.weight.copy_(inp["W2"])
    return m


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("name", list(MTA_CASES))
def test_mta_forward(name, fused, golden):
    wl = MTA_CASES[name]
    inp = make_mta_inputs(wl)
    m = build_mta(wl, inp, fused)
    with torch.no_grad():
        out = m(inp["q"].to(DEV), inp["k"].to(DEV), inp["v"].to(DEV), None, None)
    assert out.shape == (wl.B, wl.S, wl.H, wl.D) and out.dtype == wl.dtype
    assert not out.is_contiguous() or wl.S == 1 or wl.H == 1     # the (B,S,H,D) transpose view, as the reference returns
    got = npf(out.transpose(1, 2))
    a = [npf(inp[k]) for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    exact = orc.mta_fwd(*a, True, orc.ROUND_NONE)
    assert_parity(got, exact, wl.dtype, f"{name} vs oracle")
    assert_parity(got, golden[f"mta/{name}"], wl.dtype, f"{name} vs golden")
    if wl.dtype != torch.float32:
        staged = orc.mta_fwd(*a, True, ROUND[wl.dtype])
        assert_parity(got, staged, wl.dtype, f"{name} vs stage-rounded oracle")


@pytest.mark.parametrize("name", ["s130_6x11_bf16", "s128_11x15_bf16", "s192_h32_f16"])
def test_scores_computed_inside_the_first_conv_change_no_bit(name):
    """Default forward (Q K^T computed inside the first conv's kernel, never stored) against the forward with the two
    kernels apart: the conv reads the same rounded scores in the same order, so the outputs are identical - also for a
    row range, whose tiles start at other rows."""
    wl = MTA_CASES[name]
    inp = make_mta_inputs(wl)
    args = [inp[k].to(DEV) for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    folded = ops.mta_fused_fwd(*args, True)
    part = torch.zeros_like(folded)
    ops.mta_fused_fwd(*args, True, rows=(9, wl.S - 2), out=part)
    _lib.device_status()
    try:
        _lib.set_variant("fused", 3)
        apart = ops.mta_fused_fwd(*args, True)
    finally:
        _lib.set_variant("fused", 0)
    _lib.device_status()
    assert torch.equal(folded, apart)
    assert torch.equal(part[:, :, 9:wl.S - 2], folded[:, :, 9:wl.S - 2])


@pytest.mark.parametrize("H,dtype", [(16, torch.bfloat16), (32, torch.float16), (8, torch.bfloat16)])
def test_row_range_over_many_key_tiles_changes_no_bit(H, dtype):
    """Rows long enough for eight key tiles of the head mix + softmax kernel, whose partial row statistics come from four
    groups of warps: a row range that starts at an odd row (other row groups, other tile counts before each unit) must
    reproduce the full run bit for bit, and two full runs must agree."""
    wl = MTAWorkload("rowrange", 2, H, 1000, 64, 6, 11, 3, 3, dtype, seed=300 + H, random_post_conv=True)
    inp = make_mta_inputs(wl)
    args = [inp[k].to(DEV) for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    full = ops.mta_fused_fwd(*args, True)
    assert torch.equal(full, ops.mta_fused_fwd(*args, True))
    for r0, r1 in ((37, 911), (512, 1000), (0, 130)):
        part = torch.zeros_like(full)
        ops.mta_fused_fwd(*args, True, rows=(r0, r1), out=part)
        assert torch.equal(part[:, :, r0:r1], full[:, :, r0:r1]), f"rows [{r0},{r1})"
    _lib.device_status()
    a = [npf(inp[k]) for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    assert_parity(npf(full), orc.mta_fwd(*a, True, orc.ROUND_NONE), dtype, f"H{H} S1000 vs oracle")


@pytest.mark.parametrize("H,S,D,cq,ck,dtype", [(128, 72, 32, 3, 5, torch.float16), (4, 160, 64, 77, 77, torch.float16),
                                              (64, 96, 64, 6, 11, torch.bfloat16), (2, 200, 128, 21, 21, torch.float32)])
def test_mta_forward_published_shape_limits(H, S, D, cq, ck, dtype):
    """Shapes at the edges of what the reference publishes numbers for (up to 128 heads, conv kernels up to 77 x 77,
    fp16): they run through the general kernels and must match the oracle like every other case."""
    wl = MTAWorkload("limits", 1, H, S, D, cq, ck, 3, 3, dtype, seed=70 + H, random_post_conv=True)
    inp = make_mta_inputs(wl)
    args = [inp[k].to(DEV) for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    out = ops.mta_fused_fwd(*args, True)
    _lib.device_status()
    a = [npf(inp[k]) for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    assert_parity(npf(out), orc.mta_fwd(*a, True, orc.ROUND_NONE), dtype, f"H{H} S{S} {cq}x{ck}")


def test_stage_trace_reports_every_kernel_of_the_forward():
    wl = MTA_CASES["s128_11x15_bf16"]
    inp = make_mta_inputs(wl)
    args = [inp[k].to(DEV) for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    _lib.set_stage_trace(True)
    try:
        ops.mta_fused_fwd(*args, True)
        got = _lib.stage_times_ms()
        assert [n for n, _ in got] == ["qk_scores+conv1", "head_mix1+softmax", "conv2", "head_mix2", "pv"]
        assert all(0.0 < ms < 100.0 for _, ms in got)
        _lib.set_variant("fused", 3)
        ops.mta_fused_fwd(*args, True)
        assert [n for n, _ in _lib.stage_times_ms()] == ["qk_scores", "conv1", "head_mix1+softmax", "conv2", "head_mix2", "pv"]
        _lib.set_variant("fused", 1)
        ops.mta_fused_fwd(*args, True)
        assert [n for n, _ in _lib.stage_times_ms()] == ["qk_scores", "conv1", "head_mix1", "softmax", "conv2", "head_mix2", "pv"]
    finally:
        _lib.set_variant("fused", 0)
        _lib.set_stage_trace(False)
    ops.mta_fused_fwd(*args, True)
    assert _lib.stage_times_ms() == []


@pytest.mark.parametrize("chunk", [0, 1, 2, 3])
@pytest.mark.parametrize("name", ["c1", "s128_11x15_bf16"])
def test_mta_forward_host_matches_device_forward(name, chunk):
    """Host tensors in, host tensor out, batch chunks overlapped on three streams: same bits as the device forward."""
    wl = dataclasses.replace(MTA_CASES[name], B=5)
    inp = make_mta_inputs(wl)
    m = build_mta(wl, inp, True)
    with torch.no_grad():
        want = m(inp["q"].to(DEV), inp["k"].to(DEV), inp["v"].to(DEV), None, None)
        host = [inp[k].pin_memory() for k in ("q", "k", "v")]
        got = m.forward_host(*host, chunk_batch=chunk)
        assert not got.is_cuda and got.shape == want.shape
        assert torch.equal(got, want.cpu())
        again = m.forward_host(inp["q"], inp["k"], inp["v"], chunk_batch=chunk)      # pageable memory works too
        assert torch.equal(again, got)
    _lib.device_status()
    ops.host_pipeline_release()


@pytest.mark.parametrize("name,rows", [("ragged_f32", (3, 20)), ("ragged_f32", (64, 65)), ("s130_6x11_bf16", (17, 130)),
                                       ("c1", (100, 164)), ("s192_h32_f16", (0, 9))])
def test_mta_forward_row_range(name, rows):
    wl = MTA_CASES[name]
    inp = make_mta_inputs(wl)
    d = {k: t.to(DEV) for k, t in inp.items()}
    full = ops.mta_fused_fwd(d["q"], d["k"], d["v"], d["w1"], d["W1"], d["w2"], d["W2"], True)
    out = torch.full_like(full, 7.0)
    ops.mta_fused_fwd(d["q"], d["k"], d["v"], d["w1"], d["W1"], d["w2"], d["W2"], True, rows=rows, out=out)
    r0, r1 = rows
    assert torch.equal(out[:, :, r0:r1], full[:, :, r0:r1]), "a row range must reproduce the rows of the full forward"
    assert torch.all(out[:, :, :r0] == 7.0) and torch.all(out[:, :, r1:] == 7.0), "rows outside the range must not be written"
    a = [npf(inp[k]) for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    ref = orc.mta_fwd_rows(*a, 0, r0, r1, True, orc.ROUND_NONE)
    assert_parity(npf(out[0, :, r0:r1]), ref, wl.dtype, f"{name} rows {rows}")


@pytest.mark.parametrize("name,world", [("c1", 4), ("s130_6x11_bf16", 4), ("s192_h32_f16", 2), ("c1", 2)])
def test_sharded_forward_on_one_gpu(name, world):
    """Every shard of a plan, run one after the other on this GPU through the row-range entry point, reassembles
    into the unsharded forward bit for bit (the multi-process gather itself is covered on CPU ranks)."""
    from multitokenatention_triton_b200 import sharding
    wl = MTA_CASES[name]
    inp = make_mta_inputs(wl)
    d = {k: t.to(DEV) for k, t in inp.items()}
    weights = [d[n] for n in ("w1", "W1", "w2", "W2")]
    full = ops.mta_fused_fwd(d["q"], d["k"], d["v"], *weights, True)
    out = torch.zeros_like(full)
    for b0, b1, r0, r1 in sharding.plan_shards(wl.B, wl.S, world, row_align=16):
        loc = sharding.local_forward(d["q"][b0:b1], d["k"][b0:b1], d["v"][b0:b1], weights, (b0, b1, r0, r1))
        out[b0:b1, :, r0:r1] = loc
    assert torch.equal(out, full)


@pytest.mark.parametrize("name", list(CONV_ATTN_CASES))
def test_conv_attention(name, golden):
    wl, causal = CONV_ATTN_CASES[name]
    inp = make_mta_inputs(wl)
    m = TritonConvAttention(wl.H, (wl.cq, wl.ck), causal=causal).to(DEV).to(wl.dtype)
    with torch.no_grad():
        m.weight.copy_(inp["w1"])
        res = m(inp["q"].to(DEV), inp["k"].to(DEV), inp["v"].to(DEV), causal, wl.D ** -0.5)
    out = res[0]
    assert out.shape == (wl.B, wl.H, wl.S, wl.D)
    a = [npf(inp[k]) for k in ("q", "k", "v", "w1")]
    ref = orc.conv_attn_fwd(*a, causal, None, orc.ROUND_NONE)
    assert_parity(npf(out), ref, wl.dtype, f"{name} vs oracle")
    assert_parity(npf(out), golden[f"conv_attn/{name}"], wl.dtype, f"{name} vs golden")


def test_error_paths_on_device():
    x = torch.zeros(1, 2, 8, 8, device=DEV)
    with pytest.raises(AssertionError):
        ops.head_linear_fwd(x, torch.eye(3, device=DEV))
    with pytest.raises(_lib.MTALibraryError):
        ops.head_linear_fwd(torch.zeros(1, 200, 8, 8, device=DEV), torch.eye(200, device=DEV))
    with pytest.raises(_lib.MTALibraryError):
        ops.conv2d_fwd(x.to(torch.float64), torch.zeros(2, 3, 3, device=DEV, dtype=torch.float64), True)
    with pytest.raises(_lib.MTALibraryError):   # even key kernel
        q = torch.zeros(1, 2, 8, 8, device=DEV)
        ops.mta_fused_fwd(q, q, q, torch.zeros(2, 3, 4, device=DEV), torch.eye(2, device=DEV),
                          torch.zeros(2, 3, 3, device=DEV), torch.eye(2, device=DEV))
    # the context is still healthy
    assert torch.isfinite(ops.softmax_fwd(torch.randn(1, 1, 8, 8, device=DEV))).all()


@pytest.mark.parametrize("dtype,S,D", [(torch.bfloat16, 256, 128), (torch.float32, 136, 64)])
def test_forward_replays_from_a_cuda_graph(dtype, S, D):
    """mta_fused_fwd with caller-owned output and workspace makes no allocation and no host synchronisation, so a
    stream capture records it; the replay on new inputs written into the same buffers equals the direct call."""
    from multitokenatention_triton_b200.synthetic import MTAWorkload, make_mta_inputs
    wl = MTAWorkload("graph", 2, 16, S, D, 6, 11, 3, 3, dtype, 77, random_post_conv=True)
    t = {k: v.to(DEV) for k, v in make_mta_inputs(wl).items()}
    out = torch.empty_like(t["q"])
    nbytes = _lib.lib().mta_workspace_bytes(wl.B, wl.H, S, D, 6, 11, 3, 3, 0, S, _lib.dtype_code(t["q"]))
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)

    def run():
        ops.mta_fused_fwd(t["q"], t["k"], t["v"], t["w1"], t["W1"], t["w2"], t["W2"], True, out=out, workspace=ws)
    run()                                       # per-device setup happens on the first call, outside the capture
    _lib.device_status()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            run()
    torch.cuda.synchronize()
    fresh = make_mta_inputs(MTAWorkload("graph2", 2, 16, S, D, 6, 11, 3, 3, dtype, 78, random_post_conv=True))
    for key in ("q", "k", "v"):
        t[key].copy_(fresh[key])
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    replayed = out.clone()
    out.zero_()
    run()
    _lib.device_status()
    assert torch.equal(replayed, out) and torch.count_nonzero(out) > 0
