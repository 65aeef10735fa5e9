"""The configurations the roofline targets are quoted on, at full size, on the GPU.

The CPU oracle cannot evaluate a whole 4 GB score plane in seconds, so these tests compare (a) whole planes or
row blocks that the oracle can do quickly, and (b) size-independent properties: exact zero / fill above the
diagonal everywhere, exact linearity under a power-of-two scale, and row ranges reproducing the full result.
"""
import dataclasses

import numpy as np
import pytest
import torch

from multitokenatention_triton_b200 import _lib, ops
from multitokenatention_triton_b200.synthetic import WORKLOADS, make_conv_inputs, make_head_linear_inputs, make_mta_inputs
from oracle import mta_oracle as orc
from util import BF16_REL, assert_parity, max_abs, npf, rel_fro, rel_max

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF16_ULP = 2.0 ** -8


def block_parity(got, args, r0, r1, what):
    """A block of output rows of a bf16 forward.  Against the oracle with the reference's 16-bit rounding points
    emulated the library must agree closely (it rounds where the reference rounds); against the exact evaluation the
    norm-wise 2e-2 holds, while the largest element of so small a block may deviate more - the reference's own bf16
    pipeline does (the rounding-emulating oracle is up to 2.6e-2 of the block's largest value away from the exact one)."""
    exact = orc.mta_fwd_rows(*args, 0, r0, r1, True, orc.ROUND_NONE)
    as_ref = orc.mta_fwd_rows(*args, 0, r0, r1, True, orc.ROUND_BF16)
    f, m = rel_fro(got, as_ref), rel_max(got, as_ref)
    assert f <= 4e-3 and m <= 2e-2, f"{what} vs the oracle with the reference's rounding points: rel fro {f:.3e}, rel max {m:.3e}"
    f = rel_fro(got, exact)
    assert f <= BF16_REL, f"{what} vs the exact oracle: rel fro {f:.3e}"


def test_c2_conv_full_size():
    """Config 2: causal 6x11 conv on a (4,16,2048,2048) bf16 plane of QK^T/sqrt(128) scores, upper triangle left as computed."""
    inp = make_conv_inputs(4, 16, 2048, 128, 6, 11, torch.bfloat16, seed=1)
    x, w = inp["x"].to(DEV), inp["w"].to(DEV)
    y = ops.conv2d_fwd(x, w, True)
    _lib.device_status()
    assert torch.count_nonzero(torch.triu(y, diagonal=1)) == 0, "output above the diagonal must be exactly 0"
    rng = np.random.default_rng(2)
    planes = [(0, 0), (3, 15)] + [(int(rng.integers(4)), int(rng.integers(16))) for _ in range(2)]
    for n, c in planes:                              # whole planes (two fixed, two drawn) against the oracle
        ref = orc.conv2d(npf(inp["x"][n:n + 1, c:c + 1]), npf(inp["w"][c:c + 1]), True, orc.ROUND_BF16)
        got = npf(y[n:n + 1, c:c + 1])
        assert max_abs(got, ref) <= 2 * BF16_ULP * max(1.0, np.abs(ref).max())
    y2 = ops.conv2d_fwd(x * 2, w, True)              # exact linearity under a power-of-two scale
    assert torch.equal(y2, y * 2)
    xz = torch.tril(x)                               # what sits above the diagonal of the input is ignored
    assert torch.equal(ops.conv2d_fwd(xz, w, True), y)


@pytest.mark.parametrize("fill", [0.0, float("-inf")])
def test_c3_head_linear_full_size(fill):
    """Config 3: 16x16 head mix on causal post-softmax probabilities (4,16,2048,2048) bf16."""
    inp = make_head_linear_inputs(4, 16, 2048, torch.bfloat16, seed=2)
    x, W = inp["x"].to(DEV), inp["W"].to(DEV)
    y = ops.head_linear_fwd(x, W, True, fill)
    _lib.device_status()
    upper = torch.triu(torch.ones(2048, 2048, dtype=torch.bool, device=DEV), diagonal=1)
    assert torch.all(y[..., upper] == fill), "entries above the diagonal must equal output_value"
    ref = orc.head_linear(npf(inp["x"][1:2, :, :512, :512]), npf(inp["W"]), True, fill, orc.ROUND_BF16)   # top-left corner
    got = npf(y[1:2, :, :512, :512])
    fin = np.isfinite(ref)
    assert np.array_equal(fin, np.isfinite(got)) and np.max(np.abs(got[fin] - ref[fin])) <= 2 * BF16_ULP
    # seeded random row blocks of random batch elements against a float32 evaluation of the same einsum
    rng = np.random.default_rng(3)
    for _ in range(4):
        n, r0 = int(rng.integers(4)), int(rng.integers(0, 2048 - 16))
        r32 = torch.einsum("oh,hpq->opq", W.float(), x[n, :, r0:r0 + 16].float())
        lowb = ~upper[r0:r0 + 16]
        assert torch.max(torch.abs(y[n, :, r0:r0 + 16].float() - r32)[..., lowb]) <= 2 * BF16_ULP
    # bottom rows against a float32 evaluation of the same einsum
    r32 = torch.einsum("oh,bhpq->bopq", W.float(), x[:, :, 2040:].float())
    low = ~upper[2040:]
    assert torch.max(torch.abs(y[:, :, 2040:].float() - r32)[..., low]) <= 2 * BF16_ULP


def test_c4_full_forward_sampled_rows():
    """Config 4: full MTA forward B8 H16 S4096 D128 bf16; row blocks of two batch elements against the oracle,
    and a row range against the full result."""
    wl = WORKLOADS["c4b"]                            # random post-softmax conv: no stage is trivially skippable
    inp = make_mta_inputs(wl)
    d = {k: t.to(DEV) for k, t in inp.items()}
    weights = [d[n] for n in ("w1", "W1", "w2", "W2")]
    out = ops.mta_fused_fwd(d["q"], d["k"], d["v"], *weights, True)
    _lib.device_status()
    assert torch.isfinite(out).all()
    rng = np.random.default_rng(4)
    for b in (0, 7, int(rng.integers(1, 7))):
        one = {k: npf(inp[k][b:b + 1]) for k in ("q", "k", "v")}
        wts = [npf(inp[n]) for n in ("w1", "W1", "w2", "W2")]
        blocks = [(0, 16), (4080, 4096)] + [(r, r + 16) for r in (int(x) for x in rng.integers(16, 4064, size=2))]
        for r0, r1 in blocks:                        # first rows, last rows and two blocks drawn from the interior
            block_parity(npf(out[b, :, r0:r1]), (one["q"], one["k"], one["v"], *wts), r0, r1, f"c4 b={b} rows [{r0},{r1})")
    part = torch.zeros_like(out[:2])
    ops.mta_fused_fwd(d["q"][:2], d["k"][:2], d["v"][:2], *weights, True, rows=(1024, 1280), out=part)
    assert torch.equal(part[:, :, 1024:1280], out[:2, :, 1024:1280])


def test_c5_shape_one_batch_element():
    """Config 5's shape (H32 S8192 D128) on one batch element: the last row block against the oracle."""
    wl = dataclasses.replace(WORKLOADS["c5"], B=1, random_post_conv=True)
    inp = make_mta_inputs(wl)
    d = {k: t.to(DEV) for k, t in inp.items()}
    out = ops.mta_fused_fwd(d["q"], d["k"], d["v"], d["w1"], d["W1"], d["w2"], d["W2"], True)
    _lib.device_status()
    args = [npf(inp[n]) for n in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    rng = np.random.default_rng(5)
    for r0 in [0, 8180] + [int(x) for x in rng.integers(12, 8100, size=2)]:      # first rows, last rows, two interior blocks
        block_parity(npf(out[0, :, r0:r0 + 12]), args, r0, r0 + 12, f"c5 rows [{r0},{r0 + 12})")
