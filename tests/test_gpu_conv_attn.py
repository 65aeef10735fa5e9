"""The conv attention forward as one kernel (no score plane anywhere): parity with the oracle on ragged and
multi-tile shapes, both 16-bit dtypes and head dimensions, agreement with the stage-by-stage path, reproducibility,
and the full-size shape on sampled row blocks."""
import numpy as np
import pytest
import torch

from multitokenatention_triton_b200 import _lib, ops
from multitokenatention_triton_b200.synthetic import MTAWorkload, make_mta_inputs
from oracle import mta_oracle as orc
from util import assert_parity, npf, rel_fro

pytestmark = pytest.mark.gpu
DEV = "cuda"
bf16, f16 = torch.bfloat16, torch.float16

CASES = {
    # name: workload (B, H, S, D, cq, ck)
    "s1": MTAWorkload("s1", 1, 2, 1, 64, 3, 5, dtype=bf16, seed=81),
    "s5_d64": MTAWorkload("s5_d64", 2, 3, 5, 64, 2, 3, dtype=f16, seed=82),
    "s123_6x11": MTAWorkload("s123_6x11", 1, 4, 123, 128, 6, 11, dtype=bf16, seed=83),       # exactly one row block
    "s124_6x11": MTAWorkload("s124_6x11", 1, 4, 124, 128, 6, 11, dtype=bf16, seed=84),       # one row into the second
    "s257_3x3": MTAWorkload("s257_3x3", 2, 2, 257, 64, 3, 3, dtype=bf16, seed=85),           # ragged S, three key tiles
    "s300_1x1": MTAWorkload("s300_1x1", 1, 2, 300, 128, 1, 1, dtype=f16, seed=86),           # plain attention
    "s515_6x11_f16": MTAWorkload("s515_6x11_f16", 1, 3, 515, 128, 6, 11, dtype=f16, seed=87),
    "s640_6x17": MTAWorkload("s640_6x17", 1, 2, 640, 128, 6, 17, dtype=bf16, seed=88),       # largest kernel the tile takes at D = 128
    "s640_9x17_d64": MTAWorkload("s640_9x17_d64", 1, 2, 640, 64, 9, 17, dtype=bf16, seed=91),
    "s1024_h20": MTAWorkload("s1024_h20", 2, 20, 1024, 128, 6, 11, dtype=bf16, seed=89),     # more units than SMs
}


def run(wl, inp=None, causal=True):
    inp = inp or make_mta_inputs(wl)
    d = {k: inp[k].to(DEV) for k in ("q", "k", "v", "w1")}
    return inp, ops.conv_attn_fwd(d["q"], d["k"], d["v"], d["w1"], causal, wl.D ** -0.5)


@pytest.mark.parametrize("name", list(CASES))
def test_one_kernel_conv_attention_against_the_oracle(name):
    wl = CASES[name]
    L = _lib.lib()
    assert L.mta_conv_attn_workspace_bytes(wl.B, wl.H, wl.S, wl.D, wl.cq, wl.ck, 1, _lib.DTYPE_CODE[wl.dtype],
                                           _lib.DTYPE_CODE[wl.dtype]) == 0, "this shape must need no scratch"
    _lib.reset_launch_count()
    inp, out = run(wl)
    torch.cuda.synchronize()
    assert _lib.launch_count() == 1, "one kernel"
    _lib.device_status()
    ref = orc.conv_attn_fwd(*[npf(inp[k]) for k in ("q", "k", "v", "w1")], True, None, orc.ROUND_NONE)
    assert_parity(npf(out), ref, wl.dtype, name)


@pytest.mark.parametrize("name", ["s124_6x11", "s515_6x11_f16", "s1024_h20"])
def test_one_kernel_agrees_with_the_stage_by_stage_path(name):
    wl = CASES[name]
    inp, out = run(wl)
    _lib.set_variant("fused", 2)                    # scores + conv, softmax and P V as three launches over score planes
    _lib.reset_launch_count()
    try:
        _, staged = run(wl, inp)
    finally:
        _lib.set_variant("fused", 0)
    assert _lib.launch_count() >= 3
    torch.cuda.synchronize()
    # the two differ only by where the softmax rounds (normalised probabilities against exponentials)
    assert rel_fro(npf(out), npf(staged)) <= 8e-3
    _, again = run(wl, inp)
    assert torch.equal(out, again), "the kernel must be bit-reproducible"


def test_float32_weights_fall_back_to_the_staged_path_or_run():
    """float32 conv weights with 16-bit activations: either path must agree with the oracle."""
    wl = CASES["s257_3x3"]
    inp = make_mta_inputs(wl)
    d = {k: inp[k].to(DEV) for k in ("q", "k", "v")}
    out = ops.conv_attn_fwd(d["q"], d["k"], d["v"], inp["w1"].float().to(DEV), True, wl.D ** -0.5)
    ref = orc.conv_attn_fwd(*[npf(inp[k]) for k in ("q", "k", "v", "w1")], True, None, orc.ROUND_NONE)
    assert_parity(npf(out), ref, wl.dtype, "float32 weights")


@pytest.mark.parametrize("dtype", [bf16, f16])
def test_conv_attention_at_b1_h16_s4096(dtype):
    """B1 H16 S4096 D128, 6x11: seeded random row blocks (first rows, interior, last rows) against the oracle."""
    wl = MTAWorkload("ca4096", 1, 16, 4096, 128, 6, 11, dtype=dtype, seed=90)
    inp, out = run(wl)
    _lib.device_status()
    assert torch.isfinite(out).all()
    rng = np.random.default_rng(90)
    starts = [0, 117, 4084] + [int(s) for s in rng.integers(130, 4000, size=3)]
    args = [npf(inp[k]) for k in ("q", "k", "v", "w1")]
    for r0 in starts:
        ref = orc.conv_attn_fwd_rows(*args, 0, r0, r0 + 12, True, None, orc.ROUND_NONE)
        assert_parity(npf(out[0, :, r0:r0 + 12]), ref, dtype, f"rows [{r0},{r0 + 12})")


def test_a_timed_out_wait_is_reported_by_the_next_call_and_cleared_by_device_status():
    """The host marks the device as a kernel's timed-out wait would (nothing is made to wait on the GPU): the next
    forward must return status 4 instead of a result, mta_device_status must report and clear the condition, and the
    forward after that must be right again."""
    wl = CASES["s257_3x3"]
    inp, good = run(wl)
    _lib.device_status()
    L = _lib.lib()
    assert L.mta_inject_wait_timeout(torch.cuda.current_stream().cuda_stream) == 0
    with pytest.raises(_lib.MTALibraryError, match="gave up"):
        run(wl, inp)
    with pytest.raises(_lib.MTALibraryError):
        ops.mta_fused_fwd(*[inp[k].to(DEV) for k in ("q", "k", "v", "w1", "W1", "w2", "W2")], True)
    assert L.mta_device_status(torch.cuda.current_stream().cuda_stream) == 4
    assert L.mta_device_status(torch.cuda.current_stream().cuda_stream) == 0
    _, again = run(wl, inp)
    assert torch.equal(again, good)
