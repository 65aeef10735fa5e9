"""mta_conv_attn_fwd_static: the conv attention forward whose scratch lives inside the library, for callers that
cannot allocate device memory (frozen pools, allocator callbacks, bindings without device buffers).

Called through the C ABI and compared with the workspace-taking entry point it wraps, twice in a row with
different shapes so that the second call runs over what the first left in the shared array.
"""
import ctypes

import numpy as np
import pytest
import torch

from multitokenatention_triton_b200 import _lib, ops
from multitokenatention_triton_b200.synthetic import MTAWorkload, make_mta_inputs
from oracle import mta_oracle as orc
from util import assert_parity, npf

pytestmark = pytest.mark.gpu
DEV = "cuda"


def run_static(d, wl, causal=True):
    L = _lib.lib()
    o = torch.empty_like(d["q"])
    rc = L.mta_conv_attn_fwd_static(d["q"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(), d["w1"].data_ptr(),
                                    o.data_ptr(), wl.B, wl.H, wl.S, wl.D, wl.cq, wl.ck, int(causal), wl.D ** -0.5,
                                    _lib.dtype_code(d["q"]), _lib.dtype_code(d["w1"]),
                                    torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "mta_conv_attn_fwd_static")
    return o


def test_static_scratch_matches_workspace_entry_point_twice():
    L = _lib.lib()
    assert L.mta_static_scratch_bytes() == 64 << 20
    assert L.mta_static_scratch_prepare() == 0           # start-up: the array's address on this device is looked up here
    cases = [MTAWorkload("na1", 1, 8, 1024, 32, 3, 5, dtype=torch.float32, seed=71),        # exactly the 64 MiB the array holds
             MTAWorkload("na2", 2, 4, 200, 64, 3, 19, dtype=torch.float16, seed=72),        # 19 taps wide: stage by stage, over stale contents
             MTAWorkload("na3", 1, 2, 130, 32, 3, 3, dtype=torch.float32, seed=73),         # CUDA-core path, ragged size
             MTAWorkload("na4", 1, 8, 1024, 128, 6, 11, dtype=torch.bfloat16, seed=74)]     # one-kernel path: no scratch at all
    for wl in cases:
        inp = make_mta_inputs(wl)
        d = {k: inp[k].to(DEV) for k in ("q", "k", "v", "w1")}
        got = run_static(d, wl)
        want = ops.conv_attn_fwd(d["q"], d["k"], d["v"], d["w1"], True, wl.D ** -0.5)
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"{wl.name}: the two entry points run the same kernels and must agree exactly"
        ref = orc.conv_attn_fwd(*[npf(inp[k]) for k in ("q", "k", "v", "w1")], True, None, orc.ROUND_NONE)
        assert_parity(npf(got), ref, wl.dtype, wl.name)
    _lib.device_status()


def test_static_scratch_rejects_oversized_problems():
    L = _lib.lib()
    one = ctypes.c_void_p(256)
    rc = L.mta_conv_attn_fwd_static(one, one, one, one, one, 1, 16, 2048, 128, 6, 11, 1, 0.1, 0, 0, None)   # float32: 512 MiB needed
    assert rc == 1 and b"built-in array" in L.mta_last_error()
    rc = L.mta_conv_attn_fwd_static(one, one, one, one, one, 1, 8, 1032, 32, 3, 5, 1, 0.1, 0, 0, None)      # a few rows over 64 MiB
    assert rc == 1 and b"built-in array" in L.mta_last_error()
    rc = L.mta_conv_attn_fwd_static(one, one, one, one, one, 0, 16, 2048, 128, 6, 11, 1, 0.1, 0, 0, None)   # empty batch: no-op
    assert rc == 0
