"""Case tables shared by the golden-vector generator and the tests: small, seeded, ragged sizes."""
import os
import sys

import torch

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..")))
from multitokenatention_triton_b200.synthetic import WORKLOADS, MTAWorkload  # noqa: E402

f32, bf16, f16 = torch.float32, torch.bfloat16, torch.float16

# name -> workload for the full four-stage forward (oracle: MTAAttention)
MTA_CASES = {
    "c1": WORKLOADS["c1"],
    "c1b": WORKLOADS["c1b"],
    "ragged_f32": MTAWorkload("ragged_f32", 1, 3, 65, 16, 3, 5, 3, 3, f32, 11, mix_var=0.05, random_post_conv=True),
    "tiny_f32": MTAWorkload("tiny_f32", 2, 2, 5, 8, 2, 3, 2, 1, f32, 12, mix_var=0.05, random_post_conv=True),
    "one_f32": MTAWorkload("one_f32", 1, 1, 1, 8, 1, 1, 1, 1, f32, 13),
    "s130_6x11_bf16": MTAWorkload("s130_6x11_bf16", 1, 4, 130, 32, 6, 11, 3, 3, bf16, 14, random_post_conv=True),
    "s257_6x11_f32": MTAWorkload("s257_6x11_f32", 1, 8, 257, 64, 6, 11, 3, 3, f32, 15, random_post_conv=True),
    "s128_11x15_bf16": MTAWorkload("s128_11x15_bf16", 2, 8, 128, 64, 11, 15, 5, 7, bf16, 16, random_post_conv=True),
    "s192_h32_f16": MTAWorkload("s192_h32_f16", 1, 32, 192, 64, 6, 11, 3, 3, f16, 17, random_post_conv=True),
}

# name -> (N, C, S, D, R, Sk, dtype, seed, causal) for the standalone conv (oracle: pytorch_conv)
CONV_CASES = {
    "s1": (1, 1, 1, 8, 1, 1, f32, 21, True),
    "s5_3x3": (2, 2, 5, 8, 3, 3, f32, 22, True),
    "s63_3x5": (1, 3, 63, 16, 3, 5, f32, 23, True),
    "s64_6x11": (2, 2, 64, 16, 6, 11, bf16, 24, True),
    "s65_6x11": (1, 2, 65, 16, 6, 11, f32, 25, True),
    "s127_11x15": (1, 2, 127, 16, 11, 15, bf16, 26, True),
    "s130_6x11": (1, 3, 130, 32, 6, 11, f32, 27, True),
    "s257_3x3": (1, 2, 257, 32, 3, 3, bf16, 28, True),
    "s256_6x11_f16": (1, 4, 256, 64, 6, 11, f16, 29, True),
    "s130_5x7_noncausal": (1, 2, 130, 32, 5, 7, f32, 30, False),
    "s64_6x11_noncausal": (1, 2, 64, 16, 6, 11, bf16, 31, False),
}

# name -> (N, C, S, dtype, seed, causal, fill) for the standalone head mix (oracle: F.linear on the transposed view)
NEG_INF = float("-inf")
HEAD_CASES = {
    "s1_h1": (1, 1, 1, f32, 41, True, 0.0),
    "s5_h3": (2, 3, 5, f32, 42, True, NEG_INF),
    "s63_h8": (1, 8, 63, f32, 43, True, 0.0),
    "s64_h16": (2, 16, 64, bf16, 44, True, NEG_INF),
    "s65_h16": (1, 16, 65, bf16, 45, True, 0.0),
    "s130_h32": (1, 32, 130, bf16, 46, True, NEG_INF),
    "s128_h16_f16": (1, 16, 128, f16, 47, True, 0.0),
    "s193_h5": (1, 5, 193, f32, 48, True, 0.0),
    "s64_h16_noncausal": (1, 16, 64, bf16, 49, False, 0.0),
    "s130_h8_noncausal": (1, 8, 130, f32, 50, False, 0.0),
}

# name -> (workload (only cq,ck and q,k,v,w1 used), causal) for the fused conv attention (oracle: ConvAttention)
CONV_ATTN_CASES = {
    "s130_3x5_f32": (MTAWorkload("ca1", 2, 4, 130, 32, 3, 5, dtype=f32, seed=61), True),
    "s257_6x11_f32": (MTAWorkload("ca2", 1, 2, 257, 64, 6, 11, dtype=f32, seed=62), True),
    "s128_6x11_bf16": (MTAWorkload("ca3", 1, 4, 128, 128, 6, 11, dtype=bf16, seed=63), True),
    "s65_3x3_f32_noncausal": (MTAWorkload("ca4", 1, 2, 65, 16, 3, 3, dtype=f32, seed=64), False),
}


# Backward cases: subsets of the tables above; the upstream gradient is make_upstream_grad(shape, dtype, seed + 1000).
CONV_BWD_CASES = ["s1", "s5_3x3", "s63_3x5", "s64_6x11", "s65_6x11", "s130_5x7_noncausal", "s64_6x11_noncausal"]
HEAD_BWD_CASES = ["s1_h1", "s5_h3", "s63_h8", "s64_h16", "s65_h16", "s193_h5", "s64_h16_noncausal"]
BACKWARD_GOLDEN = "golden_backward.npz"
# full-module gradients (dq, dk, dv and the four weights) of these MTA cases; upstream gradient seeded with seed + 2000
MTA_BWD_CASES = ["tiny_f32", "ragged_f32", "c1b"]


# Explicit-mask cases: name -> (MTA case name, mask kind).  Masks (make_mask below): "none" = the causal mask the
# module builds itself; "padding" = a (1, S) boolean key mask (last keys padded out), batch 1; "documents" = a
# (1,1,S,S) additive mask, causal inside concatenated documents and -inf across them.
MASK_CASES = {
    "tiny_none": ("tiny_f32", "none"),
    "ragged_padding": ("ragged_f32", "padding"),
    "ragged_documents": ("ragged_f32", "documents"),
    "s130_bf16_documents": ("s130_6x11_bf16", "documents"),
    "s257_documents": ("s257_6x11_f32", "documents"),
}
MASK_GOLDEN = "golden_masked.npz"


# pad_key = "left" / "right" cases (only the reference's PyTorch module places the key window there,
# mta_attention_pytorch.py:91-98): name -> (MTA workload, pad_key, mask kind).  Forward outputs for all of them; for
# the float32 cases without a mask also the full-module gradients, upstream gradient seeded with seed + 2000.
PADKEY_WORKLOADS = {
    "ragged_f32": MTA_CASES["ragged_f32"],
    "s130_6x11_bf16": MTA_CASES["s130_6x11_bf16"],
    "even_f32": MTAWorkload("even_f32", 2, 3, 37, 16, 3, 4, 2, 2, f32, 71, mix_var=0.05, random_post_conv=True),
}
PADKEY_CASES = {
    "ragged_left": ("ragged_f32", "left", "none"),
    "ragged_right": ("ragged_f32", "right", "none"),
    "even_left": ("even_f32", "left", "none"),
    "even_right": ("even_f32", "right", "none"),
    "s130_bf16_left": ("s130_6x11_bf16", "left", "none"),
    "s130_bf16_right": ("s130_6x11_bf16", "right", "none"),
    "ragged_left_documents": ("ragged_f32", "left", "documents"),
    "ragged_right_documents": ("ragged_f32", "right", "documents"),
}
PADKEY_GOLDEN = "golden_padkey.npz"


def make_mask(kind: str, S: int, dtype):
    """The mask argument of forward for a mask case (None, (1,S) bool, or (1,1,S,S) additive in `dtype`)."""
    if kind == "none":
        return None
    if kind == "padding":
        keep = torch.ones(1, S, dtype=torch.bool)
        keep[:, S - max(1, S // 5):] = False
        return keep
    if kind == "documents":
        bounds = [0, S // 3, (2 * S) // 3 + 1, S]
        doc = torch.zeros(S, dtype=torch.long)
        for i in range(3):
            doc[bounds[i]:bounds[i + 1]] = i
        ok = (doc[:, None] == doc[None, :]) & (torch.arange(S)[:, None] >= torch.arange(S)[None, :])
        return torch.where(ok, 0.0, float("-inf")).to(dtype)[None, None]
    raise ValueError(kind)


def load_golden(path=None):
    """name -> float32 numpy array.  16-bit outputs are stored as bit patterns under 'name@bf16' / 'name@f16'."""
    import numpy as np
    path = path or os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_mta.npz")
    out = {}
    with np.load(path) as z:
        for key in z.files:
            a = z[key]
            if "@" in key:
                name, dt = key.split("@")
                t = torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16 if dt == "bf16" else torch.float16)
                out[name] = t.float().numpy()
            else:
                out[key] = a
    return out
