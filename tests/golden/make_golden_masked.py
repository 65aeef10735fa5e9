"""Generate golden outputs of the explicit-mask forward from the reference's PyTorch module.

    python tests/golden/make_golden_masked.py /path/to/reference

For every case of MASK_CASES (tests/golden/cases.py) the reference's MTAAttention (mta_attention_pytorch.py, which
always works with an explicit mask) is run on the seeded inputs of the named MTA case with the mask the case names,
and the output is stored in golden_masked.npz as (B,H,S,D).  Same two shims as make_golden.py.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))
sys.path.insert(0, HERE)

from multitokenatention_triton_b200.synthetic import make_mta_inputs  # noqa: E402
from cases import MASK_CASES, MASK_GOLDEN, MTA_CASES, make_mask  # noqa: E402
from make_golden import _patch_torch_tensor, store  # noqa: E402


def main(ref_path: str):
    sys.path.insert(0, ref_path)
    _patch_torch_tensor()
    import mta_attention_pytorch as ref_mta
    out = {}
    for name, (mta_case, kind) in MASK_CASES.items():
        wl = MTA_CASES[mta_case]
        inp = make_mta_inputs(wl)
        cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=wl.cq, key_kernel_size=wl.ck,
                                    after_sm_query_kernel_size=wl.cq2, after_sm_key_kernel_size=wl.ck2,
                                    pre_sm_linear_head=True, post_sm_linear_head=True, pad_key="both",
                                    init_method="identity", dim=wl.H * wl.D)
        m = ref_mta.MTAAttention(wl.H, cfg, dropout=0.0).eval().to(wl.dtype)
        mask = make_mask(kind, wl.S, wl.dtype)
        B = 1 if kind == "padding" else wl.B               # the reference's 2-D mask branch is shape-correct for one batch element
        with torch.no_grad():
            m.mta_kernel.copy_(inp["w1"].unsqueeze(1))
            m.wpsm.weight.copy_(inp["W1"])
            m.mta_kernel_after_sm.copy_(inp["w2"].unsqueeze(1))
            m.wposm.weight.copy_(inp["W2"])
            y = m(inp["q"][:B], inp["k"][:B], inp["v"][:B], mask, None)
        store(out, f"masked/{name}", y.transpose(1, 2).contiguous())
        print("masked", name, tuple(y.shape))
    path = os.path.join(HERE, MASK_GOLDEN)
    np.savez_compressed(path, **out)
    print("wrote", path, len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(f"usage: python {sys.argv[0]} /path/to/reference")
    main(sys.argv[1])
