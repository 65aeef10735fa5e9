"""Places the reference's own hot-path modules under oracle/_ref/ so that benchmarks can time them.

    python oracle/make_ref.py /path/to/multitokenatention_triton

The reference is a flat directory of Python scripts with no installer.  This copies, unmodified, the seven
modules the MTA forward path consists of into oracle/_ref/ (git-ignored: the files are the reference's, not this
repository's; the folder travels with a working copy like the built libraries do).  Test and benchmark
infrastructure only: nothing in the package imports it.  oracle/ref_runner.py loads the modules from there.
"""
import os
import shutil
import sys

HOT_PATH_MODULES = [
    "mta_attention_pytorch.py",      # MTAAttention: the ground truth and the CPU baseline
    "mta_attention_triton.py",       # MTAAttentionTriton: the reference's GPU path
    "convolution_2d_trit.py",        # Conv2dTriton + pytorch_conv
    "triton_linear_head.py",         # TritonLinearHead
    "conv_attention_pytorch.py",     # ConvAttention
    "conv_attention_triton.py",      # TritonConvAttention
    "qk_conv_kernel.py",             # device functions conv_attention_triton.py imports
]
HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def make_ref(src: str) -> str:
    missing = [m for m in HOT_PATH_MODULES if not os.path.isfile(os.path.join(src, m))]
    if missing:
        raise FileNotFoundError(f"{src} does not look like the reference checkout: missing {missing}")
    os.makedirs(DEST, exist_ok=True)
    for m in HOT_PATH_MODULES:
        shutil.copyfile(os.path.join(src, m), os.path.join(DEST, m))
    return DEST


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    print(make_ref(sys.argv[1]))
