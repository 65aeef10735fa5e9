"""B200-native (sm_100a) Multi-Token-Attention forward, behind the reference project's Python API.

The compute lives in libmta_b200.so (hand-written CUDA, C ABI in include/mta_b200.h), built in-tree by
`python -m multitokenatention_triton_b200.build`.  There is no Triton, no CPU path and no fallback.
"""
from .convolution_2d import Conv2dTriton, Conv2dTritonFunction
from .linear_head import TritonLinearHead, TritonLinearHeadFunction
from .conv_attention import TritonAttention, TritonConvAttention
from .mta_attention import MTAAttentionTriton

__all__ = [
    "Conv2dTriton", "Conv2dTritonFunction", "TritonLinearHead", "TritonLinearHeadFunction",
    "TritonAttention", "TritonConvAttention", "MTAAttentionTriton",
]
