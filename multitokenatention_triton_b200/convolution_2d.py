"""Depthwise causal 2-D convolution over score planes: the module, with the reference's names.

Mirrors Conv2dTritonFunction / Conv2dTriton of the reference (convolution_2d_trit.py:300-401): same
constructor, same weight shape (C,R,S), same default initialisation, same forward semantics.  The
forward runs the CUDA kernel behind mta_conv2d_fwd.
"""
import torch
import torch.nn as nn
from torch.autograd import Function

from . import ops


class Conv2dTritonFunction(Function):
    @staticmethod
    def forward(ctx, input, weight, causal):
        return ops.conv2d_fwd(input, weight, causal)

    @staticmethod
    def backward(ctx, grad_output):
        raise NotImplementedError("the B200 MTA library implements the forward pass only")


class Conv2dTriton(nn.Module):
    def __init__(self, channels, kernel_size, causal=False):
        super().__init__()
        self.channels = channels
        self.kernel_size = kernel_size if isinstance(kernel_size, tuple) else (kernel_size, kernel_size)
        self.causal = causal
        self.weight = nn.Parameter(torch.randn(channels, self.kernel_size[0], self.kernel_size[1]))
        self._init_parameters()

    def _init_parameters(self):
        # reference default (convolution_2d_trit.py:393-398): 1.0 at the geometric centre of the kernel
        with torch.no_grad():
            self.weight.zero_()
            self.weight[:, self.kernel_size[0] // 2, self.kernel_size[1] // 2] = 1.0

    def forward(self, x):
        return Conv2dTritonFunction.apply(x, self.weight, self.causal)
