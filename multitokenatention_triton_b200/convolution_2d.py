"""Depthwise causal 2-D convolution over score planes: the module, with the reference's names.

Mirrors Conv2dTritonFunction / Conv2dTriton of the reference (convolution_2d_trit.py:300-401): same
constructor, same weight shape (C,R,S), same default initialisation, same forward and backward
semantics.  The forward runs the CUDA kernel behind mta_conv2d_fwd, the backward those behind
mta_conv2d_bwd_input / mta_conv2d_bwd_weight.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.autograd import Function

from . import ops


class Conv2dTritonFunction(Function):
    @staticmethod
    def forward(ctx, input, weight, causal):
        ctx.save_for_backward(input, weight)
        ctx.causal = causal
        return ops.conv2d_fwd(input, weight, causal)

    @staticmethod
    def backward(ctx, grad_output):
        # the reference's backward (convolution_2d_trit.py:335-378); the weight gradient comes back in the weight's dtype
        input, weight = ctx.saved_tensors
        grad_input = grad_weight = None
        grad_output = grad_output.to(input.dtype)
        if ctx.needs_input_grad[0]:
            grad_input = ops.conv2d_bwd_input(grad_output, weight, ctx.causal)
        if ctx.needs_input_grad[1]:
            grad_weight = ops.conv2d_bwd_weight(input, grad_output, tuple(weight.shape[1:]), ctx.causal).to(weight.dtype)
        return grad_input, grad_weight, None


class Conv2dTriton(nn.Module):
    """`pad_key` places the key window as MTAAttention._mta_convolution does (mta_attention_pytorch.py:91-103): "both"
    (the reference's Triton kernel, window centred on the key), "left" (keys k-(S-1)..k) or "right" (keys k..k+S-1).
    "left" / "right" run the same kernels on the (C,R,2S-1) kernel that carries the S taps on one side of its centre
    and zeros on the other - the same sums, term by term - and the weight gradient comes back through that padding."""

    def __init__(self, channels, kernel_size, causal=False, pad_key="both"):
        super().__init__()
        if pad_key not in ("both", "left", "right"):
            raise ValueError(f"pad_key must be 'both', 'left' or 'right', not {pad_key!r}")
        self.pad_key = pad_key
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

    def effective_weight(self):
        """The kernel the CUDA entry points take: the weight itself for pad_key "both", else its zero-extended form."""
        S = self.kernel_size[1]
        if self.pad_key == "left":
            return F.pad(self.weight, (0, S - 1))
        if self.pad_key == "right":
            return F.pad(self.weight, (S - 1, 0))
        return self.weight

    def forward(self, x):
        return Conv2dTritonFunction.apply(x, self.effective_weight(), self.causal)
