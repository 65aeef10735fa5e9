"""Head-mixing linear over the head axis of (batch, heads, seq, seq) planes, with the reference's names.

Mirrors TritonLinearHeadFunction / TritonLinearHead (triton_linear_head.py:281-401): weight (H,H) in
nn.Linear orientation, `causal`, and `output_value` written above the diagonal.  The forward runs the
CUDA kernel behind mta_head_linear_fwd.
"""
import torch
import torch.nn as nn

from . import ops


class TritonLinearHeadFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, causal=True, output_value=0.0):
        return ops.head_linear_fwd(input, weight, causal, output_value)

    @staticmethod
    def backward(ctx, grad_output):
        raise NotImplementedError("the B200 MTA library implements the forward pass only")


class TritonLinearHead(nn.Module):
    def __init__(self, head_dim, causal=True, output_value=0.0):
        super().__init__()
        self.head_dim = head_dim
        self.weight = nn.Parameter(torch.randn(head_dim, head_dim) / (head_dim ** 0.5))
        self.causal = causal
        self.output_value = output_value

    def forward(self, x):
        return TritonLinearHeadFunction.apply(x, self.weight, self.causal, self.output_value)

    def extra_repr(self):
        return f"head_dim={self.head_dim}"
