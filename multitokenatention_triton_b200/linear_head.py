"""Head-mixing linear over the head axis of (batch, heads, seq, seq) planes, with the reference's names.

Mirrors TritonLinearHeadFunction / TritonLinearHead (triton_linear_head.py:281-401): weight (H,H) in
nn.Linear orientation, `causal`, and `output_value` written above the diagonal.  The forward runs the
CUDA kernel behind mta_head_linear_fwd, the backward those behind mta_head_linear_bwd_input /
mta_head_linear_bwd_weight.
"""
import torch
import torch.nn as nn

from . import ops


class TritonLinearHeadFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, causal=True, output_value=0.0):
        ctx.save_for_backward(input, weight)
        ctx.causal = causal
        return ops.head_linear_fwd(input, weight, causal, output_value)

    @staticmethod
    def backward(ctx, grad_output):
        # the reference's backward (triton_linear_head.py:321-370); entries above the diagonal carry no gradient
        input, weight = ctx.saved_tensors
        grad_input = grad_weight = None
        grad_output = grad_output.to(input.dtype)
        if ctx.needs_input_grad[0]:
            grad_input = ops.head_linear_bwd_input(grad_output, weight, ctx.causal)
        if ctx.needs_input_grad[1]:
            grad_weight = ops.head_linear_bwd_weight(input, grad_output, ctx.causal).to(weight.dtype)
        return grad_input, grad_weight, None, None


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
