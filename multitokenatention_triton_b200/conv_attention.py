"""Fused conv attention softmax(scale * conv(Q K^T)) V, with the reference's names.

Mirrors TritonAttention / TritonConvAttention (conv_attention_triton.py:359-502).  The reference returns
(O, QK) where QK is its S x S scratch of raw scores; this implementation keeps no such tensor, so the
second element is None.
"""
import torch
import torch.nn as nn

from . import ops


class TritonAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, Q, K, V, W, causal, softmax_scale):
        return ops.conv_attn_fwd(Q, K, V, W, causal, softmax_scale)

    @staticmethod
    def backward(ctx, dO):
        raise NotImplementedError("the B200 MTA library implements the forward pass only")


class TritonConvAttention(nn.Module):
    def __init__(self, channels, kernel_size, causal=False):
        super().__init__()
        self.channels = channels
        self.kernel_size = kernel_size if isinstance(kernel_size, tuple) else (kernel_size, kernel_size)
        self.causal = causal
        self.weight = nn.Parameter(torch.randn(channels, self.kernel_size[0], self.kernel_size[1]))
        self._init_parameters()

    def _init_parameters(self):
        with torch.no_grad():
            self.weight.zero_()
            self.weight[:, self.kernel_size[0] // 2, self.kernel_size[1] // 2] = 1.0

    def forward(self, Q, K, V, causal, softmax_scale):
        return TritonAttention.apply(Q, K, V, self.weight, causal, softmax_scale), None
