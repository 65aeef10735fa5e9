"""The MTA attention module, with the reference's name and interface.

Mirrors MTAAttentionTriton (mta_attention_triton.py:7-201): constructor arguments, sub-module and
parameter names (mta_conv_triton.weight, wpsm_triton.weight, mta_conv_after_sm_triton.weight,
wposm_triton.weight), reset_mta_parameters / copy_mta_parameters, and forward(xq, xk, xv, mask,
chunk_start_ids) returning the (B,S,H,D) transpose view of a (B,H,S,D) tensor.

`fused=True` (default) runs the whole forward through mta_fused_fwd.  `fused=False` runs the reference's
seven steps one by one through the stand-alone entry points, which keeps every 16-bit rounding point of
the reference.
"""
import torch
import torch.nn as nn

from . import ops
from .convolution_2d import Conv2dTriton
from .linear_head import TritonLinearHead


class MTAAttentionTriton(nn.Module):
    def __init__(self, n_heads: int, mta, dropout: float, causal: bool, use_mask: bool = False, fused: bool = True):
        super().__init__()
        assert mta.use_mta, "MTAAttentionTriton can only be used with MTA"
        assert mta.query_kernel_size is not None and mta.key_kernel_size is not None
        assert mta.pre_sm_linear_head is True
        if not hasattr(mta, "after_sm_query_kernel_size"):
            mta.after_sm_query_kernel_size = 3
        if not hasattr(mta, "after_sm_key_kernel_size"):
            mta.after_sm_key_kernel_size = 3
        if not hasattr(mta, "post_sm_linear_head"):
            mta.post_sm_linear_head = True

        self.n_heads = n_heads
        self.mta = mta
        self.dropout = dropout
        self.causal = causal
        self.use_mask = use_mask
        self.fused = fused

        self.mta_conv_triton = Conv2dTriton(n_heads, kernel_size=(mta.query_kernel_size, mta.key_kernel_size), causal=causal)
        self.wpsm_triton = TritonLinearHead(n_heads, causal=causal, output_value=float("-inf"))
        self.mta_conv_after_sm_triton = Conv2dTriton(
            n_heads, kernel_size=(mta.after_sm_query_kernel_size, mta.after_sm_key_kernel_size), causal=causal)
        self.wposm_triton = TritonLinearHead(n_heads, causal=causal)

        self.pad_key = mta.pad_key
        self.mta_init_method = mta.init_method

    def forward(self, xq, xk, xv, mask=None, chunk_start_ids=None):
        assert chunk_start_ids is None, "MTAAttentionTriton does not support chunked attention"
        if self.use_mask:
            raise NotImplementedError("explicit masks (use_mask=True) are not implemented; the causal flag is")
        if self.training and self.dropout > 0.0:
            raise NotImplementedError("dropout on the attention weights is not implemented: use eval() or dropout=0")
        if not self.causal:
            raise NotImplementedError("MTAAttentionTriton without a mask requires causal=True, as in the reference's benchmarks")
        if self.fused:
            out = ops.mta_fused_fwd(xq, xk, xv, self.mta_conv_triton.weight, self.wpsm_triton.weight,
                                    self.mta_conv_after_sm_triton.weight, self.wposm_triton.weight, causal=True)
            return out.transpose(1, 2)
        head_dim = xq.size(-1)
        scores = ops.qk_scores_fwd(xq, xk, head_dim ** -0.5, causal=True)
        scores = self.mta_conv_triton(scores)
        scores = self.wpsm_triton(scores)
        scores = ops.softmax_fwd(scores, causal=True)
        scores = self.mta_conv_after_sm_triton(scores)
        scores = self.wposm_triton(scores)
        output = ops.pv_fwd(scores, xv, causal=True)
        return output.transpose(1, 2)

    def forward_host(self, xq, xk, xv, out=None, chunk_batch: int = 0):
        """forward for HOST tensors (B,H,S,D), ideally page-locked: the library overlaps the transfers with the
        computation chunk by chunk, and the result comes back as a host tensor, (B,S,H,D) view as forward returns."""
        if not self.causal:
            raise NotImplementedError("MTAAttentionTriton without a mask requires causal=True, as in the reference's benchmarks")
        o = ops.mta_fused_fwd_host(xq, xk, xv, self.mta_conv_triton.weight, self.wpsm_triton.weight,
                                   self.mta_conv_after_sm_triton.weight, self.wposm_triton.weight, causal=True, out=out,
                                   chunk_batch=chunk_batch)
        return o.transpose(1, 2)

    def reset_mta_parameters(self, init_std=None):
        """Initialise as the reference does (mta_attention_triton.py:129-145): conv kernels by
        `mta.init_method`, both head mixes to the identity."""
        init_std = init_std or (self.mta.dim ** (-0.5))
        self._init_conv_kernel(self.mta_conv_triton.weight, init_std)
        self._init_conv_kernel(self.mta_conv_after_sm_triton.weight, init_std)
        torch.nn.init.eye_(self.wpsm_triton.weight)
        torch.nn.init.eye_(self.wposm_triton.weight)

    def _init_conv_kernel(self, kernel, init_std):
        method = self.mta_init_method
        with torch.no_grad():
            if method == "uniform":
                kernel.uniform_(-1.0, 1.0)
            elif method == "normal":
                std = 0.3
                torch.nn.init.trunc_normal_(kernel, mean=0.0, std=std, a=-3 * std, b=3 * std)
            elif method == "diagonal":
                _, A, Bk = kernel.shape
                d = (Bk + 1) // 2 - A
                ones = torch.ones_like(kernel)
                kernel.copy_(torch.triu(torch.tril(ones, diagonal=d), diagonal=d))
            elif method == "identity":
                assert self.pad_key == "both"
                kernel.zero_()
                kernel[:, -1, kernel.shape[2] // 2] = 1.0   # the tap on the current query and key
            elif method == "const":
                kernel.fill_(0.3)
            else:
                raise ValueError(f"Unsupported mta_init_method: {method}")

    def copy_mta_parameters(self, mta_attention):
        """Copy the four weights from a module with the PyTorch oracle's parameter names
        (mta_kernel (H,1,cq,ck), mta_kernel_after_sm, wpsm.weight, wposm.weight)."""
        with torch.no_grad():
            if hasattr(mta_attention, "mta_kernel"):
                self.mta_conv_triton.weight.copy_(mta_attention.mta_kernel.data.squeeze(1))
            if hasattr(mta_attention, "mta_kernel_after_sm"):
                self.mta_conv_after_sm_triton.weight.copy_(mta_attention.mta_kernel_after_sm.data.squeeze(1))
            if hasattr(mta_attention, "wpsm"):
                self.wpsm_triton.weight.copy_(mta_attention.wpsm.weight.data)
            if hasattr(mta_attention, "wposm"):
                self.wposm_triton.weight.copy_(mta_attention.wposm.weight.data)
