"""The MTA attention module, with the reference's name and interface.

Mirrors MTAAttentionTriton (mta_attention_triton.py:7-201): constructor arguments, sub-module and
parameter names (mta_conv_triton.weight, wpsm_triton.weight, mta_conv_after_sm_triton.weight,
wposm_triton.weight), reset_mta_parameters / copy_mta_parameters, and forward(xq, xk, xv, mask,
chunk_start_ids) returning the (B,S,H,D) transpose view of a (B,H,S,D) tensor.

`fused=True` (default) runs the whole forward through mta_fused_fwd.  `fused=False` runs the reference's
seven steps one by one through the stand-alone entry points, which keeps every 16-bit rounding point of
the reference.  `use_mask=True` runs the reference's explicit-mask path (None, boolean, additive, padding or
(1,1,S,S) masks) stage by stage over full score planes.
"""
import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .autograd_ops import CausalSoftmaxFunction, PVFunction, QKScoresFunction
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

        # the reference's Triton module only takes pad_key "both" (mta_attention_triton.py:171); "left" and "right" are
        # those of its PyTorch module (mta_attention_pytorch.py:91-98)
        pad_key = getattr(mta, "pad_key", "both")
        self.mta_conv_triton = Conv2dTriton(n_heads, kernel_size=(mta.query_kernel_size, mta.key_kernel_size), causal=causal,
                                            pad_key=pad_key)
        self.wpsm_triton = TritonLinearHead(n_heads, causal=causal, output_value=float("-inf"))
        self.mta_conv_after_sm_triton = Conv2dTriton(
            n_heads, kernel_size=(mta.after_sm_query_kernel_size, mta.after_sm_key_kernel_size), causal=causal,
            pad_key=pad_key)
        self.wposm_triton = TritonLinearHead(n_heads, causal=causal)

        self.pad_key = pad_key
        self.mta_init_method = mta.init_method

    def forward(self, xq, xk, xv, mask=None, chunk_start_ids=None):
        assert chunk_start_ids is None, "MTAAttentionTriton does not support chunked attention"
        if self.use_mask:
            return self._forward_with_mask(xq, xk, xv, mask)
        if not self.causal:
            raise NotImplementedError("MTAAttentionTriton without a mask requires causal=True, as in the reference's benchmarks")
        dropping = self.training and self.dropout > 0.0
        if self.fused and not (torch.is_grad_enabled() and any(t.requires_grad for t in (xq, xk, xv, *self.parameters()))):
            # F.dropout(scores, p=self.dropout, training=self.training) (mta_attention_triton.py:87) runs inside the last
            # kernel; its seed is drawn from torch's CPU generator, so torch.manual_seed makes a forward repeatable
            seed = int(torch.randint(0, 2 ** 62, (1,), dtype=torch.int64).item()) if dropping else 0
            out = ops.mta_fused_fwd(xq, xk, xv, self.mta_conv_triton.effective_weight(), self.wpsm_triton.weight,
                                    self.mta_conv_after_sm_triton.effective_weight(), self.wposm_triton.weight, causal=True,
                                    dropout_p=self.dropout if dropping else 0.0, dropout_seed=seed)
            return out.transpose(1, 2)
        # stage by stage; every stage is differentiable (the conv and the head mix through their backward kernels, the
        # scores, the softmax and the product with V through autograd_ops), so this is the path a training step uses
        head_dim = xq.size(-1)
        scores = QKScoresFunction.apply(xq, xk, head_dim ** -0.5, True)
        scores = self.mta_conv_triton(scores)
        scores = self.wpsm_triton(scores)
        scores = CausalSoftmaxFunction.apply(scores, True)
        scores = self.mta_conv_after_sm_triton(scores)
        scores = self.wposm_triton(scores)
        scores = F.dropout(scores, p=self.dropout, training=self.training)      # mta_attention_triton.py:87
        output = PVFunction.apply(scores, xv, True)
        return output.transpose(1, 2)

    def _forward_with_mask(self, xq, xk, xv, mask):
        """The explicit-mask path of the reference (mta_attention_triton.py:63-92 with use_mask=True): full score
        planes, the mask applied around the two convs and before the softmax exactly where the reference applies it.
        The convs, head mixes, softmax and the two contractions are this library's kernels; the mask arithmetic
        (masked_fill, add, where) is elementwise torch."""
        mask = self._update_mask(mask=mask, bsz=xq.size(0), xq=xq, xk_size=xk.size(-2))
        dead = mask == float("-inf")
        head_dim = xq.size(-1)
        scores = ops.qk_scores_fwd(xq, xk, head_dim ** -0.5, causal=False)
        scores = self.mta_conv_triton(scores.masked_fill(dead, 0.0))
        scores = self.wpsm_triton(scores)
        scores = scores + mask
        scores = ops.softmax_fwd(scores, causal=False)
        scores = self.mta_conv_after_sm_triton(scores.masked_fill(dead, 0.0))
        scores = torch.where(dead, torch.zeros((), dtype=scores.dtype, device=scores.device), scores)
        scores = self.wposm_triton(scores)
        scores = F.dropout(scores, p=self.dropout, training=self.training)
        output = ops.pv_fwd(scores, xv, causal=False)
        return output.transpose(1, 2)

    def _update_mask(self, mask, bsz: int, xq, xk_size: int):
        """The reference's mask normalisation (mta_attention_triton.py:106-127): None -> the causal mask; bool -> 0 / -inf;
        a (bsz, keys) padding mask -> broadcast over heads and queries with the causal part added; a (1,1,S,S) mask ->
        repeated over batch and heads.  Returns a (B,H,S,S) tensor of 0 / -inf in the dtype of xq."""
        if not isinstance(mask, torch.Tensor):
            mask = torch.full((xq.size(-2), xk_size), float("-inf"), device=xq.device)
            mask = torch.triu(mask, diagonal=1).type_as(xq)
            mask = mask.repeat(bsz, self.n_heads, 1, 1)
        else:
            if mask.dtype == torch.bool:
                mask = torch.where(mask, 0.0, float("-inf")).to(xq.dtype)
            if mask.dtype != xq.dtype:
                mask = mask.type(xq.dtype)
            if len(mask.shape) == 2:
                assert mask.size(0) == bsz
                # (bsz, keys) -> (bsz, heads, queries, keys); the reference's repeat on the 2-D tensor is only
                # shape-correct for bsz == 1, this is the same mask for that case and the evident intent otherwise
                mask = mask[:, None, None, :].repeat(1, self.n_heads, xq.size(-2), 1)
                mask_i, mask_j = torch.triu_indices(xq.size(-2), xk_size, offset=1)
                mask[:, :, mask_i, mask_j] = float("-inf")
            else:
                if mask.size(0) == 1 and mask.size(1) == 1:
                    mask = mask.repeat(bsz, self.n_heads, 1, 1)
        return mask.to(xq.device)

    def forward_host(self, xq, xk, xv, out=None, chunk_batch: int = 0):
        """forward for HOST tensors (B,H,S,D), ideally page-locked: the library overlaps the transfers with the
        computation chunk by chunk, and the result comes back as a host tensor, (B,S,H,D) view as forward returns."""
        if not self.causal:
            raise NotImplementedError("MTAAttentionTriton without a mask requires causal=True, as in the reference's benchmarks")
        o = ops.mta_fused_fwd_host(xq, xk, xv, self.mta_conv_triton.effective_weight().detach(), self.wpsm_triton.weight,
                                   self.mta_conv_after_sm_triton.effective_weight().detach(), self.wposm_triton.weight,
                                   causal=True, out=out,
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
