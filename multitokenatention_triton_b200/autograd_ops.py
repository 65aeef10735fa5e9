"""Differentiable wrappers of the remaining stages of the stage-by-stage forward.

The conv and the head mix have their own backward kernels (convolution_2d.py, linear_head.py).  The three stages
wrapped here - the scaled scores Q K^T, the causal row softmax and the product with V - run this library's kernels in
the forward; their backward is written with torch operations on the saved tensors (two dense matrix products per
contraction, the usual softmax Jacobian product in float32), which is what autograd does for the reference's
torch.matmul / F.softmax calls (mta_attention_triton.py:68-71, :79, :89).  Entries above the diagonal are constants of
the forward (0), so they receive and propagate no gradient.
"""
import torch

from . import ops


def _tril_(t: torch.Tensor) -> torch.Tensor:
    return torch.tril(t)


class QKScoresFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, scale, causal):
        ctx.save_for_backward(q, k)
        ctx.scale, ctx.causal = scale, causal
        return ops.qk_scores_fwd(q, k, scale, causal=causal)

    @staticmethod
    def backward(ctx, grad_scores):
        q, k = ctx.saved_tensors
        g = (_tril_(grad_scores) if ctx.causal else grad_scores).to(q.dtype) * ctx.scale
        return torch.matmul(g, k), torch.matmul(g.transpose(-1, -2), q), None, None


class CausalSoftmaxFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, scores, causal):
        probs = ops.softmax_fwd(scores, causal=causal)
        ctx.save_for_backward(probs)
        return probs

    @staticmethod
    def backward(ctx, grad_probs):
        (probs,) = ctx.saved_tensors
        p = probs.float()                                   # zero above the diagonal, so those entries drop out
        g = grad_probs.float()
        dot = (g * p).sum(dim=-1, keepdim=True)
        return (p * (g - dot)).to(probs.dtype), None


class PVFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, probs, v, causal):
        ctx.save_for_backward(probs, v)
        ctx.causal = causal
        return ops.pv_fwd(probs, v, causal=causal)

    @staticmethod
    def backward(ctx, grad_out):
        probs, v = ctx.saved_tensors
        grad_out = grad_out.to(v.dtype)
        p = _tril_(probs) if ctx.causal else probs
        grad_probs = torch.matmul(grad_out, v.transpose(-1, -2))
        if ctx.causal:
            grad_probs = _tril_(grad_probs)
        return grad_probs, torch.matmul(p.transpose(-1, -2), grad_out), None
