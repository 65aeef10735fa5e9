"""Functional front end of the CUDA library: one function per C-ABI entry point.

Every function takes contiguous CUDA tensors, allocates its output (and scratch) with PyTorch and
enqueues the kernels on PyTorch's current stream.  Nothing here computes on the CPU.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import MTALibraryError, check, dtype_code, lib, stream_ptr


def _cuda_contig(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_cuda:
        raise MTALibraryError(f"{name} must be a CUDA tensor: this package has no CPU path")
    return t if t.is_contiguous() else t.contiguous()


def _weight(w: torch.Tensor, like: torch.Tensor, name: str) -> torch.Tensor:
    w = _cuda_contig(w.detach(), name)
    if w.dtype not in (torch.float32, like.dtype):
        w = w.to(like.dtype)
    return w


def conv2d_fwd(x: torch.Tensor, weight: torch.Tensor, causal: bool) -> torch.Tensor:
    """Depthwise causal conv: x (N,C,H,W), weight (C,R,S) -> (N,C,H,W)."""
    x = _cuda_contig(x, "input")
    if x.dim() != 4 or weight.dim() != 3:
        raise MTALibraryError(f"conv2d: expected input (N,C,H,W) and weight (C,R,S), got {tuple(x.shape)} and {tuple(weight.shape)}")
    N, C, H, W = x.shape
    Cw, R, S = weight.shape
    assert C == Cw, "This implementation assumes depthwise convolution (C_in == C_out)"
    w = _weight(weight, x, "weight")
    y = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(lib().mta_conv2d_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), N, C, H, W, R, S, int(bool(causal)),
                                   dtype_code(x), dtype_code(w), stream_ptr(x.device)), "mta_conv2d_fwd")
    return y


def head_linear_fwd(x: torch.Tensor, weight: torch.Tensor, causal: bool = True, output_value: float = 0.0) -> torch.Tensor:
    """Head mix: x (N,C,P,Q), weight (C,C) -> (N,C,P,Q); entries with q > p become output_value when causal."""
    x = _cuda_contig(x, "input")
    if x.dim() != 4:
        raise MTALibraryError(f"head_linear: expected input (N,C,P,Q), got {tuple(x.shape)}")
    N, C, P, Q = x.shape
    L = weight.shape[0]
    assert weight.shape == (L, L), f"Weight must be square matrix, got {weight.shape}"
    assert C == L, f"Channel dimension {C} must match weight dimension {L}"
    w = _weight(weight, x, "weight")
    y = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(lib().mta_head_linear_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), N, C, P, Q, int(bool(causal)),
                                        float(output_value), dtype_code(x), dtype_code(w), stream_ptr(x.device)),
              "mta_head_linear_fwd")
    return y


def conv2d_bwd_input(grad_output: torch.Tensor, weight: torch.Tensor, causal: bool) -> torch.Tensor:
    """Gradient of conv2d_fwd with respect to its input: (N,C,H,W), zeros above the diagonal when causal."""
    g = _cuda_contig(grad_output, "grad_output")
    N, C, H, W = g.shape
    Cw, R, S = weight.shape
    assert C == Cw, "This implementation assumes depthwise convolution (C_in == C_out)"
    w = _weight(weight, g, "weight")
    dx = torch.empty_like(g)
    with torch.cuda.device(g.device):
        check(lib().mta_conv2d_bwd_input(g.data_ptr(), w.data_ptr(), dx.data_ptr(), N, C, H, W, R, S, int(bool(causal)),
                                         dtype_code(g), dtype_code(w), stream_ptr(g.device)), "mta_conv2d_bwd_input")
    return dx


def conv2d_bwd_weight(x: torch.Tensor, grad_output: torch.Tensor, kernel_size: Tuple[int, int], causal: bool) -> torch.Tensor:
    """Gradient of conv2d_fwd with respect to its weight: (C,R,S) float32."""
    x, g = _cuda_contig(x, "input"), _cuda_contig(grad_output, "grad_output")
    assert x.shape == g.shape and x.dtype == g.dtype
    N, C, H, W = x.shape
    R, S = kernel_size
    dw = torch.empty(C, R, S, device=x.device, dtype=torch.float32)
    L = lib()
    nbytes = L.mta_conv2d_bwd_weight_workspace_bytes(N, C, H, W, R, S)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(L.mta_conv2d_bwd_weight(x.data_ptr(), g.data_ptr(), dw.data_ptr(), ws.data_ptr(), ws.numel(), N, C, H, W, R, S,
                                      int(bool(causal)), dtype_code(x), stream_ptr(x.device)), "mta_conv2d_bwd_weight")
    return dw


def head_linear_bwd_input(grad_output: torch.Tensor, weight: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """Gradient of head_linear_fwd with respect to its input: sum_o W[o,h] dy[o]; zeros above the diagonal when causal."""
    g = _cuda_contig(grad_output, "grad_output")
    N, C, P, Q = g.shape
    assert weight.shape == (C, C), f"Weight must be a ({C},{C}) matrix, got {tuple(weight.shape)}"
    w = _weight(weight, g, "weight")
    dx = torch.empty_like(g)
    with torch.cuda.device(g.device):
        check(lib().mta_head_linear_bwd_input(g.data_ptr(), w.data_ptr(), dx.data_ptr(), N, C, P, Q, int(bool(causal)),
                                              dtype_code(g), dtype_code(w), stream_ptr(g.device)), "mta_head_linear_bwd_input")
    return dx


def head_linear_bwd_weight(x: torch.Tensor, grad_output: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """Gradient of head_linear_fwd with respect to its weight: (C,C) float32."""
    x, g = _cuda_contig(x, "input"), _cuda_contig(grad_output, "grad_output")
    assert x.shape == g.shape and x.dtype == g.dtype
    N, C, P, Q = x.shape
    dW = torch.empty(C, C, device=x.device, dtype=torch.float32)
    L = lib()
    nbytes = L.mta_head_linear_bwd_weight_workspace_bytes(C)
    if nbytes == 0:
        raise MTALibraryError(f"head_linear_bwd_weight: C = {C} heads is outside the supported range 1..128")
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(L.mta_head_linear_bwd_weight(x.data_ptr(), g.data_ptr(), dW.data_ptr(), ws.data_ptr(), ws.numel(), N, C, P, Q,
                                           int(bool(causal)), dtype_code(x), stream_ptr(x.device)), "mta_head_linear_bwd_weight")
    return dW


def head_linear_softmax_fwd(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Causal head mix then row softmax of the mixed logits in one pass: x (N,C,P,Q), weight (C,C) -> probabilities
    (N,C,P,Q), zero above the diagonal.  Equals softmax_fwd(head_linear_fwd(x, weight, True, -inf)) up to the order of
    the fp32 sums."""
    x = _cuda_contig(x, "input")
    if x.dim() != 4:
        raise MTALibraryError(f"head_linear_softmax: expected input (N,C,P,Q), got {tuple(x.shape)}")
    N, C, P, Q = x.shape
    assert weight.shape == (C, C), f"Weight must be a ({C},{C}) matrix, got {tuple(weight.shape)}"
    w = _weight(weight, x, "weight")
    y = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(lib().mta_head_linear_softmax_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), N, C, P, Q, dtype_code(x),
                                                dtype_code(w), stream_ptr(x.device)), "mta_head_linear_softmax_fwd")
    return y


def softmax_fwd(x: torch.Tensor, causal: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 row softmax over keys q <= p; zeros above the diagonal.  x (N,C,P,Q)."""
    x = _cuda_contig(x, "input")
    N, C, P, Q = x.shape
    y = torch.empty_like(x) if out is None else out
    with torch.cuda.device(x.device):
        check(lib().mta_softmax_fwd(x.data_ptr(), y.data_ptr(), N, C, P, Q, int(bool(causal)), dtype_code(x),
                                    stream_ptr(x.device)), "mta_softmax_fwd")
    return y


def qk_scores_fwd(q: torch.Tensor, k: torch.Tensor, scale: float, causal: bool = True,
                  round_like_reference: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(B,H,S,S) scores Q K^T * scale.  When causal, entries above the diagonal are zero."""
    q, k = _cuda_contig(q, "q"), _cuda_contig(k, "k")
    B, H, S, D = q.shape
    if out is not None:
        s = out      # entries above the diagonal keep whatever they held
    elif causal:
        s = torch.zeros(B, H, S, S, device=q.device, dtype=q.dtype)
    else:
        s = torch.empty(B, H, S, S, device=q.device, dtype=q.dtype)
    with torch.cuda.device(q.device):
        check(lib().mta_qk_scores_fwd(q.data_ptr(), k.data_ptr(), s.data_ptr(), B, H, S, D, float(scale),
                                      int(round_like_reference and q.dtype != torch.float32), int(bool(causal)),
                                      dtype_code(q), stream_ptr(q.device)), "mta_qk_scores_fwd")
    return s


def pv_fwd(p: torch.Tensor, v: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """(B,H,S,D) = P V, reading only keys k <= q of P when causal."""
    p, v = _cuda_contig(p, "p"), _cuda_contig(v, "v")
    B, H, S, D = v.shape
    o = torch.empty_like(v)
    with torch.cuda.device(v.device):
        check(lib().mta_pv_fwd(p.data_ptr(), v.data_ptr(), o.data_ptr(), B, H, S, D, int(bool(causal)), dtype_code(v),
                               stream_ptr(v.device)), "mta_pv_fwd")
    return o


def conv_attn_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, weight: torch.Tensor, causal: bool,
                  softmax_scale: Optional[float] = None) -> torch.Tensor:
    """softmax(scale * conv(Q K^T)) V with q,k,v (B,H,S,D), weight (H,cq,ck) -> (B,H,S,D)."""
    q, k, v = _cuda_contig(q, "Q"), _cuda_contig(k, "K"), _cuda_contig(v, "V")
    B, H, S, D = q.shape
    Cw, cq, ck = weight.shape
    assert Cw == H
    assert k.shape == q.shape and v.shape == q.shape
    if softmax_scale is None:
        softmax_scale = 1.0 / (D ** 0.5)
    w = _weight(weight, q, "weight")
    o = torch.empty_like(q)
    L = lib()
    nbytes = L.mta_conv_attn_workspace_bytes(B, H, S, D, cq, ck, int(bool(causal)), dtype_code(q), dtype_code(w))
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        check(L.mta_conv_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), w.data_ptr(), o.data_ptr(), ws.data_ptr(),
                                  nbytes, B, H, S, D, cq, ck, int(bool(causal)), float(softmax_scale), dtype_code(q),
                                  dtype_code(w), stream_ptr(q.device)), "mta_conv_attn_fwd")
    return o


def mta_fused_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w1: torch.Tensor, W1: torch.Tensor,
                  w2: torch.Tensor, W2: torch.Tensor, causal: bool = True,
                  rows: Optional[Tuple[int, int]] = None, out: Optional[torch.Tensor] = None,
                  workspace: Optional[torch.Tensor] = None, dropout_p: float = 0.0, dropout_seed: int = 0) -> torch.Tensor:
    """Full four-stage MTA forward; returns (B,H,S,D) contiguous.  With `rows=(r0,r1)` only those query rows
    of the output are written (the rest of a fresh output is zero).  `dropout_p` > 0 drops attention weights before
    the product with V inside the kernel (keep decisions are a function of `dropout_seed` and the weight's position)."""
    q, k, v = _cuda_contig(q, "xq"), _cuda_contig(k, "xk"), _cuda_contig(v, "xv")
    B, H, S, D = q.shape
    assert k.shape == q.shape and v.shape == q.shape
    w1, w2 = _weight(w1, q, "conv weight"), _weight(w2, q, "post-softmax conv weight")
    W1, W2 = _weight(W1, q, "head-mix weight"), _weight(W2, q, "post-softmax head-mix weight")
    wd = {w1.dtype, w2.dtype, W1.dtype, W2.dtype}
    if len(wd) != 1:
        w1, w2, W1, W2 = (t.float() for t in (w1, w2, W1, W2))
    _, cq, ck = w1.shape
    _, cq2, ck2 = w2.shape
    r0, r1 = (0, S) if rows is None else rows
    if out is None:
        out = torch.empty_like(q) if (r0, r1) == (0, S) else torch.zeros_like(q)
    L = lib()
    nbytes = L.mta_workspace_bytes(B, H, S, D, cq, ck, cq2, ck2, r0, r1, dtype_code(q))
    if workspace is None or workspace.numel() < nbytes:
        workspace = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=q.device)
    with torch.cuda.device(q.device):
        check(L.mta_fused_fwd_dropout(q.data_ptr(), k.data_ptr(), v.data_ptr(), w1.data_ptr(), W1.data_ptr(), w2.data_ptr(),
                                      W2.data_ptr(), out.data_ptr(), workspace.data_ptr(), workspace.numel(), B, H, S, D, cq, ck,
                                      cq2, ck2, r0, r1, int(bool(causal)), dtype_code(q), dtype_code(w1), float(dropout_p),
                                      int(dropout_seed) & 0xFFFFFFFFFFFFFFFF, stream_ptr(q.device)),
              "mta_fused_fwd")
    return out


def mta_fused_fwd_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, w1: torch.Tensor, W1: torch.Tensor,
                       w2: torch.Tensor, W2: torch.Tensor, causal: bool = True, out: Optional[torch.Tensor] = None,
                       chunk_batch: int = 0) -> torch.Tensor:
    """Full MTA forward for HOST tensors q, k, v (B,H,S,D), ideally page-locked: copies in, computes and copies out
    chunk by chunk on three streams inside the library, and returns a page-locked host tensor (B,H,S,D) once it is
    complete.  The weights are the module's device tensors; their device is the one that computes."""
    for name, t in (("xq", q), ("xk", k), ("xv", v)):
        if t.is_cuda or not t.is_contiguous():
            raise MTALibraryError(f"{name} must be a contiguous host tensor, got device={t.device} contiguous={t.is_contiguous()}")
    B, H, S, D = q.shape
    assert k.shape == q.shape and v.shape == q.shape and k.dtype == q.dtype and v.dtype == q.dtype
    w1, w2 = _weight(w1, q, "conv weight"), _weight(w2, q, "post-softmax conv weight")
    W1, W2 = _weight(W1, q, "head-mix weight"), _weight(W2, q, "post-softmax head-mix weight")
    if len({w1.dtype, w2.dtype, W1.dtype, W2.dtype}) != 1:
        w1, w2, W1, W2 = (t.float() for t in (w1, w2, W1, W2))
    _, cq, ck = w1.shape
    _, cq2, ck2 = w2.shape
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
    elif out.is_cuda or not out.is_contiguous() or out.shape != q.shape or out.dtype != q.dtype:
        raise MTALibraryError("out must be a contiguous host tensor with the shape and dtype of xq")
    with torch.cuda.device(w1.device):
        torch.cuda.current_stream().synchronize()            # weights written on torch's stream are read on the library's
        check(lib().mta_fused_fwd_host(q.data_ptr(), k.data_ptr(), v.data_ptr(), w1.data_ptr(), W1.data_ptr(), w2.data_ptr(),
                                       W2.data_ptr(), out.data_ptr(), B, H, S, D, cq, ck, cq2, ck2, int(bool(causal)),
                                       dtype_code(q), dtype_code(w1), int(chunk_batch)), "mta_fused_fwd_host")
    return out


def host_pipeline_release(device: Optional[torch.device] = None) -> None:
    """Frees the staging and scratch memory mta_fused_fwd_host keeps on `device` (default: the current one)."""
    with torch.cuda.device(device):
        check(lib().mta_host_pipeline_release(), "mta_host_pipeline_release")
