"""Loads the reference's own modules from oracle/_ref/ (see make_ref.py) and builds its models on the inputs of
multitokenatention_triton_b200.synthetic.  Benchmark and test infrastructure: the CPU baseline and the "kernel to beat"
GPU timings of bench.py come through here; nothing in the package imports it.

Two shims, neither of which edits a reference file: MTAAttention.forward asks for a tensor on device "cuda"
(mta_attention_pytorch.py:63-65), which is redirected to the inputs' device while a CPU forward runs, and the module
weights are assigned directly instead of through reset_mta_parameters (which calls .cuda(), :176).
"""
from __future__ import annotations

import contextlib
import importlib
import os
import sys
import types

import torch

REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def available() -> bool:
    return os.path.isfile(os.path.join(REF_DIR, "mta_attention_pytorch.py"))


def module(name: str):
    """Imports a reference module by its file name without the extension."""
    if not available():
        raise FileNotFoundError(f"{REF_DIR} is empty: run `python oracle/make_ref.py <reference checkout>` first")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    return importlib.import_module(name)


@contextlib.contextmanager
def tensors_on(device: torch.device):
    """While active, torch.tensor(..., device="cuda") creates its tensor on `device` instead."""
    real = torch.tensor

    def tensor(*a, **kw):
        if kw.get("device") == "cuda":
            kw["device"] = device
        return real(*a, **kw)

    torch.tensor = tensor
    try:
        yield
    finally:
        torch.tensor = real


def mta_config(wl) -> types.SimpleNamespace:
    return types.SimpleNamespace(use_mta=True, query_kernel_size=wl.cq, key_kernel_size=wl.ck,
                                 after_sm_query_kernel_size=wl.cq2, after_sm_key_kernel_size=wl.ck2,
                                 pre_sm_linear_head=True, post_sm_linear_head=True, pad_key="both",
                                 init_method="identity", dim=wl.H * wl.D)


def pytorch_mta(wl, weights, device, dtype):
    """The reference's MTAAttention (mta_attention_pytorch.py:5-83) with the four weights set."""
    m = module("mta_attention_pytorch").MTAAttention(wl.H, mta_config(wl), 0.0)
    with torch.no_grad():
        m.mta_kernel.copy_(weights["w1"].float().unsqueeze(1))
        m.wpsm.weight.copy_(weights["W1"].float())
        m.mta_kernel_after_sm.copy_(weights["w2"].float().unsqueeze(1))
        m.wposm.weight.copy_(weights["W2"].float())
    return m.to(device).to(dtype).eval()


def triton_mta(wl, weights, device, dtype):
    """The reference's MTAAttentionTriton (mta_attention_triton.py:8-92) with the four weights set."""
    m = module("mta_attention_triton").MTAAttentionTriton(wl.H, mta_config(wl), 0.0, causal=True)
    m = m.to(device).to(dtype).eval()
    with torch.no_grad():
        m.mta_conv_triton.weight.copy_(weights["w1"])
        m.wpsm_triton.weight.copy_(weights["W1"])
        m.mta_conv_after_sm_triton.weight.copy_(weights["w2"])
        m.wposm_triton.weight.copy_(weights["W2"])
    return m


def cpu_forward(model, q, k, v):
    """One forward of the reference's PyTorch module on host tensors."""
    with torch.no_grad(), tensors_on(q.device):
        return model(q, k, v, None, None)
