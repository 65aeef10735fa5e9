"""CPU-only checks of the drop-in boundary: the shared library loads, exports every symbol the header
declares, and rejects bad arguments with a status code before touching a device."""
import ctypes
import os
import re

import pytest
import torch

from multitokenatention_triton_b200 import _lib

ROOT = os.path.abspath(os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "mta_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mta_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    syms = header_symbols()
    assert len(syms) >= 12
    for s in syms:
        assert hasattr(L, s), f"{s} is declared in include/mta_b200.h but not exported"
    assert set(_lib.SIGNATURES) == set(syms), "ctypes table and header disagree"
    assert L.mta_abi_version() == 2


def test_bad_arguments_are_rejected_without_a_device():
    L = _lib.lib()
    z = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)
    assert L.mta_conv2d_fwd(z, z, z, 1, 1, 4, 4, 3, 3, 1, 0, 0, z) == 1
    assert b"null" in L.mta_last_error()
    assert L.mta_conv2d_fwd(one, one, one, 1, 1, 4, 4, 3, 3, 1, 7, 0, z) == 1        # dtype code
    assert L.mta_conv2d_fwd(one, one, ctypes.c_void_p(32), 1, 1, 4, 4, 0, 3, 1, 0, 0, z) == 1   # R = 0
    assert L.mta_head_linear_fwd(z, z, z, 1, 4, 4, 4, 1, 0.0, 0, 0, z) == 1
    assert L.mta_head_linear_fwd(one, one, one, 1, 4, 4, 4, 1, 0.0, 0, 0, z) == 1    # in place
    assert L.mta_softmax_fwd(z, z, 1, 1, 4, 4, 1, 0, z) == 1
    assert L.mta_qk_scores_fwd(z, z, z, 1, 1, 4, 8, 1.0, 0, 1, 0, z) == 1
    assert L.mta_pv_fwd(z, z, z, 1, 1, 4, 8, 1, 0, z) == 1
    # even key kernel, bad row range, short workspace
    args = [one] * 9
    assert L.mta_fused_fwd(*args, 1 << 30, 1, 2, 8, 8, 3, 4, 3, 3, 0, 8, 1, 0, 0, z) == 1
    assert b"odd" in L.mta_last_error()
    assert L.mta_fused_fwd(*args, 1 << 30, 1, 2, 8, 8, 3, 3, 3, 3, 4, 9, 1, 0, 0, z) == 1
    assert L.mta_fused_fwd(*args, 16, 1, 2, 8, 8, 3, 3, 3, 3, 0, 8, 1, 0, 0, z) == 1
    assert b"workspace" in L.mta_last_error()
    # empty problems are a no-op
    assert L.mta_conv2d_fwd(z, z, z, 0, 1, 4, 4, 3, 3, 1, 0, 0, z) == 0
    assert L.mta_fused_fwd(*args, 0, 0, 2, 8, 8, 3, 3, 3, 3, 0, 0, 1, 0, 0, z) == 0


def test_workspace_size_formula():
    L = _lib.lib()
    # two score planes of B*H*(rows incl. halo)*S elements, each rounded up to 256 bytes
    n = L.mta_workspace_bytes(2, 4, 64, 32, 6, 11, 3, 3, 0, 64, 1)
    assert n == 2 * 2 * 4 * 64 * 64 * 2
    n = L.mta_workspace_bytes(2, 4, 64, 32, 6, 11, 3, 3, 32, 48, 0)
    r256 = lambda v: (v + 255) // 256 * 256
    assert n == 2 * r256(2 * 4 * (48 - 32 + 7) * 64 * 4)
    # the conv attention: no scratch where the one-kernel path applies, two score planes otherwise
    assert L.mta_conv_attn_workspace_bytes(2, 4, 512, 128, 6, 11, 1, 1, 1) == 0
    assert L.mta_conv_attn_workspace_bytes(2, 4, 512, 128, 6, 11, 1, 0, 0) == 2 * 2 * 4 * 512 * 512 * 4      # float32
    assert L.mta_conv_attn_workspace_bytes(2, 4, 512, 128, 6, 11, 0, 1, 1) == 2 * 2 * 4 * 512 * 512 * 2      # not causal
    assert L.mta_conv_attn_workspace_bytes(2, 4, 512, 128, 6, 19, 1, 1, 1) == 2 * 2 * 4 * 512 * 512 * 2      # 19 taps wide
    assert L.mta_workspace_bytes(2, 4, 64, 32, 6, 11, 3, 3, 32, 70, 0) == 0
    assert L.mta_set_variant(b"nope", 1) == 1 and L.mta_set_variant(b"conv2d", 0) == 0 and L.mta_set_variant(b"mix_softmax", 0) == 0


def test_ops_refuse_cpu_tensors():
    from multitokenatention_triton_b200 import Conv2dTriton, MTAAttentionTriton, TritonLinearHead
    with pytest.raises(_lib.MTALibraryError):
        Conv2dTriton(2, (3, 3), causal=True)(torch.zeros(1, 2, 4, 4))
    with pytest.raises(_lib.MTALibraryError):
        TritonLinearHead(2)(torch.zeros(1, 2, 4, 4))


def test_module_surface_matches_reference_names():
    import types
    from multitokenatention_triton_b200 import MTAAttentionTriton
    cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=6, key_kernel_size=11, pre_sm_linear_head=True,
                                pad_key="both", init_method="identity", dim=512)
    m = MTAAttentionTriton(8, cfg, dropout=0.0, causal=True)
    names = {n for n, _ in m.named_parameters()}
    assert names == {"mta_conv_triton.weight", "wpsm_triton.weight", "mta_conv_after_sm_triton.weight", "wposm_triton.weight"}
    assert m.mta_conv_triton.weight.shape == (8, 6, 11) and m.mta_conv_after_sm_triton.weight.shape == (8, 3, 3)
    m.reset_mta_parameters()
    assert torch.equal(m.wpsm_triton.weight, torch.eye(8))
    w = m.mta_conv_triton.weight
    assert w.sum() == 8 and torch.all(w[:, 5, 5] == 1)
    src = types.SimpleNamespace(mta_kernel=torch.randn(8, 1, 6, 11), mta_kernel_after_sm=torch.randn(8, 1, 3, 3),
                                wpsm=torch.nn.Linear(8, 8, bias=False), wposm=torch.nn.Linear(8, 8, bias=False))
    m.copy_mta_parameters(src)
    assert torch.equal(m.mta_conv_triton.weight.data, src.mta_kernel.squeeze(1))
    assert torch.equal(m.wposm_triton.weight.data, src.wposm.weight.data)
