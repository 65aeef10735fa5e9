"""Dropout on the attention weights inside the forward (F.dropout(scores, p, training) before the product with V,
mta_attention_triton.py:87): the keep mask is a function of (seed, plane, query, key) built on Philox4x32-10.

CPU part: the numpy restatement against the published known-answer vectors of Philox4x32-10 (Random123's kat_vectors)
and its statistics.  GPU part: the library's forward against the oracle composed with the same mask."""
import numpy as np
import pytest
import torch

from oracle import mta_oracle as orc
from util import assert_parity, npf


def test_philox_known_answers():
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0), (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for ctr, key, want in kat:
        got = orc.philox4x32_10(*ctr, *key)
        assert tuple(int(x) for x in got) == want


def test_keep_mask_statistics_and_determinism():
    m = orc.dropout_keep_mask(987654321012345, 5, 203, 0.25)
    assert m.shape == (5, 203, 203)
    assert abs(m.mean() - 0.75) < 0.01
    assert np.array_equal(m, orc.dropout_keep_mask(987654321012345, 5, 203, 0.25))
    assert not np.array_equal(m, orc.dropout_keep_mask(987654321012346, 5, 203, 0.25))
    assert orc.dropout_keep_mask(1, 2, 16, 0.0).all()
    # a mask for fewer planes / rows is a corner of the larger one: decisions depend on the position only
    assert np.array_equal(orc.dropout_keep_mask(7, 2, 64, 0.5)[:, :40, :40], orc.dropout_keep_mask(7, 2, 40, 0.5))


CASES = [("bf16_tc", 2, 4, 136, 64, 3, 5, torch.bfloat16, 0.3), ("f16_tc", 1, 16, 200, 128, 6, 11, torch.float16, 0.1),
         ("f32_cores", 2, 3, 65, 16, 3, 5, torch.float32, 0.5), ("bf16_ragged_cores", 1, 2, 77, 32, 2, 3, torch.bfloat16, 0.2)]


@pytest.mark.gpu
@pytest.mark.parametrize("name,B,H,S,D,cq,ck,dtype,p", CASES)
def test_forward_with_dropout_against_the_oracle(name, B, H, S, D, cq, ck, dtype, p):
    from multitokenatention_triton_b200 import _lib, ops
    from multitokenatention_triton_b200.synthetic import MTAWorkload, make_mta_inputs
    wl = MTAWorkload(name, B, H, S, D, cq, ck, 3, 3, dtype, seed=300 + S, random_post_conv=True)
    inp = make_mta_inputs(wl)
    d = [inp[k].to("cuda") for k in ("q", "k", "v", "w1", "W1", "w2", "W2")]
    seed = 0x1234567890ABCDEF + S
    out = ops.mta_fused_fwd(*d, True, dropout_p=p, dropout_seed=seed)
    _lib.device_status()
    ref = orc.mta_fwd_dropout(*[npf(inp[k]) for k in ("q", "k", "v", "w1", "W1", "w2", "W2")], p, seed)
    assert_parity(npf(out), ref, dtype, name)
    plain = ops.mta_fused_fwd(*d, True)
    assert not torch.equal(out, plain)
    assert torch.equal(ops.mta_fused_fwd(*d, True, dropout_p=0.0, dropout_seed=seed), plain)
    assert torch.equal(ops.mta_fused_fwd(*d, True, dropout_p=p, dropout_seed=seed), out), "same seed, same result"
    part = torch.zeros_like(out)
    ops.mta_fused_fwd(*d, True, rows=(S // 3, S - 5), out=part, dropout_p=p, dropout_seed=seed)
    assert torch.equal(part[:, :, S // 3:S - 5], out[:, :, S // 3:S - 5]), "the mask does not depend on the row range"


@pytest.mark.gpu
def test_module_in_training_mode_drops_inside_the_kernel():
    import types
    from multitokenatention_triton_b200 import MTAAttentionTriton, _lib
    from multitokenatention_triton_b200.synthetic import MTAWorkload, make_mta_inputs
    wl = MTAWorkload("drop_module", 1, 8, 128, 64, 3, 5, 3, 3, torch.bfloat16, seed=77, random_post_conv=True)
    inp = make_mta_inputs(wl)
    cfg = types.SimpleNamespace(use_mta=True, query_kernel_size=3, key_kernel_size=5, pre_sm_linear_head=True,
                                pad_key="both", init_method="identity", dim=512)
    m = MTAAttentionTriton(8, cfg, dropout=0.4, causal=True).to("cuda").to(torch.bfloat16)
    with torch.no_grad():
        m.mta_conv_triton.weight.copy_(inp["w1"]); m.wpsm_triton.weight.copy_(inp["W1"])
        m.mta_conv_after_sm_triton.weight.copy_(inp["w2"]); m.wposm_triton.weight.copy_(inp["W2"])
        q, k, v = (inp[n].to("cuda") for n in ("q", "k", "v"))
        m.train()
        _lib.reset_launch_count()
        torch.manual_seed(5)
        a = m(q, k, v)
        assert _lib.launch_count() == 5, "the fused forward, not the stage-by-stage path"
        torch.manual_seed(5)
        b = m(q, k, v)
        c = m(q, k, v)
        m.eval()
        e = m(q, k, v)
    assert torch.equal(a, b) and not torch.equal(a, c) and not torch.equal(a, e)
    # E[dropout(x)] = x: the mean over many seeds approaches the eval output
    m.train()
    with torch.no_grad():
        acc = sum(m(q, k, v).float() for _ in range(64)) / 64
    assert (acc - e.float()).abs().mean() < 0.12 * e.float().abs().mean()
