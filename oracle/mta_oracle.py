"""ctypes/numpy front end of the C oracle in mta_oracle.c.  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import this
module; the product package never does.  Every function takes and returns float32 numpy arrays
(values already rounded to the run dtype by the caller) and mirrors one entry of the C file, which
cites the reference lines it restates.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmta_oracle.so")
_lib: Optional[ctypes.CDLL] = None

ROUND_NONE, ROUND_BF16, ROUND_FP16 = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile mta_oracle.c with gcc (via the Makefile beside it) and return the .so path."""
    src = os.path.join(_HERE, "mta_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "libmta_oracle.so"])
    return _SO


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        fp = ctypes.POINTER(ctypes.c_float)
        i = ctypes.c_int
        L.mta_oracle_conv2d.argtypes = [fp, fp, fp, i, i, i, i, i, i, i, i]
        L.mta_oracle_conv2d_key_lead.argtypes = [fp, fp, fp, i, i, i, i, i, i, i, i, i]
        L.mta_oracle_head_linear.argtypes = [fp, fp, fp, i, i, i, i, i, ctypes.c_float, i]
        L.mta_oracle_softmax.argtypes = [fp, fp, ctypes.c_long, i, i, i, i]
        dp = ctypes.POINTER(ctypes.c_double)
        L.mta_oracle_conv2d_bwd_input.argtypes = [fp, fp, fp, i, i, i, i, i, i, i, i]
        L.mta_oracle_conv2d_bwd_weight.argtypes = [fp, fp, dp, i, i, i, i, i, i, i]
        L.mta_oracle_head_linear_bwd_input.argtypes = [fp, fp, fp, i, i, i, i, i, i]
        L.mta_oracle_head_linear_bwd_weight.argtypes = [fp, fp, dp, i, i, i, i, i]
        L.mta_oracle_round.argtypes = [fp, fp, ctypes.c_long, i]
        L.mta_oracle_mta_fwd_rows.argtypes = [fp] * 7 + [i] * 13 + [fp]
        L.mta_oracle_conv_attn_fwd_rows.argtypes = [fp] * 4 + [i] * 7 + [ctypes.c_float] + [i] * 4 + [fp]
        L.mta_oracle_set_threads.argtypes = [i]
        for name in ("mta_oracle_conv2d", "mta_oracle_conv2d_key_lead", "mta_oracle_head_linear", "mta_oracle_softmax",
                     "mta_oracle_mta_fwd_rows", "mta_oracle_conv_attn_fwd_rows",
                     "mta_oracle_num_threads", "mta_oracle_abi_version"):
            getattr(L, name).restype = i
        _lib = L
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"oracle {what} failed with status {rc}")


def num_threads() -> int:
    return lib().mta_oracle_num_threads()


def set_threads(n: int) -> None:
    lib().mta_oracle_set_threads(int(n))


def round_to(a, mode: int) -> np.ndarray:
    a = _f32(a)
    out = np.empty_like(a)
    lib().mta_oracle_round(_p(a), _p(out), a.size, mode)
    return out


def key_lead(pad_key: str, S: int) -> int:
    """Left padding of the key axis for a kernel of width S (mta_attention_pytorch.py:91-103)."""
    if pad_key == "both":
        return (S - 1) // 2
    if pad_key == "left":
        return S - 1
    if pad_key == "right":
        return 0
    raise ValueError(f"pad_key {pad_key!r}")


def embed_pad_key(w, pad_key: str) -> np.ndarray:
    """A (C,R,S) kernel applied with pad_key "left" / "right" equals the (C,R,2S-1) kernel with zero taps on the other
    side applied with pad_key "both"; "both" returns w unchanged."""
    w = _f32(w)
    if pad_key == "both":
        return w
    S = w.shape[-1]
    pad = ((0, 0), (0, 0), (0, S - 1)) if pad_key == "left" else ((0, 0), (0, 0), (S - 1, 0))
    assert pad_key in ("left", "right")
    return np.ascontiguousarray(np.pad(w, pad))


def conv2d(x, w, causal: bool, round_mode: int = ROUND_NONE, pad_key: str = "both") -> np.ndarray:
    """Depthwise causal conv on (N,C,H,W) with weight (C,R,S); pad_key places the key window."""
    x, w = _f32(x), _f32(w)
    N, C, H, W = x.shape
    Cw, R, S = w.shape
    assert Cw == C
    y = np.empty_like(x)
    _check(lib().mta_oracle_conv2d_key_lead(_p(x), _p(w), _p(y), N, C, H, W, R, S, int(causal), round_mode,
                                            key_lead(pad_key, S)), "conv2d")
    return y


def head_linear(x, Wm, causal: bool = True, fill: float = 0.0, round_mode: int = ROUND_NONE) -> np.ndarray:
    """Head-mixing linear on (N,C,P,Q) with weight (C,C) in nn.Linear orientation."""
    x, Wm = _f32(x), _f32(Wm)
    N, C, P, Q = x.shape
    assert Wm.shape == (C, C)
    y = np.empty_like(x)
    _check(lib().mta_oracle_head_linear(_p(x), _p(Wm), _p(y), N, C, P, Q, int(causal), float(fill), round_mode),
           "head_linear")
    return y


def _pd(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_double))


def conv2d_bwd_input(dy, w, causal: bool, round_mode: int = ROUND_NONE) -> np.ndarray:
    """Gradient of conv2d with respect to its input; dy (N,C,H,W), w (C,R,S)."""
    dy, w = _f32(dy), _f32(w)
    N, C, H, W = dy.shape
    _, R, S = w.shape
    dx = np.empty_like(dy)
    _check(lib().mta_oracle_conv2d_bwd_input(_p(dy), _p(w), _p(dx), N, C, H, W, R, S, int(causal), round_mode), "conv2d_bwd_input")
    return dx


def conv2d_bwd_weight(x, dy, kernel_size, causal: bool) -> np.ndarray:
    """Gradient of conv2d with respect to its weight, float64 (C,R,S)."""
    x, dy = _f32(x), _f32(dy)
    N, C, H, W = x.shape
    R, S = kernel_size
    dw = np.empty((C, R, S), dtype=np.float64)
    _check(lib().mta_oracle_conv2d_bwd_weight(_p(x), _p(dy), _pd(dw), N, C, H, W, R, S, int(causal)), "conv2d_bwd_weight")
    return dw


def head_linear_bwd_input(dy, Wm, causal: bool = True, round_mode: int = ROUND_NONE) -> np.ndarray:
    dy, Wm = _f32(dy), _f32(Wm)
    N, C, P, Q = dy.shape
    dx = np.empty_like(dy)
    _check(lib().mta_oracle_head_linear_bwd_input(_p(dy), _p(Wm), _p(dx), N, C, P, Q, int(causal), round_mode),
           "head_linear_bwd_input")
    return dx


def head_linear_bwd_weight(x, dy, causal: bool = True) -> np.ndarray:
    x, dy = _f32(x), _f32(dy)
    N, C, P, Q = x.shape
    dW = np.empty((C, C), dtype=np.float64)
    _check(lib().mta_oracle_head_linear_bwd_weight(_p(x), _p(dy), _pd(dW), N, C, P, Q, int(causal)), "head_linear_bwd_weight")
    return dW


def softmax(x, causal: bool = True, round_mode: int = ROUND_NONE) -> np.ndarray:
    x = _f32(x)
    P, Q = x.shape[-2], x.shape[-1]
    y = np.empty_like(x)
    _check(lib().mta_oracle_softmax(_p(x), _p(y), x.size // Q, P, Q, int(causal), round_mode), "softmax")
    return y


def mta_fwd_rows(q, k, v, w1, W1, w2, W2, b: int, r0: int, r1: int, causal: bool = True,
                 round_mode: int = ROUND_NONE, pad_key: str = "both") -> np.ndarray:
    """Full MTA forward for batch element b, rows [r0,r1): returns (H, r1-r0, D).  pad_key "left" / "right" goes in as
    the equivalent zero-extended kernel (embed_pad_key; conv2d above has the direct form to check it against)."""
    q, k, v, w1, W1, w2, W2 = map(_f32, (q, k, v, embed_pad_key(w1, pad_key), W1, embed_pad_key(w2, pad_key), W2))
    B, H, S, D = q.shape
    _, cq, ck = w1.shape
    _, cq2, ck2 = w2.shape
    out = np.empty((H, r1 - r0, D), dtype=np.float32)
    _check(lib().mta_oracle_mta_fwd_rows(_p(q), _p(k), _p(v), _p(w1), _p(W1), _p(w2), _p(W2), B, H, S, D,
                                         cq, ck, cq2, ck2, int(causal), round_mode, b, r0, r1, _p(out)),
           "mta_fwd_rows")
    return out


def mta_fwd(q, k, v, w1, W1, w2, W2, causal: bool = True, round_mode: int = ROUND_NONE,
            pad_key: str = "both") -> np.ndarray:
    """Full MTA forward: returns (B,H,S,D) (the reference returns its (B,S,H,D) transpose view)."""
    q = _f32(q)
    B, H, S, D = q.shape
    return np.stack([mta_fwd_rows(q, k, v, w1, W1, w2, W2, b, 0, S, causal, round_mode, pad_key) for b in range(B)])


def conv_attn_fwd_rows(q, k, v, w, b: int, r0: int, r1: int, causal: bool = True,
                       softmax_scale: Optional[float] = None, round_mode: int = ROUND_NONE) -> np.ndarray:
    q, k, v, w = map(_f32, (q, k, v, w))
    B, H, S, D = q.shape
    _, cq, ck = w.shape
    if softmax_scale is None:
        softmax_scale = 1.0 / (D ** 0.5)
    out = np.empty((H, r1 - r0, D), dtype=np.float32)
    _check(lib().mta_oracle_conv_attn_fwd_rows(_p(q), _p(k), _p(v), _p(w), B, H, S, D, cq, ck, int(causal),
                                               float(softmax_scale), round_mode, b, r0, r1, _p(out)),
           "conv_attn_fwd_rows")
    return out


def conv_attn_fwd(q, k, v, w, causal: bool = True, softmax_scale: Optional[float] = None,
                  round_mode: int = ROUND_NONE) -> np.ndarray:
    q = _f32(q)
    B, H, S, D = q.shape
    return np.stack([conv_attn_fwd_rows(q, k, v, w, b, 0, S, causal, softmax_scale, round_mode) for b in range(B)])


def mta_fwd_masked(q, k, v, w1, W1, w2, W2, mask, causal: bool = True, pad_key: str = "both") -> np.ndarray:
    """The explicit-mask forward (mta_attention_triton.py:63-92 with use_mask=True; with a mask that contains the causal
    part it equals mta_attention_pytorch.py:56-83): mask (B,H,S,S) of 0 / -inf.  Full score planes in float64 / the C
    primitives above; returns (B,H,S,D) float32.  Small sizes only."""
    q, k, v, w1, W1, w2, W2 = map(_f32, (q, k, v, w1, W1, w2, W2))
    mask = np.broadcast_to(_f32(mask), (q.shape[0], q.shape[1], q.shape[2], k.shape[2]))
    dead = np.isneginf(mask)
    scores = (np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(q.shape[-1])).astype(np.float32)
    scores = conv2d(np.where(dead, 0.0, scores).astype(np.float32), w1, causal, pad_key=pad_key)
    scores = head_linear(scores, W1, causal, float("-inf"))
    with np.errstate(invalid="ignore"):
        scores = (scores + mask).astype(np.float32)
    probs = softmax(scores, causal=False)
    probs = conv2d(np.where(dead, 0.0, probs).astype(np.float32), w2, causal, pad_key=pad_key)
    probs = np.where(dead, 0.0, probs).astype(np.float32)
    probs = head_linear(probs, W2, causal, 0.0)
    return np.einsum("bhqk,bhkd->bhqd", probs.astype(np.float64), v.astype(np.float64)).astype(np.float32)


# ---- dropout of the attention weights (host restatement of the library's position-keyed mask) -------------------------
def philox4x32_10(c0, c1, c2, c3, k0, k1):
    """Philox4x32 with 10 rounds (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC11) on
    numpy uint32 arrays; returns the four output words."""
    M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
    W0, W1 = 0x9E3779B9, 0xBB67AE85
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint32) for c in (c0, c1, c2, c3))
    c0, c1, c2, c3 = np.broadcast_arrays(c0, c1, c2, c3)
    k0, k1 = int(k0) & 0xFFFFFFFF, int(k1) & 0xFFFFFFFF
    mask32 = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = M0 * c0.astype(np.uint64)
        p1 = M1 * c2.astype(np.uint64)
        hi0, lo0 = (p0 >> np.uint64(32)).astype(np.uint32), (p0 & mask32).astype(np.uint32)
        hi1, lo1 = (p1 >> np.uint64(32)).astype(np.uint32), (p1 & mask32).astype(np.uint32)
        c0, c1, c2, c3 = hi1 ^ c1 ^ np.uint32(k0), lo1, hi0 ^ c3 ^ np.uint32(k1), lo0
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def dropout_keep_mask(seed: int, planes: int, S: int, p: float) -> np.ndarray:
    """(planes, S, S) boolean: weight (plane, query, key) is kept.  One Philox block per 8 consecutive keys, counter
    (key // 8, query, plane, 0), key = the 64-bit seed; key 8c + e takes the e-th 16-bit field of the 128 output bits and is
    kept when the field is below round((1 - p) * 65536) - the function the library's P.V kernels evaluate."""
    thr = int(min(65536.0, max(0.0, np.float32(np.float32(1.0 - np.float32(p)) * np.float32(65536.0)) + np.float32(0.5))))
    chunks = (S + 7) // 8
    c0 = np.arange(chunks, dtype=np.uint32)[None, None, :]
    c1 = np.arange(S, dtype=np.uint32)[None, :, None]
    c2 = np.arange(planes, dtype=np.uint32)[:, None, None]
    out = philox4x32_10(c0, c1, c2, np.uint32(0), seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    fields = np.stack([(out[e >> 1] >> np.uint32(16 * (e & 1))) & np.uint32(0xFFFF) for e in range(8)], axis=-1)   # (planes,S,chunks,8)
    keep = (fields < thr).reshape(planes, S, chunks * 8)[:, :, :S]
    return keep


def mta_fwd_dropout(q, k, v, w1, W1, w2, W2, p: float, seed: int) -> np.ndarray:
    """The causal forward with the reference's dropout on the attention weights (mta_attention_triton.py:87) under the
    mask of dropout_keep_mask; composed from the C primitives, small sizes only.  Returns (B,H,S,D) float32."""
    q, k, v, w1, W1, w2, W2 = map(_f32, (q, k, v, w1, W1, w2, W2))
    B, H, S, D = q.shape
    scores = np.tril(np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(D)).astype(np.float32)
    scores = conv2d(scores, w1, True)
    scores = head_linear(scores, W1, True, float("-inf"))
    probs = softmax(scores, causal=True)
    probs = conv2d(probs, w2, True)
    probs = head_linear(probs, W2, True, 0.0)
    keep = dropout_keep_mask(seed, B * H, S, p).reshape(B, H, S, S)
    probs = np.where(keep, probs * np.float32(1.0 / (1.0 - p)), np.float32(0.0)).astype(np.float32)
    return np.einsum("bhqk,bhkd->bhqd", probs.astype(np.float64), v.astype(np.float64)).astype(np.float32)
