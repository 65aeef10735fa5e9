"""Seeded synthetic inputs for the MTA forward path.

One recipe serves the parity tests, the golden-vector generator and the benchmark, so that the CPU
checker and the GPU see bit-identical values: everything is drawn in float32 on the CPU from one
`torch.Generator`, in a fixed order, then rounded to the run dtype.

Draw order: Q, K, V (B,H,S,D) ~ N(0,1); pre-softmax conv (H,cq,ck) ~ N(0, conv_var) with 1.0 added
at the identity tap [:, cq-1, ck//2] (the tap aligned with the current query and key, as in the
reference's "identity" initialisation, mta_attention_pytorch.py:176-178); pre-softmax head mix
eye(H) + sqrt(mix_var) * randn(H,H); post-softmax conv (H,cq2,ck2): identity tap only, or random
like the first when `random_post_conv`; post-softmax head mix, an independent draw.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch


@dataclass(frozen=True)
class MTAWorkload:
    name: str
    B: int
    H: int
    S: int
    D: int
    cq: int
    ck: int
    cq2: int = 3
    ck2: int = 3
    dtype: torch.dtype = torch.bfloat16
    seed: int = 0
    conv_var: Optional[float] = None      # default 1/(cq*ck)
    mix_var: float = 0.02
    identity_tap: bool = True
    random_post_conv: bool = False

    @property
    def tokens(self) -> int:
        return self.B * self.S

    def lower_elements(self) -> int:
        """Score-plane entries with key <= query, over all batches and heads."""
        return self.B * self.H * (self.S * (self.S + 1) // 2)

    def algorithmic_flops(self) -> int:
        """Each stage counted once per lower-triangle entry: QK^T 2D, conv1 2*cq*ck, mix 2H,
        conv2 2*cq2*ck2, mix 2H, PV 2D."""
        per = 2 * self.D + 2 * self.cq * self.ck + 2 * self.H + 2 * self.cq2 * self.ck2 + 2 * self.H + 2 * self.D
        return per * self.lower_elements()


# The five configurations the headline metric and the parity suite are defined on.
WORKLOADS: Dict[str, MTAWorkload] = {
    "c1": MTAWorkload("c1", 2, 8, 256, 64, 3, 5, dtype=torch.float32, seed=0, conv_var=1.0 / 15, mix_var=0.01),
    "c1b": MTAWorkload("c1b", 2, 8, 256, 64, 3, 5, dtype=torch.float32, seed=0, conv_var=1.0 / 15, mix_var=0.01,
                       random_post_conv=True),
    "c4": MTAWorkload("c4", 8, 16, 4096, 128, 6, 11, dtype=torch.bfloat16, seed=3, conv_var=1.0 / 66),
    "c4b": MTAWorkload("c4b", 8, 16, 4096, 128, 6, 11, dtype=torch.bfloat16, seed=3, conv_var=1.0 / 66,
                       random_post_conv=True),
    "c5": MTAWorkload("c5", 8, 32, 8192, 128, 6, 11, dtype=torch.bfloat16, seed=4, conv_var=1.0 / 66),
}


def _conv_weight(g: torch.Generator, H: int, r: int, s: int, var: float, tap: bool, random: bool) -> torch.Tensor:
    w = torch.randn(H, r, s, generator=g) * (var ** 0.5) if random else torch.zeros(H, r, s)
    if tap:
        w[:, r - 1, s // 2] += 1.0
    return w


def make_mta_inputs(wl: MTAWorkload, batch_slice: Optional[slice] = None) -> Dict[str, torch.Tensor]:
    """CPU tensors in wl.dtype: q,k,v (B,H,S,D), w1 (H,cq,ck), W1 (H,H), w2 (H,cq2,ck2), W2 (H,H).

    `batch_slice` keeps only some batch elements of q,k,v; the generator still advances through
    the others, so the kept elements equal those of the full draw.
    """
    g = torch.Generator(device="cpu").manual_seed(wl.seed)
    shape = (wl.B, wl.H, wl.S, wl.D)
    keep = range(wl.B) if batch_slice is None else range(*batch_slice.indices(wl.B))
    qkv = []
    for _ in range(3):  # one draw per batch element, so a slice equals the slice of the full tensor
        parts = []
        for b in range(wl.B):
            t = torch.randn(shape[1:], generator=g)
            if b in keep:
                parts.append(t.to(wl.dtype))
        qkv.append(torch.stack(parts))
    var = wl.conv_var if wl.conv_var is not None else 1.0 / (wl.cq * wl.ck)
    w1 = _conv_weight(g, wl.H, wl.cq, wl.ck, var, wl.identity_tap, True)
    W1 = torch.eye(wl.H) + (wl.mix_var ** 0.5) * torch.randn(wl.H, wl.H, generator=g)
    w2 = _conv_weight(g, wl.H, wl.cq2, wl.ck2, 1.0 / (wl.cq2 * wl.ck2), True, wl.random_post_conv)
    W2 = torch.eye(wl.H) + (wl.mix_var ** 0.5) * torch.randn(wl.H, wl.H, generator=g)
    out = {"q": qkv[0], "k": qkv[1], "v": qkv[2], "w1": w1, "W1": W1, "w2": w2, "W2": W2}
    return {k: t.to(wl.dtype) for k, t in out.items()}


def make_conv_inputs(N: int, C: int, S: int, D: int, R: int, Sk: int, dtype: torch.dtype, seed: int,
                     zero_upper: bool = False) -> Dict[str, torch.Tensor]:
    """Pre-softmax score plane x = Q K^T / sqrt(D) (N,C,S,S) and a conv weight (C,R,Sk) ~ N(0, 1/(R*Sk)).
    The upper triangle is left as computed unless `zero_upper`: the conv must ignore it."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(N, C, S, D, generator=g)
    k = torch.randn(N, C, S, D, generator=g)
    w = torch.randn(C, R, Sk, generator=g) * (1.0 / (R * Sk)) ** 0.5
    x = torch.matmul(q, k.transpose(2, 3)) / (D ** 0.5)
    if zero_upper:
        x = torch.tril(x)
    return {"x": x.to(dtype), "w": w.to(dtype)}


def make_head_linear_inputs(N: int, C: int, S: int, dtype: torch.dtype, seed: int,
                            mix_var: float = 0.02) -> Dict[str, torch.Tensor]:
    """Post-softmax probabilities (N,C,S,S): causal rows summing to 1, zero above the diagonal; weight
    (C,C) = eye + N(0, mix_var)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    W = torch.eye(C) + (mix_var ** 0.5) * torch.randn(C, C, generator=g)
    x = torch.empty(N, C, S, S)
    mask = torch.triu(torch.full((S, S), float("-inf")), diagonal=1)
    for n in range(N):  # plane by plane: bounds the float32 temporaries at large S
        logits = torch.randn(C, S, S, generator=g) + mask
        x[n] = torch.softmax(logits, dim=-1)
    return {"x": x.to(dtype), "W": W.to(dtype)}


def make_upstream_grad(shape, dtype: torch.dtype, seed: int) -> torch.Tensor:
    """Seeded upstream gradient for the backward checks: N(0,1) drawn in float32 on the CPU, cast to `dtype`."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype)


def make_mta_weights(wl: MTAWorkload) -> Dict[str, torch.Tensor]:
    """The four weights alone (w1, W1, w2, W2 in wl.dtype), drawn from their own generator so that they do not depend
    on B, S or D: for runs whose q, k, v are drawn elsewhere (on the device, shard by shard)."""
    g = torch.Generator(device="cpu").manual_seed(wl.seed + 7919)
    var = wl.conv_var if wl.conv_var is not None else 1.0 / (wl.cq * wl.ck)
    w1 = _conv_weight(g, wl.H, wl.cq, wl.ck, var, wl.identity_tap, True)
    W1 = torch.eye(wl.H) + (wl.mix_var ** 0.5) * torch.randn(wl.H, wl.H, generator=g)
    w2 = _conv_weight(g, wl.H, wl.cq2, wl.ck2, 1.0 / (wl.cq2 * wl.ck2), True, wl.random_post_conv)
    W2 = torch.eye(wl.H) + (wl.mix_var ** 0.5) * torch.randn(wl.H, wl.H, generator=g)
    return {k: t.to(wl.dtype) for k, t in {"w1": w1, "W1": W1, "w2": w2, "W2": W2}.items()}


def device_qkv(wl: MTAWorkload, b: int, device) -> Dict[str, torch.Tensor]:
    """q, k, v of batch element b, (1,H,S,D) in wl.dtype, drawn on `device` from a generator seeded by (wl.seed, b):
    any rank can draw any batch element without drawing the others (not the values of make_mta_inputs)."""
    g = torch.Generator(device=device).manual_seed(wl.seed * 1000003 + b)
    return {n: torch.randn(1, wl.H, wl.S, wl.D, device=device, generator=g).to(wl.dtype) for n in ("q", "k", "v")}
