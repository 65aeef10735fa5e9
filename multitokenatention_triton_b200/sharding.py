"""Sharding of the MTA forward over the GPUs of one box: by batch element first, then by query-row blocks.

The forward has no exchange step.  Batch elements are independent, and inside one batch element a block
of query rows [r0, r1) only needs Q rows [r0 - halo, r1) and K/V rows [0, r1) of the same GPU's copy: the
(cq-1) + (cq2-1) halo rows above the block are recomputed locally (mta_fused_fwd does this for any row range),
all heads stay together because the head mixes couple them.  The only collective is an optional all-gather
of the output shards.

A plan is a list, per rank, of (b0, b1, r0, r1): batch elements [b0, b1) and query rows [r0, r1).
Row blocks are cut where the causal work (proportional to the number of (query, key) pairs) is equal.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence, Tuple

import torch

Shard = Tuple[int, int, int, int]


def plan_shards(B: int, S: int, world: int, row_align: int = 128) -> List[Shard]:
    """One shard per rank.  world <= B: contiguous batch ranges (sizes differ by at most one).  world > B:
    world must be a multiple of B; each batch element is cut into world // B row blocks of equal causal work,
    boundaries rounded to `row_align` (the kernels' tile height)."""
    if world <= 0 or B <= 0 or S <= 0:
        raise ValueError("B, S and world must be positive")
    if world <= B:
        base, extra = divmod(B, world)
        out, b = [], 0
        for r in range(world):
            n = base + (1 if r < extra else 0)
            out.append((b, b + n, 0, S))
            b += n
        return out
    if world % B:
        raise ValueError(f"world size {world} must be a multiple of the batch size {B} to shard query rows")
    parts = world // B
    cuts = [0]
    for i in range(1, parts):
        x = S * math.sqrt(i / parts)                     # rows [0, x) hold i/parts of the causal work
        c = int(round(x / row_align)) * row_align
        cuts.append(min(max(c, cuts[-1]), S))
    cuts.append(S)
    out = []
    for b in range(B):
        for i in range(parts):
            out.append((b, b + 1, cuts[i], cuts[i + 1]))
    return out


def halo_rows(cq: int, cq2: int) -> int:
    """Query rows above a block that the two convs reach back to."""
    return (cq - 1) + (cq2 - 1)


def local_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, weights: Sequence[torch.Tensor], shard: Shard,
                  compute: Optional[Callable] = None) -> torch.Tensor:
    """Runs one shard.  q, k, v hold the batch elements [b0, b1) of the shard (all S rows); returns the
    (b1-b0, H, r1-r0, D) block of output rows.  `compute(q, k, v, w1, W1, w2, W2, rows)` defaults to the CUDA
    forward; tests pass a CPU stand-in to exercise the index arithmetic without a GPU."""
    b0, b1, r0, r1 = shard
    if q.shape[0] != b1 - b0:
        raise ValueError(f"shard covers {b1 - b0} batch elements but q holds {q.shape[0]}")
    if r1 <= r0:
        return q.new_zeros((b1 - b0, q.shape[1], 0, q.shape[3]))
    if compute is None:
        from . import ops
        full = ops.mta_fused_fwd(q, k, v, *weights, causal=True, rows=(r0, r1))
        return full[:, :, r0:r1].contiguous()
    return compute(q, k, v, *weights, (r0, r1))


def gather_outputs(local: torch.Tensor, plan: Sequence[Shard], B: int, S: int, group=None) -> torch.Tensor:
    """All-gathers the shards into the full (B, H, S, D) output on every rank (NCCL over NVLink on GPUs, gloo on
    CPU tensors).  Shards are padded to the largest one because all_gather wants equal sizes."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if world != len(plan):
        raise ValueError(f"plan has {len(plan)} shards but the group has {world} ranks")
    H, D = local.shape[1], local.shape[3]
    nb = max(b1 - b0 for b0, b1, _, _ in plan)
    nr = max(r1 - r0 for _, _, r0, r1 in plan)
    padded = local.new_zeros((nb, H, nr, D))
    padded[: local.shape[0], :, : local.shape[2]] = local
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded, group=group)
    out = local.new_empty((B, H, S, D))
    for (b0, b1, r0, r1), p in zip(plan, pieces):
        out[b0:b1, :, r0:r1] = p[: b1 - b0, :, : r1 - r0]
    return out
