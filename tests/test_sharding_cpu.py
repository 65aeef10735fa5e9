"""The multi-GPU path on CPU ranks (gloo, world sizes 2 and 4): shard plan, halo recompute and output gather,
with the CPU oracle standing in for the per-rank CUDA forward, against the unsharded oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cases import MTA_CASES
from multitokenatention_triton_b200 import sharding
from multitokenatention_triton_b200.synthetic import make_mta_inputs


def test_plan_batch_split():
    assert sharding.plan_shards(8, 4096, 8) == [(b, b + 1, 0, 4096) for b in range(8)]
    assert sharding.plan_shards(8, 4096, 2) == [(0, 4, 0, 4096), (4, 8, 0, 4096)]
    assert sharding.plan_shards(3, 64, 2) == [(0, 2, 0, 64), (2, 3, 0, 64)]
    assert sharding.plan_shards(1, 64, 1) == [(0, 1, 0, 64)]


def test_plan_row_split_balances_causal_work():
    plan = sharding.plan_shards(2, 8192, 8)          # 4 row blocks per batch element
    assert len(plan) == 8 and plan[0][:2] == (0, 1) and plan[4][:2] == (1, 2)
    blocks = [(r0, r1) for _, _, r0, r1 in plan[:4]]
    assert blocks[0][0] == 0 and blocks[-1][1] == 8192
    assert all(a[1] == b[0] for a, b in zip(blocks, blocks[1:])) and all(r0 % 128 == 0 for r0, _ in blocks)
    work = [(r1 * (r1 + 1) - r0 * (r0 + 1)) / 2 for r0, r1 in blocks]
    assert max(work) / min(work) < 1.15, work
    with pytest.raises(ValueError):
        sharding.plan_shards(3, 64, 4)
    assert sharding.halo_rows(6, 3) == 7


def _oracle_compute(q, k, v, w1, W1, w2, W2, rows):
    from oracle import mta_oracle as orc
    f = lambda t: t.float().numpy()
    r0, r1 = rows
    out = [orc.mta_fwd_rows(f(q), f(k), f(v), f(w1), f(W1), f(w2), f(W2), b, r0, r1) for b in range(q.shape[0])]
    return torch.from_numpy(np.stack(out))


def _worker(rank, world, port, name, result_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        wl = MTA_CASES[name]
        inp = make_mta_inputs(wl)                       # every rank derives the inputs from the seed: no broadcast
        plan = sharding.plan_shards(wl.B, wl.S, world, row_align=16)
        b0, b1, r0, r1 = plan[rank]
        weights = [inp[n] for n in ("w1", "W1", "w2", "W2")]
        local = sharding.local_forward(inp["q"][b0:b1], inp["k"][b0:b1], inp["v"][b0:b1], weights, plan[rank], _oracle_compute)
        assert local.shape == (b1 - b0, wl.H, r1 - r0, wl.D)
        full = sharding.gather_outputs(local, plan, wl.B, wl.S)
        if rank == 0:
            np.save(result_path, full.numpy())
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("name,world", [("tiny_f32", 2), ("ragged_f32", 2), ("ragged_f32", 4), ("c1", 2), ("c1", 4)])
def test_sharded_forward_matches_unsharded(name, world, tmp_path):
    """world <= B splits the batch; world > B splits query rows with the halo recomputed inside each shard."""
    from oracle import mta_oracle as orc
    wl = MTA_CASES[name]
    path = str(tmp_path / "out.npy")
    mp.spawn(_worker, args=(world, _free_port(), name, path), nprocs=world, join=True)
    got = np.load(path)
    inp = make_mta_inputs(wl)
    f = lambda t: t.float().numpy()
    ref = orc.mta_fwd(*[f(inp[n]) for n in ("q", "k", "v", "w1", "W1", "w2", "W2")])
    assert got.shape == ref.shape
    assert np.array_equal(got, ref), "row-range shards must reproduce the unsharded forward bit for bit"
