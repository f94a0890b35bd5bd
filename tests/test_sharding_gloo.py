"""Multi-rank host logic on CPU (gloo, world size 2): unit partitioning and the no-collective claim."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import AttnCase, attention_fwd_bwd_blockwise, make_inputs
from oregon_gpt_oss_patching_b200.sharding import group_range, partition_units, shard_by_group


def test_partition_covers_every_unit_once():
    for B, Hkv, world in [(4, 8, 1), (4, 8, 2), (2, 8, 8), (8, 8, 4), (3, 5, 2), (2, 2, 8), (1, 8, 3)]:
        parts = partition_units(B, Hkv, world)
        flat = [u for r in parts for u in r]
        assert sorted(flat) == sorted((b, g) for b in range(B) for g in range(Hkv))
        assert max(len(r) for r in parts) - min(len(r) for r in parts) <= max(B, 1)
        if world <= Hkv:  # whole groups per rank: dSinks of a head is complete on its owner
            for r, units in enumerate(parts):
                g0, g1 = group_range(Hkv, r, world)
                assert {g for _, g in units} == set(range(g0, g1))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = AttnCase("t", B=2, S=96, Hq=8, Hkv=4, window=32, seed=3)
        q, k, v, do, sinks = make_inputs(case)  # every rank generates the same seeded inputs
        (qs, ks, vs, dos, ss), (g0, g1) = shard_by_group(q, k, v, do, sinks, rank, world)
        res = attention_fwd_bwd_blockwise(qs, ks, vs, ss, dos, case.scale, case.window)
        # the only cross-rank traffic a benchmark needs: the max of the ranks' times
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[rank] = {"range": (g0, g1), "res": {k_: v_.clone() for k_, v_ in res.items()}, "tmax": t.item()}
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_ranks_reproduce_the_single_rank_result_without_exchanging_data():
    world, port = 2, _free_port()
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    case = AttnCase("t", B=2, S=96, Hq=8, Hkv=4, window=32, seed=3)
    q, k, v, do, sinks = make_inputs(case)
    full = attention_fwd_bwd_blockwise(q, k, v, sinks, do, case.scale, case.window)
    G = 2
    for rank in range(world):
        g0, g1 = out[rank]["range"]
        r = out[rank]["res"]
        assert out[rank]["tmax"] == 2.0
        assert torch.equal(r["o"], full["o"][:, :, g0 * G:g1 * G])
        assert torch.equal(r["dq"], full["dq"][:, g0 * G:g1 * G])
        assert torch.equal(r["dk"], full["dk"][:, g0:g1]) and torch.equal(r["dv"], full["dv"][:, g0:g1])
        assert torch.equal(r["dsinks"], full["dsinks"][g0 * G:g1 * G])   # complete on the owner, no reduction
