"""World-size-2 gloo ranks on the CPU: the host logic of the N-sharded linear (row ranges,
gather permutation) and of the expert-parallel MoE (destination sort, count exchange,
all-to-all dispatch / combine, padded routes) with the local compute injected."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = fn(rank, world)
    finally:
        dist.destroy_process_group()


def _run(fn, world=2):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    return dict(ret)


def _dense_case(rank, world):
    from gridbook_b200 import parallel
    torch.manual_seed(0)
    parts, K, M = [8, 4, 4], 16, 3                     # q | k | v style roles
    W = torch.randn(sum(parts), K)
    x = torch.randn(M, K)
    Wl = parallel.shard_rows(W, parts, rank, world)
    lin = parallel.ShardedCBLinear(lambda a: a @ Wl.t(), parts)
    return torch.allclose(lin(x), x @ W.t(), atol=1e-6)


def _moe_case(rank, world):
    from gridbook_b200 import parallel
    E, topk, H, T = 8, 3, 4, 5
    g = torch.Generator().manual_seed(100 + rank)      # every rank brings its own tokens
    x = torch.randn(T, H, generator=g)
    ids = torch.stack([torch.randperm(E, generator=g)[:topk] for _ in range(T)])
    w = torch.rand(T, topk, generator=g)
    ids[1, 2] = -1                                     # padded route
    e_local = E // world

    def local_fn(rows, local_ids):                     # "expert e" scales a row by (e + 1)
        return rows * (local_ids.to(rows.dtype) + 1 + rank * e_local)[:, None]

    def combine(y, weights, T_, k_):
        return (y.reshape(T_, k_, -1) * weights.reshape(T_, k_, 1)).sum(1)

    moe = parallel.ExpertParallelMoE(E, local_fn, combine)
    out = moe(x, w, ids)
    keep = (ids >= 0).to(x.dtype)
    ref = (x[:, None, :] * ((ids.clamp_min(0) + 1).to(x.dtype) * w * keep)[:, :, None]).sum(1)
    return torch.allclose(out, ref, atol=1e-5)


def test_row_ranges_and_permutation():
    from gridbook_b200 import parallel
    assert parallel.shard_row_ranges([8, 4], 1, 2) == [(4, 4), (10, 2)]
    perm = parallel.gather_permutation([8, 4], 2)
    full = torch.arange(12)
    gathered = torch.cat([parallel.shard_rows(full, [8, 4], r, 2) for r in range(2)])
    assert torch.equal(gathered[perm], full)
    with pytest.raises(ValueError):
        parallel.shard_row_ranges([6], 0, 4)
    assert parallel.expert_owner(torch.tensor([0, 3, 4, 7]), 8, 2).tolist() == [0, 0, 1, 1]


def test_sharded_linear_two_ranks():
    assert all(_run(_dense_case).values())


def test_expert_parallel_two_ranks():
    assert all(_run(_moe_case).values())
