"""Rank program of tests/test_gpu_peer.py (run under torch.distributed.run, one rank per GPU):
the peer-memory all-gather and expert-parallel layer against the same layers on one GPU."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gridbook_b200 import _native, formats, parallel, synth  # noqa: E402
from gridbook_b200.linear import CBLinear  # noqa: E402
from gridbook_b200.moe import CBMoE  # noqa: E402
from gridbook_b200.peer import PeerExpertParallelMoE, PeerGroup, PeerShardedCBLinear  # noqa: E402
from tests.helpers import assert_close_bf16  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    _native.prepare(local)
    # once with the flag-in-data exchange (pieces fit the staging buffer), once with a staging
    # buffer too small for anything, which sends every exchange down the two-phase path
    for ll_words in (1 << 19, 16):
        peers = PeerGroup(64 << 20, dev, ll_words=ll_words)
        check(peers, rank, world, dev)
        torch.cuda.synchronize()
        peers.close()
    status = _native.device_status(local)
    assert status == 0, f"a bounded wait inside a kernel ran out (status {status})"
    dist.barrier()
    torch.cuda.synchronize()
    print(f"rank {rank}: peer paths ok", flush=True)
    sys.stdout.flush()
    os._exit(0)


def check(peers, rank, world, dev):
    # ---- dense: column shards + peer all-gather == the unsharded layer ----
    fmt = formats.NVFP4_LITERAL
    K, parts = 1024, [512, 256, 256]
    tabs = synth.codebook_tables(fmt, 3)
    gen = torch.Generator(device=dev).manual_seed(11)             # same weights on every rank
    qw = synth.make_packed_device(fmt, sum(parts), K, gen, dev)
    full = CBLinear(fmt, K, parts, [tabs], global_scale=1.0 / 448.0, prefix="full").load(qw, None, dev)
    shard = CBLinear(fmt, K, [p // world for p in parts], [tabs], global_scale=1.0 / 448.0, prefix="shard")
    shard.load(parallel.shard_rows(qw, parts, rank, world).contiguous(), None, dev)
    sharded = PeerShardedCBLinear(shard, parts, peers, max_rows=16)
    for M in (1, 5, 16, 1):
        x = torch.randn(M, K, generator=gen, device=dev).to(torch.bfloat16)
        want = full(x)
        got = sharded(x)
        torch.cuda.synchronize()
        assert_close_bf16(got.float().cpu().numpy(), want.float().cpu().numpy(), f"peer all-gather M={M}")

    # ---- routed layer: expert-parallel over peer memory == all experts on one GPU ----
    # k16v2 runs the grouped kernels, the literal format the per-pair table kernel (small batches)
    for mfmt in (formats.NVFP4_CB_K16, formats.NVFP4_LITERAL):
        E, topk, hidden, inter = 16, 4, 512, 256
        e_local = E // world
        gen = torch.Generator(device=dev).manual_seed(23)
        w13 = synth.make_packed_device(mfmt, E * 2 * inter, hidden, gen, dev).view(E, 2 * inter, -1)
        w2 = synth.make_packed_device(mfmt, E * hidden, inter, gen, dev).view(E, hidden, -1)
        t13, t2 = synth.codebook_tables(mfmt, 5), synth.codebook_tables(mfmt, 6)
        whole = CBMoE(mfmt, mfmt, E, hidden, inter, t13, t2, prefix="whole").load(w13, w2, None, None, dev)
        mine = CBMoE(mfmt, mfmt, e_local, hidden, inter, t13, t2, prefix="mine").load(
            w13[rank * e_local:(rank + 1) * e_local].contiguous(),
            w2[rank * e_local:(rank + 1) * e_local].contiguous(), None, None, dev)
        ep = PeerExpertParallelMoE(E, mine, peers, max_tokens=64, topk=topk, hidden=hidden)
        for T in (1, 5, 40, 64, 5):
            ids, tw = synth.make_routing(T, E, topk, seed=100 * T + rank)        # every rank its own batch
            if T == 5:
                ids[2, 1] = -1                                                    # a padded route
            xg = torch.Generator(device=dev).manual_seed(1000 + 10 * T + rank)
            x = torch.randn(T, hidden, generator=xg, device=dev).to(torch.bfloat16)
            ids_d, tw_d = torch.from_numpy(ids).to(dev), torch.from_numpy(tw).to(dev)
            want = whole(x, tw_d, ids_d)
            got = ep(x, tw_d, ids_d)
            torch.cuda.synchronize()
            if T <= 5:
                assert torch.equal(got, want), (str(mfmt), T, float((got.float() - want.float()).abs().max()))
            else:
                # from 18 routed pairs per expert on, the literal format takes the sorted-rows tensor-core
                # kernel, and the two sides cross that line at different batch sizes (the ranks route
                # 2 T tokens together): same operands, another summation order
                rel = float((got.float() - want.float()).norm() / want.float().norm())
                assert rel <= 1e-2, (str(mfmt), T, rel)


if __name__ == "__main__":
    main()
