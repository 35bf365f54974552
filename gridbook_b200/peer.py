"""Multi-GPU hot path over peer memory (one NVSwitch node, one process per GPU).

The dense all-gather and the expert-parallel dispatch/combine of :mod:`gridbook_b200.parallel`
go through NCCL and, for the routed layer, through a host read of the split sizes.  Here the
same exchanges are plain stores into the peers' buffers from this package's own kernels:

* ``PeerShardedCBLinear``: the local column shard's output is copied into every rank's full
  output row by one launch that also carries the flag exchange on both sides of the copy.
* ``PeerExpertParallelMoE``: the bucketed activations and the routing ids are all-gathered the
  same way, every rank runs the grouped kernels over the pairs routed to ITS experts, and the
  down-projection GEMV stores every output row straight into the buffer of the rank the token
  came from; the home rank's combine waits for the peers' "stores visible" flags in its own launch.  Five to
  seven launches, no host read.

The reference is single-GPU (gridbook/config.py:565-576); nothing here has a counterpart there.
Buffers are shared between the processes by CUDA IPC handles sent through the process group.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _native as nat
from . import kernels
from ._native import NativeKernelUnavailableError


class _RawDeviceMemory:
    """Lets torch alias device memory this package allocated."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerArena:
    """``nbytes`` of zero-filled device memory on every rank, each rank's block mapped into every
    other rank.  ``carve`` hands out the same offsets on every rank as long as every rank makes
    the same calls in the same order."""

    def __init__(self, nbytes: int, device: torch.device, group=None):
        self.lib = nat.load("peer-memory exchange")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > nat.PEER_MAX:
            raise ValueError(f"peer exchange serves up to {nat.PEER_MAX} ranks, got {self.world}")
        self.device = device
        self.nbytes = (int(nbytes) + 255) & ~255
        own = ctypes.c_void_p()
        with torch.cuda.device(device):
            nat.check(self.lib.gb_peer_alloc(self.nbytes, ctypes.byref(own)), self.lib)
            handle = ctypes.create_string_buffer(nat.PEER_HANDLE_BYTES)
            nat.check(self.lib.gb_peer_export(own, handle), self.lib)
            handles = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
            self.ptrs = []
            for r in range(self.world):
                if r == self.rank:
                    self.ptrs.append(own.value)
                    continue
                mapped = ctypes.c_void_p()
                theirs = ctypes.create_string_buffer(bytes(handles[r]), nat.PEER_HANDLE_BYTES)
                nat.check(self.lib.gb_peer_open(theirs, ctypes.byref(mapped)), self.lib)
                self.ptrs.append(mapped.value)
        self._own = own
        self._top = 0
        self._bytes = torch.as_tensor(_RawDeviceMemory(own.value, self.nbytes), device=device)

    def close(self) -> None:
        """Unmaps the peers' blocks and frees this rank's.  Call on every rank, after a barrier
        that guarantees nobody still stores into a block that is about to disappear."""
        if self._own is None:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for r, ptr in enumerate(self.ptrs):
                if r != self.rank and ptr:
                    nat.check(self.lib.gb_peer_close(ctypes.c_void_p(ptr)), self.lib)
            self._bytes = None
            nat.check(self.lib.gb_peer_free(self._own), self.lib)
        self._own, self.ptrs = None, []

    def carve(self, nbytes: int) -> int:
        off = self._top
        self._top = (off + int(nbytes) + 255) & ~255
        if self._top > self.nbytes:
            raise MemoryError(f"peer arena of {self.nbytes} bytes is full ({self._top} wanted)")
        return off

    def tensor(self, offset: int, shape, dtype) -> torch.Tensor:
        """This rank's block at ``offset`` as a tensor (aliases the shared memory)."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self._bytes[offset:offset + nbytes].view(dtype).view(*shape)

    def ptr(self, rank: int, offset: int) -> int:
        return self.ptrs[rank] + offset


class PeerGroup:
    """Arena + flag block + staging buffer: what the exchange launches need."""

    def __init__(self, arena_bytes: int, device: torch.device, group=None, ll_words: int = 1 << 19):
        world = dist.get_world_size(group)
        self.ll_bytes = 2 * world * ll_words * 8          # two halves x one slot per source rank
        self.ll_words = ll_words
        self.arena = PeerArena(arena_bytes + self.ll_bytes + 8192, device, group)
        self.rank, self.world, self.device = self.arena.rank, self.arena.world, device
        flag_off = self.arena.carve(nat.PEER_FLAG_BYTES)
        self.ll_off = self.arena.carve(self.ll_bytes)
        self.native = nat.GbPeerGroup()
        self.native.rank, self.native.world = self.rank, self.world
        self._ll = (ctypes.c_void_p * 8)()
        for r in range(self.world):
            self.native.flags[r] = self.arena.ptr(r, flag_off)
            self._ll[r] = self.arena.ptr(r, self.ll_off)
        dist.barrier(group)          # every rank has mapped every block before the first launch

    def allgather(self, pieces) -> None:
        """``pieces``: (src_ptr, rows, row_bytes, src_pitch, dst_offsets, dst_pitch) with
        ``dst_offsets[s]`` the arena offset at which rank s's piece lands (the same on every
        rank).  Small exchanges go flag-in-data (one one-way trip), large ones as plain peer
        stores between two flag exchanges."""
        lib = self.arena.lib
        words = sum(rows * row_bytes // 4 for _, rows, row_bytes, _, _, _ in pieces)
        if words <= self.ll_words:
            arr = (nat.GbPeerLLPiece * len(pieces))()
            for i, (src, rows, row_bytes, src_pitch, dst_offs, dst_pitch) in enumerate(pieces):
                q = arr[i]
                q.src, q.rows, q.row_bytes, q.src_pitch, q.dst_pitch = src, rows, row_bytes, src_pitch, dst_pitch
                for s in range(self.world):
                    q.dst_local[s] = self.arena.ptr(self.rank, dst_offs[s])
            nat.check(lib.gb_peer_allgather_ll(ctypes.byref(self.native), self._ll, self.ll_bytes, arr,
                                               len(pieces), nat.stream_ptr(self.device)), lib)
            return
        arr = (nat.GbPeerPiece * len(pieces))()
        for i, (src, rows, row_bytes, src_pitch, dst_offs, dst_pitch) in enumerate(pieces):
            q = arr[i]
            q.src, q.rows, q.row_bytes, q.src_pitch, q.dst_pitch = src, rows, row_bytes, src_pitch, dst_pitch
            for r in range(self.world):
                q.dst[r] = self.arena.ptr(r, dst_offs[self.rank])
        nat.check(lib.gb_peer_allgather(ctypes.byref(self.native), arr, len(pieces),
                                        nat.stream_ptr(self.device)), lib)

    def close(self) -> None:
        dist.barrier(self.arena.group)
        self.arena.close()

    def barrier(self) -> None:
        """Returns (on the stream) once every rank's stores enqueued before its own call are
        visible here."""
        lib = self.arena.lib
        nat.check(lib.gb_peer_barrier(ctypes.byref(self.native), nat.stream_ptr(self.device)), lib)


def role_slices(partition_sizes, world: int):
    """Per role of a fused module: (first local column, first global column of rank 0's slice,
    slice width).  Rank s's slice of the role sits at local column ``lcol`` of its shard and at
    global column ``gcol + s * width`` of the full output (an equal slice of every role per rank,
    as :func:`gridbook_b200.parallel.shard_row_ranges` lays the shards out)."""
    roles, lcol, gcol = [], 0, 0
    for n in partition_sizes:
        if n % world:
            raise ValueError(f"role of {n} rows does not divide over {world} ranks")
        per = n // world
        roles.append((lcol, gcol, per))
        lcol += per
        gcol += n
    return roles


class PeerShardedCBLinear(torch.nn.Module):
    """Column-parallel linear whose all-gather is one peer-store launch.  ``local`` maps x[M, K]
    to this rank's [M, N/world] columns, laid out role by role (an equal slice of every role,
    :func:`gridbook_b200.parallel.shard_row_ranges`)."""

    def __init__(self, local, partition_sizes, peers: PeerGroup, max_rows: int = 16):
        super().__init__()
        self.local, self.peers = local, peers
        self.partition_sizes = [int(p) for p in partition_sizes]
        world, rank = peers.world, peers.rank
        for n in self.partition_sizes:
            if n % world:
                raise ValueError(f"role of {n} rows does not divide over {world} ranks")
        self.N = sum(self.partition_sizes)
        self.n_local = self.N // world
        self.max_rows = max_rows
        self.out_off = peers.arena.carve(max_rows * self.N * 2)
        self.roles = role_slices(self.partition_sizes, world)
        self._layout = None
        self._fused_ok = None
        # one activation row: "tab" = the shard's one-launch table kernel, then the flag-in-data
        # all-gather; "fused" = the two-launch table kernel whose second launch sums the K slices
        # and exchanges the shards
        self.single_row = "tab" if getattr(local, "_cb_slots", None) is not None else "fused"
        if len(self.roles) > 4:
            raise ValueError("at most four roles per fused module")

    def _fused(self, x: torch.Tensor):
        """One activation row through a CBLinear shard: the table kernel, then one launch that
        sums the K slices and exchanges the shards.  None when the layer has no such kernel."""
        if self._fused_ok is False:
            return None
        local = self.local
        w = getattr(local, "_cb_weight", None)
        method = getattr(local, "method", None)
        if w is None or method is None or not method.fmt.is_fp4:
            self._fused_ok = False
            return None
        from . import ops
        peers = self.peers
        if self._layout is None:
            lay = nat.GbGatherLayout()
            lay.n_roles = len(self.roles)
            for i, (lc, gc, wd) in enumerate(self.roles):
                lay.lcol[i], lay.gcol0[i], lay.width[i] = lc, gc, wd
            self._layout = lay
        x2 = x.reshape(1, -1).contiguous()
        ws = local._cb_workspace
        nw = w.native()
        lib = peers.arena.lib
        rc = lib.gb_gemv_allgather(ctypes.c_void_p(x2.data_ptr()), ctypes.byref(nw), nat.ACT_FP4_GROUP16,
                                   nat.SCALE_RULE_DIV if ops.ACT_SCALE_RULE == "div" else nat.SCALE_RULE_RECIP,
                                   ctypes.byref(peers.native), peers._ll, peers.ll_bytes, ctypes.byref(self._layout),
                                   ctypes.c_void_p(peers.arena.ptr(peers.rank, self.out_off)),
                                   ctypes.c_void_p(ws.data_ptr()), ws.numel(), nat.stream_ptr(peers.device))
        if rc == nat.EUNSUPPORTED:
            self._fused_ok = False          # same verdict on every rank: the format is the same everywhere
            return None
        nat.check(rc, lib)
        return peers.arena.tensor(self.out_off, (1, self.N), torch.bfloat16)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.numel() == x.shape[-1] and x.dtype is torch.bfloat16 and self.single_row == "fused":
            full = self._fused(x)
            if full is not None:
                return full.reshape(*x.shape[:-1], self.N)
        y = self.local(x)
        lead = y.shape[:-1]
        y2 = y.reshape(-1, self.n_local).contiguous()
        M = y2.shape[0]
        if M > self.max_rows:
            raise ValueError(f"{M} rows exceed the {self.max_rows} this layer reserved peer memory for")
        base = y2.data_ptr()
        world = self.peers.world
        pieces = [(base + lc * 2, M, w * 2, self.n_local * 2,
                   [self.out_off + (gc + s * w) * 2 for s in range(world)], self.N * 2)
                  for lc, gc, w in self.roles]
        self.peers.allgather(pieces)
        full = self.peers.arena.tensor(self.out_off, (M, self.N), torch.bfloat16)
        return full.reshape(*lead, self.N)


class PeerExpertParallelMoE(torch.nn.Module):
    """Expert-parallel routed layer over peer memory.  ``moe_layer`` is a
    :class:`gridbook_b200.moe.CBMoE` holding this rank's ``E / world`` experts (global ids
    ``[rank * E/world, (rank+1) * E/world)``); every rank brings the same number of tokens."""

    def __init__(self, num_experts: int, moe_layer, peers: PeerGroup, max_tokens: int, topk: int, hidden: int):
        super().__init__()
        self.E, self.layer, self.peers = num_experts, moe_layer, peers
        self.world, self.rank = peers.world, peers.rank
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.e_local = num_experts // self.world
        self.max_tokens, self.topk, self.hidden = max_tokens, topk, hidden
        a = peers.arena
        self.x_off = a.carve(self.world * max_tokens * hidden * 2)
        self.id_off = a.carve(self.world * max_tokens * topk * 4)
        self.back_off = a.carve(max_tokens * topk * hidden * 2)
        self._x_row = {}
        # whether the layer's formats have the per-pair table kernel (decided once, the same on
        # every rank: all ranks must make the same sequence of exchange calls)
        w13, w2 = moe_layer._cb_w13, moe_layer._cb_w2
        self._pairs_ok = all(f.is_fp4 and f.mode == "full" and f.k == 8 and f.scale_coding == "v1"
                             for f in (moe_layer.method.fmt13, moe_layer.method.fmt2)) and \
            all(wt.row_stride % 16 == 0 for wt in (w13, w2))
        # ... and the sorted-rows tensor-core kernel for many rows per local expert
        self._sorted_ok = (kernels.moe_gemv_sorted_applies(w13) and kernels.moe_gemv_sorted_applies(w2)
                           and moe_layer._cb_inter % 16 == 0)

    def forward(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        from . import ops
        rule = ops.ACT_SCALE_RULE
        method, layer = self.layer.method, self.layer
        T, topk = topk_ids.shape
        H, world = self.hidden, self.world
        if T > self.max_tokens or topk != self.topk or x.shape[-1] != H:
            raise ValueError(f"batch [{T}, top-{topk}, {x.shape[-1]}] does not fit the reserved peer memory")
        if T == 0:
            raise ValueError("every rank must bring at least one token to the peer exchange")
        dev = x.device
        b13 = kernels.fp4_act_qdq if method.fmt13.is_fp4 else kernels.fp8_act_qdq
        b2 = kernels.fp4_act_qdq if method.fmt2.is_fp4 else kernels.fp8_act_qdq
        ids = topk_ids.to(torch.int32).contiguous()
        from .moe import FUSED_BUCKET_MAX_PAIRS
        PAIR_KERNEL_MAX_PAIRS = method.pair_kernel_max_pairs
        pairs_all = world * T * topk
        # small batches of the literal format: every pair is its own table GEMV (bucket fused)
        # (pairs of other ranks' experts cost a CTA that leaves at once; bound those too)
        # enough rows per expert (all ranks' tokens together): the sorted-rows tensor-core route
        use_sorted = self._sorted_ok and pairs_all >= (method.sorted_min_pairs_per_expert * self.E if self._pairs_ok
                                                       else method.sorted_min_pairs_other)
        per_pair = (not use_sorted and self._pairs_ok and pairs_all // world <= PAIR_KERNEL_MAX_PAIRS
                    and pairs_all <= 4 * PAIR_KERNEL_MAX_PAIRS)
        x2 = x.reshape(T, H).to(torch.bfloat16).contiguous()
        # the bucket is per token, so it can run before the rows travel (the per-pair kernel
        # applies it itself)
        xq = x2 if per_pair else b13(x2, rule)
        self.peers.allgather([
            (xq.data_ptr(), 1, T * H * 2, T * H * 2, [self.x_off + s * T * H * 2 for s in range(world)], T * H * 2),
            (ids.data_ptr(), 1, T * topk * 4, T * topk * 4,
             [self.id_off + s * T * topk * 4 for s in range(world)], T * topk * 4),
        ])
        x_all = self.peers.arena.tensor(self.x_off, (world * T, H), torch.bfloat16)
        ids_all = self.peers.arena.tensor(self.id_off, (world * T, topk), torch.int32)
        key = (world * T, topk)
        x_row = self._x_row.get(key)
        if x_row is None:
            x_row = (torch.arange(world * T * topk, device=dev, dtype=torch.int32) // topk).contiguous()
            self._x_row[key] = x_row
        rows = nat.GbPeerRows()
        rows.rows_per_rank = T * topk
        for r in range(world):
            rows.base[r] = self.peers.arena.ptr(r, self.back_off)
        base = self.rank * self.e_local
        done = False
        if per_pair:
            expect = max(1, pairs_all // world)
            ok = kernels.moe_mlp_pairs(x_all, layer._cb_w13, layer._cb_w2, ids_all, x_row=x_row, act="fp4",
                                       scale_rule=rule, expert_base=base, pairs_expected=expect, peer_rows=rows)
            if ok is None:
                # every rank holds the same formats, so every rank takes this branch together
                raise NativeKernelUnavailableError(
                    "per-pair table MLP refused a format the layer was built for")
            done = True
        if not done and use_sorted:
            # many rows per local expert: sort them, decode every (expert, 128-row tile) into tensor
            # memory and multiply on the tensor cores; the down projection stores each row into its
            # home rank's buffer
            _, offsets, order = kernels.moe_route(ids_all, self.e_local, expert_base=base)
            a = kernels.moe_gather_rows(x_all, order, offsets, x_row=x_row)
            h13 = kernels.moe_gemv_sorted(a, layer._cb_w13, offsets)
            if method.fmt2.is_fp4:
                h = kernels.moe_swiglu_rows(h13, offsets, act="fp4", scale_rule=rule)
            else:
                h = kernels.fp8_act_qdq(kernels.moe_swiglu_rows(h13, offsets), rule)
            kernels.moe_gemv_sorted(h, layer._cb_w2, offsets, row_map=order, peer_rows=rows)
            done = True
        if not done:
            _, offsets, order = kernels.moe_route(ids_all, self.e_local, expert_base=base)
            a = kernels.moe_gemv(x_all, layer._cb_w13, offsets, order, x_row=x_row, swiglu=True, clear=False)
            if method.fmt2.is_fp4 and pairs_all <= FUSED_BUCKET_MAX_PAIRS:
                kernels.moe_gemv(a, layer._cb_w2, offsets, order, peer_rows=rows, act="fp4", scale_rule=rule)
            else:
                kernels.moe_gemv(b2(a, rule), layer._cb_w2, offsets, order, peer_rows=rows)
        back = self.peers.arena.tensor(self.back_off, (T * topk, H), torch.bfloat16)
        # the loop chain multiplies by the bf16-rounded router weight (gridbook/moe.py:2407-2408):
        # the combine rounds the raw weights itself
        # ... and first waits, inside the same launch, until every rank's rows have landed
        out = kernels.moe_combine(back, topk_weights, T, topk, topk_ids=ids, E=self.E, round_weights=True,
                                  peer_group=self.peers.native)
        return out.to(x.dtype).reshape(x.shape)
