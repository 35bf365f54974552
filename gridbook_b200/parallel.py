"""Multi-GPU layout of the hot path on one node: column-parallel (N-sharded) dense linears
with an all-gather, and expert-parallel routed MoE with an all-to-all dispatch/combine.
The reference is single-GPU (gridbook/config.py:565-576); nothing here has a counterpart
there.  One process per GPU, collectives through ``torch.distributed`` (NCCL over NVLink;
the host logic below is backend-agnostic and is tested with gloo ranks on the CPU by
injecting the local compute)."""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


# ----------------------------------------------------------------------------- dense
def shard_row_ranges(partition_sizes, rank: int, world: int) -> list[tuple[int, int]]:
    """Rows [start, start+count) of the full matrix that ``rank`` keeps: an equal slice of
    EVERY role, so fused modules (q|k|v, gate|up) keep whole-role row ranges on each rank."""
    out, base = [], 0
    for n in partition_sizes:
        if n % world:
            raise ValueError(f"role of {n} rows does not divide over {world} ranks")
        per = n // world
        out.append((base + rank * per, per))
        base += n
    return out


def shard_rows(t: torch.Tensor, partition_sizes, rank: int, world: int) -> torch.Tensor:
    """The row shard of a per-row tensor (packed weights, weight_scale, cb_row_offset)."""
    return torch.cat([t[s:s + c] for s, c in shard_row_ranges(partition_sizes, rank, world)], dim=0)


def gather_permutation(partition_sizes, world: int) -> torch.Tensor:
    """Column permutation that turns the rank-major concatenation of local outputs
    ``[rank 0 roles..., rank 1 roles..., ...]`` into the full output order."""
    n_local = sum(p // world for p in partition_sizes)
    perm = torch.empty(sum(partition_sizes), dtype=torch.int64)
    for r in range(world):
        pos = r * n_local
        for start, count in shard_row_ranges(partition_sizes, r, world):
            perm[start:start + count] = torch.arange(pos, pos + count)
            pos += count
    return perm


class ShardedCBLinear(torch.nn.Module):
    """Column-parallel wrapper: ``local`` maps x[M, K] to this rank's [M, N/world] columns
    (a :class:`gridbook_b200.linear.CBLinear` over the row shard); forward all-gathers them
    into the full [M, N]."""

    def __init__(self, local: Callable, partition_sizes, group=None):
        super().__init__()
        self.local = local
        self.group = group
        self.world = dist.get_world_size(group)
        self.partition_sizes = list(partition_sizes)
        single_role = len(self.partition_sizes) == 1
        self._perm = None if single_role else gather_permutation(self.partition_sizes, self.world)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.local(x)
        lead, n_local = y.shape[:-1], y.shape[-1]
        y2 = y.reshape(-1, n_local).contiguous()
        out = torch.empty((self.world * y2.shape[0], n_local), dtype=y2.dtype, device=y2.device)
        dist.all_gather_into_tensor(out, y2, group=self.group)            # rank-major [world * M, n_local]
        full = out.view(self.world, y2.shape[0], n_local).permute(1, 0, 2).reshape(y2.shape[0], -1)
        if self._perm is not None:
            if self._perm.device != full.device:
                self._perm = self._perm.to(full.device)
            full = full.index_select(1, self._perm)
        return full.reshape(*lead, -1)


# ----------------------------------------------------------------------------- routed MoE
def expert_owner(expert_ids: torch.Tensor, num_experts: int, world: int) -> torch.Tensor:
    """Rank that holds each expert: contiguous blocks of ``num_experts / world``."""
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not divide over {world} ranks")
    return torch.div(expert_ids, num_experts // world, rounding_mode="floor")


class ExpertParallelMoE(torch.nn.Module):
    """Expert-parallel routed MoE.  Tokens are sharded over the ranks (each rank brings its
    own ``x[T_local, H]`` and routing); rank r holds experts ``[r*E/g, (r+1)*E/g)``.

    forward: sort this rank's (token, slot) pairs by destination rank -> exchange the counts ->
    all-to-all the activation rows and local expert ids -> ``local_fn(rows, local_ids)`` (the
    grouped kernels over the received rows, one row = one pair) -> all-to-all back ->
    ``combine_fn`` (top-k weighted sum) on the token's home rank.  The split sizes of the
    all-to-all are read on the host (one small device-to-host copy per layer)."""

    def __init__(self, num_experts: int, local_fn: Callable, combine_fn: Callable, group=None):
        super().__init__()
        self.E = num_experts
        self.local_fn = local_fn
        self.combine_fn = combine_fn
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.e_local = num_experts // self.world

    def forward(self, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor) -> torch.Tensor:
        T, topk = topk_ids.shape
        H = x.shape[-1]
        dev = x.device
        ids = topk_ids.reshape(-1).to(torch.int64)
        pad = ids < 0                                         # padded routes go nowhere useful: expert 0, weight 0
        ids = ids.masked_fill(pad, 0)
        weights = topk_weights.reshape(-1).masked_fill(pad, 0)
        dest = expert_owner(ids, self.E, self.world)
        order = torch.argsort(dest, stable=True)
        send_counts = torch.bincount(dest, minlength=self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        send_split, recv_split = send_counts.tolist(), recv_counts.tolist()
        token_of_pair = torch.div(order, topk, rounding_mode="floor")
        send_rows = x.reshape(T, H).index_select(0, token_of_pair).contiguous()
        send_ids = (ids.index_select(0, order) - dest.index_select(0, order) * self.e_local).to(torch.int32)
        R = int(sum(recv_split))
        recv_rows = torch.empty((R, H), dtype=x.dtype, device=dev)
        recv_ids = torch.empty((R,), dtype=torch.int32, device=dev)
        dist.all_to_all_single(recv_rows, send_rows, recv_split, send_split, group=self.group)
        dist.all_to_all_single(recv_ids, send_ids.contiguous(), recv_split, send_split, group=self.group)
        y_rows = self.local_fn(recv_rows, recv_ids) if R > 0 else recv_rows.new_empty((0, H))
        back = torch.empty((T * topk, H), dtype=y_rows.dtype, device=dev)
        dist.all_to_all_single(back, y_rows.contiguous(), send_split, recv_split, group=self.group)
        y_pairs = torch.empty_like(back)
        y_pairs.index_copy_(0, order, back)                   # undo the destination sort
        return self.combine_fn(y_pairs, weights, T, topk).reshape(x.shape)


def make_local_expert_fn(moe_layer):
    """``local_fn`` over a :class:`gridbook_b200.moe.CBMoE` that holds this rank's experts:
    every received row is one routed pair (top-k = 1 locally), so the grouped kernels run as
    route -> bucket -> gate/up GEMV with SwiGLU -> bucket -> down GEMV, without the combine."""
    from . import kernels, ops
    method = moe_layer.method

    def local_fn(rows: torch.Tensor, local_ids: torch.Tensor) -> torch.Tensor:
        rule = ops.ACT_SCALE_RULE
        _, offsets, order = kernels.moe_route(local_ids.reshape(-1, 1), moe_layer._cb_E)
        b13 = kernels.fp4_act_qdq if method.fmt13.is_fp4 else kernels.fp8_act_qdq
        b2 = kernels.fp4_act_qdq if method.fmt2.is_fp4 else kernels.fp8_act_qdq
        a = kernels.moe_gemv(b13(rows.contiguous(), rule), moe_layer._cb_w13, offsets, order, swiglu=True)
        return kernels.moe_gemv(b2(a, rule), moe_layer._cb_w2, offsets, order)

    return local_fn


def kernel_combine(y_pairs, weights, T, topk):
    from . import kernels
    return kernels.moe_combine(y_pairs, weights.to(torch.bfloat16).to(torch.float32), T, topk)
