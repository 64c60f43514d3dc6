"""N-column sharding of one GEMM over the GPUs of a node, one process per GPU.

C[M, N] = A[M, K] @ B[N, K]^T is split by columns of C: rank r holds all of A
(replicated), rows [n0, n1) of B, and produces C[:, n0:n1]. Output tiles are
independent, so the GEMM itself needs no communication; an all-gather of C over
NCCL is offered for a consumer that needs the full result on every rank.

The reference is single-GPU (harness/gemm_check.cpp:222 uses device 0 only); this
module has no counterpart there.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def column_shard(n: int, world: int, rank: int, align: int = 256) -> tuple[int, int]:
    """[start, stop) of rank's columns. Shards are contiguous, sized in multiples of
    `align` (the kernel's tile width) while columns last; trailing ranks may get fewer
    columns or none."""
    if world <= 0 or not (0 <= rank < world) or n < 0:
        raise ValueError("bad shard request")
    blocks = -(-n // align)
    per = -(-blocks // world)
    start = min(n, rank * per * align)
    stop = min(n, (rank + 1) * per * align)
    return start, stop


def shard_sizes(n: int, world: int, align: int = 256) -> list[int]:
    return [b - a for a, b in (column_shard(n, world, r, align) for r in range(world))]


def gemm_column_shard(ctx, A: torch.Tensor, B_shard: torch.Tensor, out: torch.Tensor | None = None,
                      alpha: float = 1.0) -> torch.Tensor:
    """This rank's C[:, n0:n1] = alpha * A @ B_shard^T on its own GPU. `out` may be a
    column slice of a full-width C (row stride N): the kernel takes the leading dimension."""
    return ctx.gemm_tn(A, B_shard, out=out, alpha=alpha)


def all_gather_columns(c_shard: torch.Tensor, n_total: int, group=None, align: int = 256) -> torch.Tensor:
    """Full C[M, n_total] on every rank from the per-rank column shards.

    Each rank contributes a contiguous [M, n_r] block; shards are gathered as
    [world * M, n_max] (padded to the widest shard so one collective moves everything)
    and interleaved back into row-major C.
    """
    world = dist.get_world_size(group)
    sizes = shard_sizes(n_total, world, align)
    rank = dist.get_rank(group)
    M = c_shard.shape[0]
    if c_shard.shape[1] != sizes[rank]:
        raise ValueError(f"rank {rank}: shard has {c_shard.shape[1]} columns, expected {sizes[rank]}")
    n_max = max(sizes)
    send = c_shard
    if sizes[rank] != n_max or not c_shard.is_contiguous():
        send = c_shard.new_zeros((M, n_max))
        send[:, :sizes[rank]] = c_shard
    flat = c_shard.new_empty((world * M, n_max))  # rank r's block is rows [r*M, (r+1)*M)
    dist.all_gather_into_tensor(flat, send.contiguous(), group=group)
    gathered = flat.view(world, M, n_max)
    out = c_shard.new_empty((M, n_total))
    col = 0
    for r, w in enumerate(sizes):
        if w:
            out[:, col:col + w] = gathered[r, :, :w]
        col += w
    return out


def share_full_c(M: int, n_total: int, group=None) -> tuple[torch.Tensor, list[torch.Tensor]]:
    """Every rank allocates one full-width C[M, n_total] (bf16) and maps every other rank's
    into its own process (CUDA IPC through torch's tensor sharing). Returns
    (local_C, [C of rank 0, ..., C of rank W-1]); the entry of this rank is local_C itself.
    Keep local_C alive as long as any rank may still write to it."""
    from torch.multiprocessing.reductions import reduce_tensor
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    local = torch.empty((M, n_total), dtype=torch.bfloat16, device="cuda")
    handles = [None] * world
    dist.all_gather_object(handles, reduce_tensor(local), group=group)
    views = []
    for r, (rebuild, args) in enumerate(handles):
        views.append(local if r == rank else rebuild(*args))
    return local, views


def gemm_scatter_columns(ctx, A: torch.Tensor, B_shard: torch.Tensor, full_views: list[torch.Tensor],
                         n_total: int, group=None, alpha: float = 1.0, align: int = 256) -> torch.Tensor:
    """This rank's column block of C, written by the GEMM's epilogue into EVERY rank's full C
    (the all-gather fused into the kernel as peer stores over NVLink). No collective is called;
    ranks must synchronise (e.g. dist.barrier + stream sync) before anyone reads its C or reuses it."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    n0, n1 = column_shard(n_total, world, rank, align)
    if B_shard.shape[0] != n1 - n0:
        raise ValueError(f"rank {rank}: B shard has {B_shard.shape[0]} rows, expected {n1 - n0}")
    if n1 == n0:
        return full_views[rank]
    order = [rank] + [r for r in range(world) if r != rank]       # own buffer first
    dests = [full_views[r][:, n0:n1] for r in order]
    ctx.gemm_bf16_tn_scatter(A, B_shard, dests, alpha=alpha)
    return full_views[rank]
