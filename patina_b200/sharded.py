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


class SharedC:
    """One full-width C[M, n_total] (bf16) per rank, each mapped into every other rank's process
    (CUDA IPC through the library's peer_alloc / peer_open). `ptrs[r]` is the address of rank
    r's C as seen from this rank's GPU; `local` is this rank's own C as a tensor. Call close()
    on every rank before the process exits."""

    def __init__(self, ctx, M: int, n_total: int, group=None):
        from .gemm import wrap_bf16
        self.ctx, self.group = ctx, group
        self.M, self.n_total = M, n_total
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        own_ptr, handle = ctx.peer_alloc(M * n_total * 2)
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        self.ptrs = [own_ptr if r == self.rank else ctx.peer_open(handles[r]) for r in range(self.world)]
        self.local = wrap_bf16(own_ptr, M, n_total, ctx.device)

    def column_block_ptrs(self, n0: int) -> list[int]:
        """Where column n0 of this rank's block starts in every rank's C, own buffer first."""
        order = [self.rank] + [r for r in range(self.world) if r != self.rank]
        return [self.ptrs[r] + 2 * n0 for r in order]

    def close(self) -> None:
        self.local = None
        dist.barrier(self.group)           # nobody is still writing into anybody's buffer
        for r, ptr in enumerate(self.ptrs):
            if r != self.rank:
                self.ctx.peer_close(ptr)
        dist.barrier(self.group)           # nobody holds a mapping of anybody's buffer any more
        self.ctx.peer_free(self.ptrs[self.rank])
        self.ptrs = []


def gemm_scatter_columns(ctx, A: torch.Tensor, B_shard: torch.Tensor, shared: SharedC,
                         alpha: float = 1.0, align: int = 256) -> torch.Tensor:
    """This rank's column block of C, written by the GEMM's epilogue into EVERY rank's full C
    (the all-gather fused into the kernel as peer stores over NVLink). No collective is called;
    ranks must synchronise (e.g. stream sync + dist.barrier) before anyone reads its C or reuses it."""
    n0, n1 = column_shard(shared.n_total, shared.world, shared.rank, align)
    if B_shard.shape[0] != n1 - n0:
        raise ValueError(f"rank {shared.rank}: B shard has {B_shard.shape[0]} rows, expected {n1 - n0}")
    if n1 > n0:
        ctx.gemm_bf16_tn_scatter(A, B_shard, shared.column_block_ptrs(n0), shared.n_total, alpha=alpha)
    return shared.local
