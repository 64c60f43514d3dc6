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

from .lib import GemmConfig

# every output summed over k in ascending order in one accumulator: what makes a shard's or a row
# block's result equal, bit for bit, to the same part of an uncut launch with this setting
ASCENDING_K = GemmConfig(k_order=1)


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
    column slice of a full-width C (row stride N): the kernel takes the leading dimension.
    Summed over k in ascending order in one accumulator (`k_order = 1`), so the shard holds the
    bits an unsharded launch with the same setting produces for these columns."""
    return ctx.gemm_tn(A, B_shard, out=out, alpha=alpha, config=ASCENDING_K)


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


# ----------------------------------------------------------- host buffers, many GPUs
def row_blocks(m: int, world: int, max_blocks: int = 8, min_rows: int = 1024) -> list[tuple[int, int, int]]:
    """Row blocks of the replicated A for the pipelined host-buffer call: (first row, one past
    the last row, rows each rank uploads). A block is `world` equal slices (one per rank, the
    last block's slices padded by the caller's buffer), so that every rank uploads 1/world of A
    over its own PCIe link and NVLink carries the rest."""
    if m <= 0:
        return []
    n_blocks = max(1, min(max_blocks, m // max(min_rows, 1)))
    rows = -(-m // n_blocks)
    rows = -(-rows // world) * world            # a whole number of slices
    out = []
    r0 = 0
    while r0 < m:
        r1 = min(m, r0 + rows)
        out.append((r0, r1, rows // world))
        r0 = r1
    return out


class _NoStream:
    """Stands in for a CUDA stream where there is none (host-side tests of the orchestration)."""

    def wait_stream(self, other): pass
    def wait_event(self, ev): pass
    def __enter__(self): return self
    def __exit__(self, *exc): return False


class _NoEvent:
    def record(self, stream=None): pass


class HostShardedGemm:
    """C[:, n0:n1] = alpha * A @ B[n0:n1]^T from HOST buffers on every rank of a node, one
    process per GPU: the multi-GPU form of `GemmContext.gemm_host`.

    A is replicated (every rank holds the same host copy), so it crosses PCIe ONCE per node:
    each rank uploads 1/world of every row block over its own link and an all-gather over
    NVLink hands every rank the whole block. A rank's PCIe traffic per call is therefore
    M*K/world + (n1-n0)*K elements in and M*(n1-n0) out. Row blocks are pipelined on three
    streams: upload + all-gather of block i+1, the GEMM of block i and the copy-out of block
    i-1 run concurrently. Device buffers are allocated once, at construction.

    `gemm(A_block, B, out=C_block, alpha=...)` is the per-rank kernel call, by default the
    context's; `device` "cpu" with an injected `gemm` runs the same orchestration without
    streams (used by the host-side tests, never by the library itself).
    """

    def __init__(self, ctx, m: int, n_shard: int, k: int, dtype=torch.bfloat16, out_dtype=torch.bfloat16,
                 group=None, device=None, gemm=None, max_blocks: int = 8):
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.m, self.n, self.k = m, n_shard, k
        self.device = torch.device("cuda", ctx.device) if device is None else torch.device(device)
        # (row blocks: ascending k, so that the result does not depend on the cut)
        self.gemm = gemm if gemm is not None else (
            lambda a, b, out=None, alpha=1.0: ctx.gemm_tn(a, b, out=out, alpha=alpha, config=ASCENDING_K))
        self.blocks = row_blocks(m, self.world, max_blocks)
        padded = (self.blocks[-1][0] + self.blocks[-1][2] * self.world) if self.blocks else 0
        self.dA = torch.empty((max(padded, m), k), dtype=dtype, device=self.device)
        self.dB = torch.empty((n_shard, k), dtype=dtype, device=self.device)
        self.dC = torch.empty((m, n_shard), dtype=out_dtype, device=self.device)
        cuda = self.device.type == "cuda"
        self.s_in = torch.cuda.Stream(self.device) if cuda else _NoStream()
        self.s_out = torch.cuda.Stream(self.device) if cuda else _NoStream()
        mk = (lambda: torch.cuda.Event()) if cuda else (lambda: _NoEvent())
        self.ev_b = mk()
        self.ev_a = [mk() for _ in self.blocks]
        self.ev_g = [mk() for _ in self.blocks]

    def pcie_bytes(self) -> tuple[int, int]:
        """(host-to-device, device-to-host) bytes this rank moves per call."""
        up_rows = sum(min(per, max(0, min(r1, r0 + (self.rank + 1) * per) - (r0 + self.rank * per)))
                      for r0, r1, per in self.blocks)
        eb, ob = self.dA.element_size(), self.dC.element_size()
        return (up_rows * self.k + self.n * self.k) * eb, self.m * self.n * ob

    def __call__(self, hA: torch.Tensor, hB: torch.Tensor, hC: torch.Tensor, alpha: float = 1.0) -> torch.Tensor:
        cuda = self.device.type == "cuda"
        cur = torch.cuda.current_stream(self.device) if cuda else _NoStream()
        scope = (lambda s: torch.cuda.stream(s)) if cuda else (lambda s: s)
        self.s_in.wait_stream(cur)
        self.s_out.wait_stream(cur)
        with scope(self.s_in):
            self.dB.copy_(hB, non_blocking=True)
            self.ev_b.record(self.s_in)
            for i, (r0, r1, per) in enumerate(self.blocks):
                blk = self.dA[r0:r0 + per * self.world]
                mine = blk[self.rank * per:(self.rank + 1) * per]
                lo = r0 + self.rank * per
                hi = min(r1, lo + per)
                if hi > lo:
                    mine[:hi - lo].copy_(hA[lo:hi], non_blocking=True)
                if self.world > 1:
                    # (in place on the GPU: `mine` is this rank's slot of `blk`)
                    dist.all_gather_into_tensor(blk, mine if cuda else mine.clone(), group=self.group)
                self.ev_a[i].record(self.s_in)
        cur.wait_event(self.ev_b)
        for i, (r0, r1, per) in enumerate(self.blocks):
            cur.wait_event(self.ev_a[i])
            self.gemm(self.dA[r0:r1], self.dB, out=self.dC[r0:r1], alpha=alpha)
            self.ev_g[i].record(cur)
            self.s_out.wait_event(self.ev_g[i])
            with scope(self.s_out):
                hC[r0:r1].copy_(self.dC[r0:r1], non_blocking=True)
        cur.wait_stream(self.s_out)
        return hC
