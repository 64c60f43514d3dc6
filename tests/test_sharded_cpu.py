"""Column sharding across ranks: shard arithmetic, and the all-gather assembly run as two
gloo ranks on CPU (the per-rank GEMM itself is checked on the GPU, where column shards are
required to reproduce the full result bit for bit)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from patina_b200 import sharded


def test_column_shards_cover_exactly():
    for n, world in [(8192, 1), (8192, 8), (4096, 8), (14336, 8), (28672, 4), (1000, 3), (100, 8), (0, 2)]:
        spans = [sharded.column_shard(n, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 == b0 and a0 <= a1
        assert sum(sharded.shard_sizes(n, world)) == n
        # every shard but the last non-empty one is a whole number of 256-wide tiles
        nonempty = [b - a for a, b in spans if b > a]
        assert all(w % 256 == 0 for w in nonempty[:-1])
    assert sharded.column_shard(14336, 8, 3) == (3 * 1792, 4 * 1792)
    with pytest.raises(ValueError):
        sharded.column_shard(10, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, n_total, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        rng = np.random.default_rng(7)                  # same operands on every rank
        A = rng.standard_normal((48, 64)).astype(np.float32)
        B = rng.standard_normal((n_total, 64)).astype(np.float32)
        n0, n1 = sharded.column_shard(n_total, world, rank)
        shard = torch.from_numpy(oracle.ref_gemm_tn(A, B[n0:n1].copy()).astype(np.float32)) \
            if n1 > n0 else torch.zeros((48, 0))
        full = sharded.all_gather_columns(shard, n_total)
        want = torch.from_numpy(oracle.ref_gemm_tn(A, B).astype(np.float32))
        q.put((rank, bool(torch.equal(full, want)), tuple(full.shape)))
    except Exception as exc:  # report instead of leaving the parent to time out
        q.put((rank, False, repr(exc)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_total", [512, 700, 256])
def test_all_gather_assembles_full_c_two_gloo_ranks(n_total):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_total, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=90) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(ok and shape == (48, n_total) for _, ok, shape in results), results


def test_row_blocks_cover_a_and_split_evenly():
    for m, world in [(8192, 8), (8192, 1), (8192, 2), (1000, 3), (100, 8), (4100, 4), (1, 2)]:
        blocks = sharded.row_blocks(m, world)
        assert blocks[0][0] == 0 and blocks[-1][1] == m
        for (a0, a1, per), (b0, _, _) in zip(blocks, blocks[1:]):
            assert a1 == b0 and a1 - a0 == per * world      # full blocks are `world` equal slices
        r0, r1, per = blocks[-1]
        assert 0 < r1 - r0 <= per * world
    assert sharded.row_blocks(0, 4) == []
    assert len(sharded.row_blocks(8192, 8)) == 8 and sharded.row_blocks(8192, 8)[0] == (0, 1024, 128)


def _host_worker(rank, world, port, shape, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        M, N, K = shape
        rng = np.random.default_rng(11)                 # the same host copy of A and B on every rank
        A = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32))
        B = torch.from_numpy(rng.standard_normal((N, K)).astype(np.float32))
        n0, n1 = sharded.column_shard(N, world, rank, align=8)

        def cpu_gemm(a, b, out=None, alpha=1.0):
            out.copy_(torch.from_numpy((alpha * oracle.ref_gemm_tn(a.contiguous().numpy(),
                                                                    b.contiguous().numpy())).astype(np.float32)))

        class FakeCtx:
            device = 0
            gemm_tn = None
        run = sharded.HostShardedGemm(FakeCtx(), M, n1 - n0, K, dtype=torch.float32, out_dtype=torch.float32,
                                      device="cpu", gemm=cpu_gemm, max_blocks=4)
        # a rank only reads ITS slices of A from the host: poison the rest of its copy
        mineA = torch.full_like(A, float("nan"))
        for r0, r1, per in run.blocks:
            lo, hi = r0 + rank * per, min(r1, r0 + (rank + 1) * per)
            if hi > lo:
                mineA[lo:hi] = A[lo:hi]
        Cn = torch.empty((M, n1 - n0), dtype=torch.float32)
        run(mineA, B[n0:n1].contiguous(), Cn, alpha=0.5)
        want = torch.from_numpy((0.5 * oracle.ref_gemm_tn(A.numpy(), B[n0:n1].contiguous().numpy())).astype(np.float32))
        up, down = run.pcie_bytes()
        rows_up = sum(max(0, min(r1, r0 + (rank + 1) * per) - (r0 + rank * per)) for r0, r1, per in run.blocks)
        q.put((rank, bool(torch.equal(Cn, want)) and up == (rows_up * K + (n1 - n0) * K) * 4
               and down == M * (n1 - n0) * 4, len(run.blocks)))
    except Exception as exc:
        q.put((rank, False, repr(exc)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("shape", [(4096, 64, 32), (4100, 40, 24), (10, 16, 8)])
def test_host_sharded_pipeline_two_gloo_ranks(shape):
    """The multi-GPU host-buffer call's orchestration on two CPU ranks: every rank uploads only
    its slices of A (the rest of its host copy is poisoned with NaN), the all-gather completes
    each row block, and each rank's column shard of C equals the oracle's."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_host_worker, args=(r, world, port, shape, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok is True for _, ok, _ in results), results


def test_c_shard_arithmetic_matches_python(built_lib):
    import ctypes as C
    for n, world in [(8192, 8), (4096, 8), (14336, 8), (28672, 4), (1000, 3), (100, 8), (0, 2), (16384, 8)]:
        for r in range(world):
            a, b = C.c_int64(), C.c_int64()
            built_lib.patina_gemm_column_shard(n, world, r, C.byref(a), C.byref(b))
            assert (a.value, b.value) == sharded.column_shard(n, world, r), (n, world, r)
