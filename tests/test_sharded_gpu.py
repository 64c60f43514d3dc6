"""N-column sharding on real GPUs: two ranks (NCCL), each computing its column shard with the
library, then the optional all-gather; every rank must end up with the single-GPU result.
Skipped unless at least two GPUs are visible."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        import torch.distributed as dist
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import patina_b200
        from patina_b200 import inputs, sharded
        M, N, K = 1024, 1792, 512
        A, B = inputs.make_operands("llm", M, N, K, seed=42)            # same operands on every rank
        ctx = patina_b200.GemmContext(rank)
        dA, dB = A.cuda(), B.cuda()
        n0, n1 = sharded.column_shard(N, world, rank)
        shard = sharded.gemm_column_shard(ctx, dA, dB[n0:n1])
        ctx.status()
        full = sharded.all_gather_columns(shard, N)
        single = ctx.gemm_tn(dA, dB, config=sharded.ASCENDING_K)        # the whole problem on this GPU, summed in
                                                                          # ascending k like the shards
        ctx.status()
        # also: write the shard straight into a full-width C through the leading dimension
        wide = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
        sharded.gemm_column_shard(ctx, dA, dB[n0:n1], out=wide[:, n0:n1])
        ctx.status()
        # the gather fused into the epilogue: every rank's GEMM stores its block into every rank's C
        shared = sharded.SharedC(ctx, M, N)
        shared.local.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        sharded.gemm_scatter_columns(ctx, dA, dB[n0:n1], shared)
        ctx.status()
        dist.barrier()
        fused_ok = bool(torch.equal(shared.local, single))
        dist.barrier()
        shared.close()
        # the host-buffer form over several GPUs: A crosses PCIe once per node (each rank uploads
        # only its slices; the rest of its host copy is poisoned), NVLink all-gather completes it
        M2 = 4100
        A2, _ = inputs.make_operands("llm", M2, 1, K, seed=43)
        run = sharded.HostShardedGemm(ctx, M2, n1 - n0, K, max_blocks=4)
        mine = torch.full((M2, K), float("nan"), dtype=torch.bfloat16).pin_memory()
        for r0, r1, per in run.blocks:
            lo, hi = r0 + rank * per, min(r1, r0 + (rank + 1) * per)
            if hi > lo:
                mine[lo:hi] = A2[lo:hi]
        hB = B[n0:n1].contiguous().pin_memory()
        hC = torch.empty((M2, n1 - n0), dtype=torch.bfloat16).pin_memory()
        for _ in range(2):
            run(mine, hB, hC)
            ctx.status()
        host_ok = bool(torch.equal(hC.cuda(), ctx.gemm_tn(A2.cuda(), dB[n0:n1], config=sharded.ASCENDING_K)))
        ctx.status()
        ok = (bool(torch.equal(full, single)) and bool(torch.equal(wide[:, n0:n1], single[:, n0:n1]))
              and fused_ok and host_ok)
        untouched = bool((wide[:, :n0] == 0).all()) and bool((wide[:, n1:] == 0).all())
        q.put((rank, ok and untouched, tuple(full.shape)))
        dist.destroy_process_group()
    except Exception as exc:
        q.put((rank, False, repr(exc)))


def test_two_gpu_column_shards_and_allgather():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    assert all(ok for _, ok, _ in results), results
