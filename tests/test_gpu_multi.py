"""Row-sharded SpMM on two GPUs of one node: every exchange mode and transport gives the product
that the same shard computes against a replicated dense operand.  Skipped on a single GPU (the
host-side logic of the same code runs under gloo in test_shard_gloo.py)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

MODES = [("allgather", "nccl", 1), ("allgather", "nccl", 4), ("needed", "nccl", 1), ("pipelined", "nccl", 1),
         ("needed_pipelined", "nccl", 1), ("pipelined", "copy_engine", 1), ("needed", "pull", 1),
         ("needed_pipelined", "pull", 1), ("needed_rowgroups", "pull", 1),
         ("needed_rowgroups", "pull_bulk_later", 1), ("needed", "pull_bulk_all", 1)]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    from paramspmm_ae_b200 import synth
    from paramspmm_ae_b200.shard import ShardedSpMM

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        m = synth.rmat(14, 400_000, seed=5, device=dev)  # same matrix on every rank
        n, dim = m.n_rows, 64
        B = synth.dense_uniform(n, dim, 6, dev)
        base = ShardedSpMM(m.rowPtr, m.colIdx, m.val, n, rank, world, device=dev)
        a, b = int(m.rowPtr[base.lo]), int(m.rowPtr[base.hi])
        base.keep_global_columns(m.colIdx[a:b].clone())
        want = base.forward_replicated(B)
        c0, c1 = base.my_cols
        shard_of_B = B[c0:c1].contiguous()
        worst = {}
        for exchange, transport, dim_chunks in MODES:
            bulk = {"pull_bulk_later": 1, "pull_bulk_all": 2}.get(transport, 0)  # fetches on the bulk-copy kernel
            label, transport = transport, ("pull" if bulk else transport)
            op = ShardedSpMM(m.rowPtr, m.colIdx, m.val, n, rank, world, device=dev, exchange=exchange,
                             transport=transport, dim_chunks=dim_chunks, row_chunks=3)
            op.pull_bulk = bulk
            src = shard_of_B
            if transport in ("copy_engine", "pull"):
                src = op.symmetric_input(dim)
                src.copy_(shard_of_B)
            for _ in range(2):  # the second call reuses buffers, fences and streams of the first
                got = op.forward(src, torch.full((op.local_rows, dim), float("nan"), device=dev))
            torch.cuda.synchronize()
            # hub rows add thousands of terms in an order that differs between launches
            worst["%s/%s/%d" % (exchange, label, dim_chunks)] = float(
                ((got - want).abs() / (1e-3 + 1e-4 * want.abs())).max())
        from paramspmm_ae_b200 import ops
        assert ops.pull_rows_status() == 0  # no bounded wait of the bulk-copy kernel ran out
        q.put((rank, worst, base.local_rows))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_spmm_on_two_gpus():
    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sum(r[2] for r in res) == 1 << 14
    for _, worst, _ in res:
        assert len(worst) == len(MODES) and all(v <= 1.0 for v in worst.values()), worst
