"""CPU tests of the multi-GPU row sharding with a 2-rank gloo group: partitioning, the padded
all-gather layout and the column remap.  The local product is computed with the CPU oracle
here (the CUDA kernel takes its place on GPUs; the exchange logic is identical)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from paramspmm_ae_b200 import shard, synth


def test_partition_balances_nnz():
    m = synth.powerlaw_graph(5000, 40000, seed=3)
    for world in (1, 2, 4, 8):
        b = shard.partition_rows_by_nnz(m.rowPtr, world)
        assert b[0] == 0 and b[-1] == m.n_rows and bool((b[1:] >= b[:-1]).all())
        per = [int(m.rowPtr[b[p + 1]] - m.rowPtr[b[p]]) for p in range(world)]
        assert sum(per) == m.nnz
        max_row = int((m.rowPtr[1:] - m.rowPtr[:-1]).max())
        assert max(per) <= m.nnz / world + max_row
    # degenerate inputs
    assert shard.partition_rows_by_nnz(torch.zeros(5, dtype=torch.int32), 3).tolist() == [0, 0, 0, 4]


def test_extract_and_remap():
    m = synth.uniform_rows(50, 4, seed=1)
    rp, ci, v = shard.extract_rows(m.rowPtr, m.colIdx, m.val, 10, 30)
    assert rp[0] == 0 and rp[-1] == 80 and ci.shape[0] == 80
    cb = torch.tensor([0, 13, 50])
    r = shard.remap_columns(torch.tensor([0, 12, 13, 49], dtype=torch.int32), cb, 37)
    assert r.tolist() == [0, 12, 37, 37 + 36]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, dim_chunks, q, exchange="allgather", relabel=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as orc
        m = synth.powerlaw_graph(1201, 9000, seed=7)          # same seed on every rank
        B = synth.dense_uniform(m.n_cols, 24, 5)
        full = orc.spmm_csr(*m.numpy(), B.numpy())
        full2 = orc.spmm_csr(*m.numpy(), full)
        if relabel:  # nodes relabelled before sharding: the same products, rows in the new order
            new_of_old = shard.scattered_labels(m.n_rows, seed=3)
            old_of_new = torch.argsort(new_of_old).numpy()
            m.rowPtr, m.colIdx, m.val = shard.relabel_symmetric(m.rowPtr, m.colIdx, m.val, new_of_old)
            B, full, full2 = B[old_of_new], full[old_of_new], full2[old_of_new]

        def local_spmm(out, Bfull, rowPtr, colIdx, val, accumulate=False):
            prod = torch.from_numpy(orc.spmm_csr(rowPtr.numpy(), colIdx.numpy(), val.numpy(),
                                                 np.ascontiguousarray(Bfull.numpy())))
            out.add_(prod) if accumulate else out.copy_(prod)
            return out

        row_b = shard.partition_rows_by_nnz(m.rowPtr, world)
        op = shard.ShardedSpMM(m.rowPtr, m.colIdx, m.val, m.n_cols, rank, world, row_bounds=row_b,
                               col_bounds=row_b, device="cpu", local_spmm=local_spmm, dim_chunks=1,
                               exchange=exchange)
        lo, hi = op.my_cols
        C_local = op.forward(B[lo:hi].contiguous(), torch.full((op.local_rows, 24), float("nan")))
        ok = np.allclose(C_local.numpy(), full[op.lo: op.hi], rtol=1e-5, atol=1e-5)
        # a second layer: the output shard is the next dense shard (row_bounds == col_bounds)
        C2 = op.forward(C_local)
        ok2 = np.allclose(C2.numpy(), full2[op.lo: op.hi], rtol=1e-4, atol=1e-4)
        q.put((rank, bool(ok), bool(ok2), op.local_rows))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange,relabel", [("allgather", False), ("needed", False), ("pipelined", False),
                                              ("needed_pipelined", False), ("needed", True)])
@pytest.mark.parametrize("world", [2, 3])
def test_sharded_spmm_two_layers_gloo(world, exchange, relabel):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, 1, q, exchange, relabel)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(r[1] and r[2] for r in res), res
    assert sum(r[3] for r in res) == 1201


def test_needed_rows_exchange_single_rank():
    """world = 1: the compact operand holds exactly the referenced rows, in column order, and the
    renumbered columns reproduce the product (no process group involved)."""
    from oracle import oracle as orc
    m = synth.with_empty_rows(synth.powerlaw_graph(801, 3000, seed=9), every=3)
    B = synth.dense_uniform(m.n_cols, 12, 4)

    def local_spmm(out, Bc, rowPtr, colIdx, val):
        out.copy_(torch.from_numpy(orc.spmm_csr(rowPtr.numpy(), colIdx.numpy(), val.numpy(),
                                                np.ascontiguousarray(Bc.numpy()))))
        return out

    op = shard.ShardedSpMM(m.rowPtr, m.colIdx, m.val, m.n_cols, 0, 1, device="cpu", local_spmm=local_spmm,
                           exchange="needed")
    used = torch.unique(m.colIdx.long())
    assert op.n_needed == used.numel() < m.n_cols
    assert torch.equal(op.send_rows, used)
    got = op.forward(B)
    want = orc.spmm_csr(*m.numpy(), B.numpy())
    assert np.allclose(got.numpy(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("row_chunks", [1, 3, 1000])
def test_needed_pipelined_exchange_single_rank(row_chunks):
    """world = 1: the chunks' receive regions tile the compact buffer, together they hold exactly the
    referenced rows, and the block products sum to the full product."""
    from oracle import oracle as orc
    m = synth.with_empty_rows(synth.powerlaw_graph(801, 3000, seed=9), every=3)
    B = synth.dense_uniform(m.n_cols, 12, 4)

    def local_spmm(out, Bc, rowPtr, colIdx, val, accumulate=False):
        prod = torch.from_numpy(orc.spmm_csr(rowPtr.numpy(), colIdx.numpy(), val.numpy(),
                                             np.ascontiguousarray(Bc.numpy())))
        out.add_(prod) if accumulate else out.copy_(prod)
        return out

    op = shard.ShardedSpMM(m.rowPtr, m.colIdx, m.val, m.n_cols, 0, 1, device="cpu", local_spmm=local_spmm,
                           exchange="needed_pipelined", row_chunks=row_chunks)
    used = torch.unique(m.colIdx.long())
    assert op.n_needed == used.numel() < m.n_cols
    assert torch.equal(torch.cat([p[4] for p in op.chunk_plan]), used)  # chunks are runs of rows: order is kept
    end = 0
    for (base, cnt, _, _, _), (rp, ci, v) in zip(op.chunk_plan, op.blocks):
        assert base == end
        end += cnt
        if ci.numel():
            assert base <= int(ci.min()) and int(ci.max()) < end
    got = op.forward(B, torch.full((m.n_rows, 12), float("nan")))
    want = orc.spmm_csr(*m.numpy(), B.numpy())
    assert np.allclose(got.numpy(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("row_chunks", [1, 3, 4, 1000])
def test_pipelined_exchange_single_rank(row_chunks):
    """world = 1: the column blocks partition the entries of the shard, every block indexes its own
    region of the chunked receive buffer, and the block products sum to the full product."""
    from oracle import oracle as orc
    m = synth.with_empty_rows(synth.powerlaw_graph(801, 3000, seed=9), every=3)
    B = synth.dense_uniform(m.n_cols, 12, 4)
    calls = []

    def local_spmm(out, Bc, rowPtr, colIdx, val, accumulate=False):
        calls.append(accumulate)
        prod = torch.from_numpy(orc.spmm_csr(rowPtr.numpy(), colIdx.numpy(), val.numpy(),
                                             np.ascontiguousarray(Bc.numpy())))
        out.add_(prod) if accumulate else out.copy_(prod)
        return out

    op = shard.ShardedSpMM(m.rowPtr, m.colIdx, m.val, m.n_cols, 0, 1, device="cpu", local_spmm=local_spmm,
                           exchange="pipelined", row_chunks=row_chunks)
    assert sum(int(b[1].numel()) for b in op.blocks) == m.nnz
    for k, (rp, ci, v) in enumerate(op.blocks):
        assert rp.numel() == m.n_rows + 1 and int(rp[-1]) == ci.numel() == v.numel()
        if ci.numel():
            assert int(ci.min()) >= k * op.chunk_rows and int(ci.max()) < (k + 1) * op.chunk_rows
    got = op.forward(B, torch.full((m.n_rows, 12), float("nan")))
    assert calls == [False] + [True] * (row_chunks - 1)
    want = orc.spmm_csr(*m.numpy(), B.numpy())
    assert np.allclose(got.numpy(), want, rtol=1e-5, atol=1e-5)
    with pytest.raises(ValueError):
        op.forward(synth.dense_uniform(m.n_cols, 10, 4))


def _pull_worker(rank, world, port, exchange, row_chunks, q):
    """The row lists of the pull transport (the CUDA copy kernel consumes them as they are): every
    rank gathers all blocks of the dense operand (what peer-mapped memory gives it on GPUs), fills its
    compact operand from (owner, row) exactly as the lists say, and the block products must give the
    global product."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as orc
        m = synth.with_empty_rows(synth.powerlaw_graph(1201, 9000, seed=7), every=4)
        B = synth.dense_uniform(m.n_cols, 8, 5)
        op = shard.ShardedSpMM(m.rowPtr, m.colIdx, m.val, m.n_cols, rank, world, device="cpu",
                               local_spmm=lambda *a, **k: None, exchange=exchange, transport="pull",
                               row_chunks=row_chunks)
        blocks = [B[int(op.col_bounds[q_]): int(op.col_bounds[q_ + 1])] for q_ in range(world)]
        recv = torch.full((max(1, op.n_needed), 8), float("nan"))
        lists = op.pull_lists()
        end = 0
        for base, first, rows in lists:
            assert base == end and first[0] == 0 and len(first) == world + 1 and rows.dtype == torch.int32
            assert all(a <= b for a, b in zip(first, first[1:])) and first[-1] == rows.numel()
            for s in range(world):
                r = rows[first[s]: first[s + 1]].long()
                assert r.numel() == 0 or (int(r.min()) >= 0 and int(r.max()) < blocks[s].shape[0])
                assert bool((r[1:] > r[:-1]).all())  # ascending and distinct inside an owner (and a fetch)
                recv[base + first[s]: base + first[s + 1]] = blocks[s][r]
            end += first[-1]
        assert end == op.n_needed and not bool(torch.isnan(recv[: op.n_needed]).any())
        want = orc.spmm_csr(*m.numpy(), B.numpy())[op.lo: op.hi]
        if exchange == "needed":
            got = orc.spmm_csr(op.rowPtr.numpy(), op.colIdx.numpy(), op.val.numpy(), recv.numpy())
        elif exchange == "needed_rowgroups":
            # group k may only touch what fetches 0..k bring
            ends = [base + first[-1] for base, first, _ in lists]
            parts = []
            for k, (rp, ci, v) in enumerate(op.blocks):
                assert ci.numel() == 0 or int(ci.max()) < ends[k]
                parts.append(orc.spmm_csr(rp.numpy(), ci.numpy(), v.numpy(), recv.numpy()))
            assert [p.shape[0] for p in parts] == [b - a for a, b in zip(op.group_bounds, op.group_bounds[1:])]
            got = np.concatenate(parts)
        else:
            got = sum(orc.spmm_csr(rp.numpy(), ci.numpy(), v.numpy(), recv.numpy()) for rp, ci, v in op.blocks)
        q.put((rank, bool(np.allclose(got, want, rtol=1e-5, atol=1e-5)), op.n_needed))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange,row_chunks", [("needed", 1), ("needed_pipelined", 3), ("needed_rowgroups", 3),
                                                 ("needed_rowgroups", 1)])
@pytest.mark.parametrize("world", [2, 3])
def test_pull_transport_row_lists_gloo(world, exchange, row_chunks):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_pull_worker, args=(r, world, port, exchange, row_chunks, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(r[1] for r in res), res
    assert all(0 < r[2] <= 1201 for r in res)


def test_pull_transport_rejects_other_exchanges():
    m = synth.uniform_rows(20, 3, seed=1)
    with pytest.raises(ValueError):
        shard.ShardedSpMM(m.rowPtr, m.colIdx, m.val, 20, 0, 1, device="cpu", exchange="allgather", transport="pull")


@pytest.mark.parametrize("world", [2, 3, 8])
def test_scattered_labels_balance_rows_entries_and_senders(world):
    """Random relabelling: P A P^T gives the same product up to the order of rows, and the
    nnz-balanced contiguous blocks of the relabelled matrix hold about equal rows, and every owner
    is asked for about the same number of dense rows (the natural order is far from both)."""
    m = synth.rmat(12, 60_000, seed=9)
    n = m.n_rows
    new_of_old = shard.scattered_labels(n, seed=5)
    assert torch.equal(new_of_old, shard.scattered_labels(n, seed=5))
    assert sorted(new_of_old.tolist()) == list(range(n))
    rp, ci, v = shard.relabel_symmetric(m.rowPtr, m.colIdx, m.val, new_of_old)
    assert rp.dtype == torch.int32 and ci.dtype == torch.int32 and int(rp[-1]) == m.nnz
    for r in range(0, n, 97):  # columns sorted inside every row
        seg = ci[int(rp[r]): int(rp[r + 1])]
        assert bool((seg[1:] > seg[:-1]).all())
    B = synth.dense_uniform(n, 8, 4)
    dense = lambda a, b, c: torch.sparse_csr_tensor(a.long(), b.long(), c.double(), (n, n)).to_dense()
    want = dense(m.rowPtr, m.colIdx, m.val) @ B.double()
    old_of_new = torch.argsort(new_of_old)
    got = dense(rp, ci, v) @ B.double()[old_of_new]
    torch.testing.assert_close(got, want[old_of_new], rtol=1e-12, atol=1e-12)

    def imbalance(rowPtr, colIdx):
        b = shard.partition_rows_by_nnz(rowPtr, world)
        owner = torch.bucketize(torch.arange(n), b[1:-1], right=True)
        sent = torch.zeros(world, dtype=torch.long)
        for r in range(world):
            need = torch.unique(colIdx[int(rowPtr[b[r]]): int(rowPtr[b[r + 1]])].long())
            c = torch.bincount(owner[need], minlength=world)
            c[r] = 0
            sent += c
        rows = (b[1:] - b[:-1]).double()
        return float(rows.max() / rows.mean()), float(sent.max()) / float(sent.double().mean())

    rows_nat, sent_nat = imbalance(m.rowPtr, m.colIdx)
    rows_int, sent_int = imbalance(rp, ci)
    assert rows_int < 1.3 and sent_int < 1.3  # a 4096-node sample with hubs: a few per cent of noise per block
    assert rows_nat > 1.5 and sent_nat > sent_int


def test_relabel_rejects_rectangular_or_short_permutations():
    m = synth.rmat(8, 1000, seed=2)
    with pytest.raises(ValueError):
        shard.relabel_symmetric(m.rowPtr, m.colIdx, m.val, torch.arange(m.n_rows - 1))
