"""Row-sharded SpMM across the GPUs of one node (one process per GPU, torch.distributed).

The reference is single-GPU.  The product C = A B shards naturally by rows of A: rank p owns
a contiguous block of rows of A (chosen on the prefix sum of rowPtr so every rank holds about
nnz / world entries), the same block of rows of C, and, between GNN layers, the matching block
of rows of the dense operand.  The one exchange step is an all-gather of the dense row blocks
(NCCL over NVLink on GPUs); the SpMM itself is local and needs no collective.

Unequal row blocks are gathered without any repacking: every rank pads its block to the
largest block's row count, ``all_gather_into_tensor`` lays the padded blocks one after the
other, and the column indices of the local shard of A are remapped ONCE, at set-up, to
positions in that padded layout (column c owned by rank q at local row i becomes
q * max_rows + i).  The gathered buffer is then the dense operand as it stands.

``exchange="needed"`` replaces the dense all-gather by a sparse one: at set-up every rank works out
which rows of the dense operand its shard of A references at all (the distinct column ids), asks
each owner for exactly those, and renumbers its columns to positions in the compact receive
buffer.  Per product every rank then gathers the requested rows into one send buffer and a single
all-to-all with uneven splits moves them.  On power-law graphs a shard touches a fraction of the
columns, so the bytes on NVLink shrink by that fraction, and the SpMM gathers from a smaller
operand.

``exchange="pipelined"`` hides the SpMM under the exchange.  Every rank's block of the dense
operand is cut into ``row_chunks`` runs of rows; chunk k of all ranks is gathered by one
all-gather into its own region of the receive buffer, and the local shard of A is cut, at set-up,
into the matching column blocks (block k holds the entries whose column lies in chunk k of its
owner).  C is then the sum over k of A_k B_k: the product of block k starts as soon as chunk k has
arrived, while chunk k+1 is still on the wire; the first product overwrites C, the others add to
it (``pspmm_cfg.accumulate``).  Unlike slicing the dense columns, this reads every entry of A
once and keeps full-width row gathers.

``transport="copy_engine"`` (pipelined exchange only) moves the chunks without NCCL kernels:
every rank keeps its block of the dense operand in a buffer that its peers have mapped
(``torch.distributed._symmetric_memory``), and each rank pulls the chunks it needs with plain
device-to-device copies, which the GPU's copy engines execute over NVLink.  No SM is taken from the
SpMM and none of its memory instructions queue behind the transfer, so the overlap is the
arithmetic one expects; two one-element all-reduces per product fence the peers' reads (blocks
ready before the first pull, pulls finished before a block may be overwritten).  A producer can
write straight into ``symmetric_input(dim)`` and pass that to ``forward`` to skip the staging copy.

``exchange="needed_pipelined"`` combines the two: the rows a shard references are requested chunk
by chunk (the same cut of every owner's block into ``row_chunks`` runs of rows), one all-to-all
per chunk, and the product of column block k runs while the rows of chunk k+1 are on the wire.

``transport="pull"`` (the two "needed" exchanges) does away with the pack, the all-to-all and the
request lists: every rank keeps its block of the dense operand in peer-mapped memory and each rank
fetches the rows it references with ONE copy kernel that reads the owners' blocks directly
(``pspmm_pull_rows``: plain 16-byte loads over NVLink, a bounded number of thread blocks, every
rank starting at a different owner), straight into its compact operand.  With
``exchange="needed_pipelined"`` the fetch of chunk k+1 runs beside the product of column block k.
The kernel waits on nothing; a one-element all-reduce before the fetches (every block is in place)
and one after them (every peer has finished reading) order it against the producers.

``exchange="needed_rowgroups"`` (pull transport) pipelines without cutting A by columns: the
shard's rows are cut into ``row_chunks`` contiguous groups of about equal entry counts, the rows
of the dense operand are fetched in the order in which the groups first need them (fetch k brings
what group k references and no earlier group did, hub columns therefore in fetch 0), and the
product of row group k, a plain overwrite of its own rows of C at full row length, starts when
fetches 0..k have arrived, beside fetch k+1.  Every entry of A is read once, no product adds into
another's output, and the groups are views of the shard's arrays.

``pull_bulk`` (an attribute of the operator: 0, 1 or 2) moves the fetches after the first (1) or
all fetches (2) with ``pspmm_pull_rows_bulk``, the same copy on bulk asynchronous copies through
shared memory: one warp and no data registers per thread block, so a fetch that runs beside a
product takes far fewer warp slots from it.

Which rank's link is busy depends on the node order.  The dense operand is dealt in equal row
blocks; where the degree of a node depends on its id (R-MAT, degree-sorted graphs) one block holds
the hub columns that every rank references and its owner sends several times the mean, and the
nnz-balanced row blocks of A are as uneven in row count.  ``scattered_labels`` +
``relabel_symmetric`` relabel the nodes once by a seeded random permutation (P A P^T: the same
product up to the order of rows), after which every block is a uniform sample of the nodes.

``dim_chunks > 1`` splits the dense columns into slices and gathers slice s+1 on a side
stream while the SpMM of slice s runs (the kernels take explicit leading dimensions, so a
slice of C is written in place).
"""
from __future__ import annotations

import torch


def partition_rows_by_nnz(rowPtr, world):
    """Row boundaries [world + 1]: block p = rows [b[p], b[p+1]) holds about nnz / world entries."""
    rp = torch.as_tensor(rowPtr).long().cpu()
    n = rp.numel() - 1
    nnz = int(rp[-1])
    targets = torch.tensor([(nnz * p) // world for p in range(1, world)], dtype=torch.long)
    cuts = torch.searchsorted(rp, targets, right=False).clamp_(0, n)
    b = torch.cat([torch.zeros(1, dtype=torch.long), cuts, torch.tensor([n])])
    return torch.cummax(b, 0).values  # non-decreasing even for degenerate inputs


def partition_rows_even(n, world):
    return torch.tensor([(n * p) // world for p in range(world + 1)], dtype=torch.long)


def scattered_labels(n, seed=0):
    """new_of_old [n] (int64): a seeded random permutation of the node ids, the same on every rank.

    On matrices whose degree depends on the node id (R-MAT: on its bits; degree-sorted graphs: on
    its size) contiguous row blocks balanced by nnz give one rank the hubs and another most of the
    rows; the latter then owns, and has to send, most of the dense rows the others reference, and
    its outgoing link bounds the exchange.  With scattered labels every block is a uniform sample of
    the nodes: about equal rows, equal entries and equal traffic in and out of every rank, for any
    number of ranks.  It also scatters whatever index locality the matrix had, so it is meant for
    skewed matrices without a band structure.  Apply once when the graph is loaded
    (:func:`relabel_symmetric`); features, labels and outputs then live in the new order."""
    g = torch.Generator()
    g.manual_seed(int(seed))
    return torch.randperm(n, generator=g, dtype=torch.int64)


def relabel_symmetric(rowPtr, colIdx, val, new_of_old):
    """P A P^T for the permutation ``new_of_old``: CSR arrays (int32, int32, fp32) of the matrix
    whose row and column ids are the new labels, columns sorted inside every row.  Runs on the
    device the arrays are on."""
    dev = colIdx.device
    n = rowPtr.shape[0] - 1
    perm = torch.as_tensor(new_of_old).to(dev).long()
    if perm.shape[0] != n or colIdx.numel() and int(colIdx.max()) >= n:
        raise ValueError("a symmetric relabelling needs a square matrix and one label per node")
    lens = (rowPtr[1:] - rowPtr[:-1]).long()
    keys = torch.repeat_interleave(perm, lens) * n
    keys += perm[colIdx.long()]
    keys, order = torch.sort(keys)
    new_val = val[order]
    del order
    rows = torch.div(keys, n, rounding_mode="floor")
    new_col = (keys - rows * n).to(torch.int32)
    del keys
    rp = torch.zeros(n + 1, dtype=torch.int64, device=dev)
    rp[1:] = torch.cumsum(torch.bincount(rows, minlength=n), 0)
    return rp.to(torch.int32), new_col, new_val


def extract_rows(rowPtr, colIdx, val, lo, hi):
    """Rows [lo, hi) of a CSR matrix with re-based row pointers and global column ids."""
    rp = torch.as_tensor(rowPtr)
    a, b = int(rp[lo]), int(rp[hi])
    part = lambda t: t[a:b].clone() if (b - a) < t.shape[0] else t  # a slice would keep the whole array alive
    return ((rp[lo: hi + 1] - rp[lo]).to(torch.int32).contiguous(), part(colIdx), part(val))


def remap_columns(colIdx, col_bounds, max_rows):
    """Global column ids -> positions in the padded all-gather layout."""
    cb = torch.as_tensor(col_bounds).long().to(colIdx.device)
    c = colIdx.long()
    owner = torch.searchsorted(cb, c, right=True) - 1
    return (owner * max_rows + (c - cb[owner])).to(torch.int32)


class ShardedSpMM:
    """One rank's share of a row-sharded SpMM.

    ``row_bounds``: rows of A / C per rank.  ``col_bounds``: rows of the dense operand per rank
    (for a square matrix between GNN layers this is ``row_bounds`` again).  ``local_spmm`` is the
    kernel launcher ``f(out, B, rowPtr, colIdx, val)``; it defaults to the CUDA operator.
    """

    def __init__(self, rowPtr, colIdx, val, n_cols, rank, world, row_bounds=None, col_bounds=None,
                 device="cuda", group=None, local_spmm=None, dim_chunks=1, exchange="allgather",
                 row_chunks=4, transport="nccl", local_block=None):
        if exchange not in ("allgather", "needed", "pipelined", "needed_pipelined", "needed_rowgroups"):
            raise ValueError("exchange must be 'allgather', 'needed', 'pipelined', 'needed_pipelined' or "
                             "'needed_rowgroups'")
        if row_chunks < 1:
            raise ValueError("row_chunks must be at least 1")
        if transport not in ("nccl", "copy_engine", "pull"):
            raise ValueError("transport must be 'nccl', 'copy_engine' or 'pull'")
        if transport == "copy_engine" and exchange != "pipelined":
            raise ValueError("the copy-engine transport moves whole row chunks: use exchange='pipelined'")
        if transport == "pull" and exchange not in ("needed", "needed_pipelined", "needed_rowgroups"):
            raise ValueError("the pull transport fetches referenced rows: use exchange='needed', "
                             "'needed_pipelined' or 'needed_rowgroups'")
        if exchange == "needed_rowgroups" and transport != "pull":
            raise ValueError("exchange='needed_rowgroups' is built on the pull transport")
        self.trace = False  # pull transport: bracket the fetches and products of a call with timing events (trace_result)
        self.pull_bulk = 0  # 1: fetches that run beside a product use the bulk-copy kernel (one warp per block); 2: all fetches
        self.pull_ctas = 128  # thread blocks of one fetch: enough loads in flight to fill NVLink (measured), few enough to leave the SMs to the SpMM
        self.transport, self._peer = transport, None
        self.rank, self.world, self.group, self.dim_chunks = rank, world, group, dim_chunks
        self.exchange, self.row_chunks = exchange, row_chunks
        self.row_bounds = partition_rows_by_nnz(rowPtr, world) if row_bounds is None else torch.as_tensor(row_bounds).long()
        self.col_bounds = partition_rows_even(n_cols, world) if col_bounds is None else torch.as_tensor(col_bounds).long()
        if int(self.col_bounds[-1]) != n_cols or int(self.row_bounds[-1]) != len(rowPtr) - 1:
            raise ValueError("bounds do not cover the matrix")
        self.max_rows = int((self.col_bounds[1:] - self.col_bounds[:-1]).max())
        lo, hi = int(self.row_bounds[rank]), int(self.row_bounds[rank + 1])
        self.lo, self.hi = lo, hi
        # local_block = (rowPtr, colIdx with global ids, val) of this rank's rows when the caller has
        # extracted them already (several operators over one shard then share these arrays)
        rp, ci, v = local_block if local_block is not None else extract_rows(rowPtr, colIdx, val, lo, hi)
        self.rowPtr = rp.to(device)
        self.val = v.to(device)
        self.device = torch.device(device)
        self.my_cols = (int(self.col_bounds[rank]), int(self.col_bounds[rank + 1]))
        if exchange == "needed":
            self._plan_needed_rows(ci.to(device))
        elif exchange == "pipelined":
            self._plan_row_chunks(ci.to(device))
        elif exchange == "needed_pipelined":
            self._plan_needed_row_chunks(ci.to(device))
        elif exchange == "needed_rowgroups":
            self._plan_needed_row_groups(ci.to(device))
        else:
            self.colIdx = remap_columns(ci.to(device), self.col_bounds, self.max_rows)
        if exchange in ("pipelined", "needed_pipelined", "needed_rowgroups"):
            self.block_spmm = [local_spmm if local_spmm is not None else self._planned_spmm(rp_k)
                               for rp_k, _, _ in self.blocks]
        else:
            self.local_spmm = local_spmm if local_spmm is not None else self._planned_spmm()
        overlap = dim_chunks > 1 or exchange in ("pipelined", "needed_pipelined") or transport == "pull"
        # The fetch kernels of the pull transport run beside SpMM launches that fill the GPU on their
        # own: a high-priority stream lets their few thread blocks take SM slots as the SpMM's blocks
        # retire instead of queueing behind the whole grid.
        self._side = (torch.cuda.Stream(priority=-1 if transport == "pull" else 0)
                      if (self.device.type == "cuda" and overlap) else None)
        self._pull_streams = ([torch.cuda.Stream() for _ in range(min(3, world - 1))]
                              if (self._side is not None and transport == "copy_engine") else [])

    def _plan_row_chunks(self, cols_global):
        """Set-up of the pipelined exchange: the receive buffer is [row_chunks][world][chunk_rows]
        rows; column c, row i of owner q's block, lives at ((i // chunk_rows) * world + q) *
        chunk_rows + i % chunk_rows.  The shard of A is regrouped into one CSR matrix per chunk
        (entries keep their row order), all of them indexing that one buffer."""
        dev = cols_global.device
        K, W, n_loc = self.row_chunks, self.world, self.hi - self.lo
        cr = max(1, -(-self.max_rows // K))
        self.chunk_rows = cr
        cb = self.col_bounds.to(dev)
        c = cols_global.long()
        owner = torch.searchsorted(cb, c, right=True) - 1
        local = c - cb[owner]
        k = torch.div(local, cr, rounding_mode="floor")
        pos = ((k * W + owner) * cr + (local - k * cr)).to(torch.int32)
        rows = torch.repeat_interleave(torch.arange(n_loc, device=dev),
                                       (self.rowPtr[1:] - self.rowPtr[:-1]).long())
        key = k * n_loc + rows
        del c, owner, local, k
        order = torch.argsort(key, stable=True)
        counts = torch.bincount(key, minlength=K * n_loc).view(K, n_loc)
        del key, rows
        pos, val = pos[order], self.val[order]
        del order
        sizes = [int(x) for x in counts.sum(1).cpu()]
        self.blocks, a = [], 0
        for kk in range(K):
            rp = torch.zeros(n_loc + 1, dtype=torch.int32, device=dev)
            rp[1:] = counts[kk].cumsum(0)
            self.blocks.append((rp, pos[a: a + sizes[kk]].contiguous(), val[a: a + sizes[kk]].contiguous()))
            a += sizes[kk]
        self.val = self.colIdx = None  # held per block from here on

    def _plan_needed_row_chunks(self, cols_global):
        """Set-up of the chunked sparse exchange.  Chunk k covers rows [k, k+1) * chunk_rows of every
        owner's block; for each chunk: the distinct referenced columns (sorted, hence grouped by
        owner), the row ids every owner has to send, and the column block of A renumbered to
        positions in one receive buffer that holds the chunks one after the other."""
        import torch.distributed as dist

        dev = cols_global.device
        K, W, n_loc = self.row_chunks, self.world, self.hi - self.lo
        cr = max(1, -(-self.max_rows // K))
        self.chunk_rows = cr
        cb = self.col_bounds.to(dev)
        c = cols_global.long()
        owner = torch.searchsorted(cb, c, right=True) - 1
        k = torch.div(c - cb[owner], cr, rounding_mode="floor")
        rows = torch.repeat_interleave(torch.arange(n_loc, device=dev),
                                       (self.rowPtr[1:] - self.rowPtr[:-1]).long())
        key = k * n_loc + rows
        order = torch.argsort(key, stable=True)
        counts = torch.bincount(key, minlength=K * n_loc).view(K, n_loc)
        del key, rows, owner
        c, val = c[order], self.val[order]
        del order
        sizes = [int(x) for x in counts.sum(1).cpu()]
        self.blocks, self.chunk_plan, a, base = [], [], 0, 0
        for kk in range(K):
            ck = c[a: a + sizes[kk]]
            need = torch.unique(ck)  # sorted distinct global column ids of this chunk
            cuts = torch.searchsorted(need, cb)
            recv_counts = (cuts[1:] - cuts[:-1]).cpu()
            own = torch.repeat_interleave(torch.arange(W, device=dev), recv_counts.to(dev))
            wanted = (need - cb[own]).to(torch.int64)
            recv_splits = [int(x) for x in recv_counts]
            if self.transport == "pull":  # the reader addresses the owners' blocks itself: nothing to request
                send_splits, send_rows = None, wanted.to(torch.int32)
            elif W == 1:
                send_splits, send_rows = list(recv_splits), wanted
            else:
                counts_out = torch.empty(W, dtype=torch.int64, device=dev)
                dist.all_to_all_single(counts_out, recv_counts.to(dev), group=self.group)
                send_splits = [int(x) for x in counts_out.cpu()]
                send_rows = torch.empty(sum(send_splits), dtype=torch.int64, device=dev)
                dist.all_to_all_single(send_rows, wanted, output_split_sizes=send_splits,
                                       input_split_sizes=recv_splits, group=self.group)
            rp = torch.zeros(n_loc + 1, dtype=torch.int32, device=dev)
            rp[1:] = counts[kk].cumsum(0)
            pos = (base + torch.searchsorted(need, ck)).to(torch.int32)
            self.blocks.append((rp, pos, val[a: a + sizes[kk]].contiguous()))
            self.chunk_plan.append((base, int(need.numel()), recv_splits, send_splits, send_rows))
            base += int(need.numel())
            a += sizes[kk]
        self.n_needed = base
        self.val = self.colIdx = None

    def _plan_needed_row_groups(self, cols_global):
        """Set-up of the row-group pipeline: contiguous groups of local rows with about equal entry
        counts; the compact operand is ordered by the group that first references a row (inside a
        group by column, hence by owner); fetch k = the rows first needed by group k."""
        dev = cols_global.device
        K, W, n_loc = self.row_chunks, self.world, self.hi - self.lo
        rp = self.rowPtr.long()
        nnz = int(rp[-1])
        targets = torch.tensor([(nnz * k) // K for k in range(1, K)], dtype=torch.long, device=dev)
        cuts = torch.searchsorted(rp, targets).clamp_(0, n_loc)
        bounds = torch.cummax(torch.cat([torch.zeros(1, dtype=torch.long, device=dev), cuts,
                                         torch.tensor([n_loc], device=dev)]), 0).values
        self.group_bounds = [int(x) for x in bounds.cpu()]
        c = cols_global.long()
        need = torch.unique(c)                      # sorted distinct global column ids
        inv = torch.searchsorted(need, c)           # entry -> index into need
        rows = torch.repeat_interleave(torch.arange(n_loc, device=dev), rp[1:] - rp[:-1])
        grp = torch.searchsorted(bounds[1:].contiguous(), rows, right=True).clamp_(max=K - 1)  # group of every entry's row
        first = torch.full((need.numel(),), K, dtype=torch.long, device=dev).scatter_reduce(0, inv, grp, "amin")
        del rows, grp
        order = torch.argsort(first, stable=True)   # compact order: by first group, then by column
        pos = torch.empty_like(order)
        pos[order] = torch.arange(order.numel(), device=dev)
        self.colIdx = pos[inv].to(torch.int32)
        del inv, pos
        cb = self.col_bounds.to(dev)
        counts = torch.bincount(first, minlength=K)[:K]
        self.chunk_plan, self.blocks, base = [], [], 0
        need_o = need[order]
        for k in range(K):
            cnt = int(counts[k])
            ids = need_o[base: base + cnt]          # ascending global column ids of this fetch
            cuts_k = torch.searchsorted(ids, cb)
            recv_counts = (cuts_k[1:] - cuts_k[:-1]).cpu()
            own = torch.repeat_interleave(torch.arange(W, device=dev), recv_counts.to(dev))
            wanted = (ids - cb[own]).to(torch.int32)
            self.chunk_plan.append((base, cnt, [int(x) for x in recv_counts], None, wanted))
            r0, r1 = self.group_bounds[k], self.group_bounds[k + 1]
            a, b = int(rp[r0]), int(rp[r1])
            self.blocks.append(((self.rowPtr[r0: r1 + 1] - self.rowPtr[r0]).contiguous(), self.colIdx[a:b], self.val[a:b]))
            base += cnt
        self.n_needed = base

    def _forward_needed_pipelined(self, B_shard, out):
        import torch.distributed as dist

        dim = B_shard.shape[1]
        recv = self._receive_buffer(max(1, self.n_needed), dim, B_shard)
        cuda = self._side is not None
        main = torch.cuda.current_stream() if cuda else None
        events = []

        def exchange(kk):
            base, cnt, recv_splits, send_splits, send_rows = self.chunk_plan[kk]
            send = B_shard.index_select(0, send_rows)
            dst = recv[base: base + cnt]
            if self.world == 1:
                dst.copy_(send)
            else:
                dist.all_to_all_single(dst, send, output_split_sizes=recv_splits,
                                       input_split_sizes=send_splits, group=self.group)

        if cuda:
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                for kk in range(self.row_chunks):
                    exchange(kk)
                    ev = torch.cuda.Event()
                    ev.record(self._side)
                    events.append(ev)
            B_shard.record_stream(self._side)
        for kk in range(self.row_chunks):
            if cuda:
                main.wait_event(events[kk])
            else:
                exchange(kk)
            rp, ci, v = self.blocks[kk]
            self.block_spmm[kk](out, recv, rp, ci, v, accumulate=kk > 0)
        return out

    def _receive_buffer(self, rows, dim, like):
        """The receive buffer of the pipelined exchanges, kept between calls: both streams use it,
        and the side stream waits for the main one before it writes, so one buffer is enough and
        the allocator is not asked for gigabytes per product."""
        buf = getattr(self, "_recv", None)
        if buf is None or buf.shape != (rows, dim) or buf.dtype != like.dtype or buf.device != like.device:
            buf = self._recv = torch.empty(rows, dim, dtype=like.dtype, device=like.device)
        return buf

    def _peer_blocks(self, dim, like):
        """This rank's block of the dense operand in peer-mapped memory, padded to whole chunks,
        plus the peers' blocks as local tensors.  Created once per width (a collective call)."""
        if self._peer is None or self._peer[0].shape[1] != dim or self._peer[0].dtype != like.dtype:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm

            rows = self.max_rows if self.transport == "pull" else self.row_chunks * self.chunk_rows
            if self.world == 1:  # no peers: an ordinary buffer stands in for the mapped one
                src = torch.zeros((rows, dim), dtype=like.dtype, device=like.device)
                self._peer = (src, [src], None)
                return self._peer
            src = symm.empty((rows, dim), dtype=like.dtype, device=like.device)
            src.zero_()
            group = self.group if self.group is not None else dist.group.WORLD
            hdl = symm.rendezvous(src, group.group_name)
            peers = [hdl.get_buffer(q, (rows, dim), like.dtype) for q in range(self.world)]
            fence = torch.zeros(1, dtype=torch.int32, device=like.device)
            self._peer = (src, peers, fence)
        return self._peer

    def symmetric_input(self, dim, dtype=torch.float32):
        """The peer-mapped buffer for this rank's block of the dense operand (copy-engine and pull transports):
        rows [0, my block's row count) of it, for a producer to write into and hand to ``forward``."""
        like = torch.empty(0, dtype=dtype, device=self.device)
        return self._peer_blocks(dim, like)[0][: self.my_cols[1] - self.my_cols[0]]

    def _forward_pull(self, B_shard, out):
        """Both "needed" exchanges over the pull transport: fetch kernels on the side stream, one per
        chunk, each followed by an event; the products on the main stream wait for their chunk."""
        import torch.distributed as dist

        from . import ops

        rows, dim = B_shard.shape
        src, peers, fence = self._peer_blocks(dim, B_shard)
        recv = self._receive_buffer(max(1, self.n_needed), dim, B_shard)
        main = torch.cuda.current_stream()
        side = self._side
        events = []
        # with `trace` set, timing events bracket every fetch and every product of this call
        tr = {"start": None, "fetch": [], "product": [], "end": None} if self.trace else None

        def mark(stream):
            e = torch.cuda.Event(enable_timing=True)
            e.record(stream)
            return e

        if tr is not None:
            tr["start"] = mark(main)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            if B_shard.data_ptr() != src.data_ptr():
                src[:rows].copy_(B_shard)
            if fence is not None:
                dist.all_reduce(fence, group=self.group)  # every block is in place
            for kk, (base, cnt, recv_splits, _, want_rows) in enumerate(self.chunk_plan):
                first = [0]
                for c in recv_splits:
                    first.append(first[-1] + c)
                t_a = mark(side) if tr is not None else None
                if cnt:
                    # start at the next rank's rows so that the ranks read different owners at a time
                    rotate = first[(self.rank + 1) % self.world] % cnt
                    # no product of this call runs beside the first fetch: it may use every SM
                    ops.pull_rows(recv[base: base + cnt], peers, first, want_rows, rotate=rotate,
                                  ctas=self.pull_ctas if kk else 8 * self.pull_ctas,
                                  bulk=self.pull_bulk > (0 if kk else 1))
                ev = torch.cuda.Event(enable_timing=tr is not None)
                ev.record(side)
                events.append(ev)
                if tr is not None:
                    tr["fetch"].append((t_a, ev))
            if fence is not None:
                dist.all_reduce(fence, group=self.group)  # every peer has finished reading this block
        B_shard.record_stream(side)

        def product(fn):
            t_a = mark(main) if tr is not None else None
            fn()
            if tr is not None:
                tr["product"].append((t_a, mark(main)))

        if self.exchange == "needed":
            main.wait_event(events[0])
            product(lambda: self.local_spmm(out, recv, self.rowPtr, self.colIdx, self.val))
        elif self.exchange == "needed_rowgroups":
            for kk in range(self.row_chunks):
                main.wait_event(events[kk])  # fetches are in stream order: 0..kk have arrived
                r0, r1 = self.group_bounds[kk], self.group_bounds[kk + 1]
                if r1 > r0:
                    rp, ci, v = self.blocks[kk]
                    product(lambda: self.block_spmm[kk](out[r0:r1], recv, rp, ci, v))
        else:
            for kk in range(self.row_chunks):
                main.wait_event(events[kk])
                rp, ci, v = self.blocks[kk]
                product(lambda: self.block_spmm[kk](out, recv, rp, ci, v, accumulate=kk > 0))
        # a producer on the main stream may overwrite the block only after the closing fence
        main.wait_stream(side)
        if tr is not None:
            tr["end"] = mark(main)
            self._trace_events = tr
        return out

    def trace_result(self):
        """Milliseconds from the start of the last traced pull-transport call (``trace = True``):
        [begin, end] of every fetch and of every product, and the end of the call.  Synchronises."""
        tr = getattr(self, "_trace_events", None)
        if tr is None:
            return None
        torch.cuda.synchronize()
        rel = lambda e: round(tr["start"].elapsed_time(e), 3)
        return {"fetch_ms": [[rel(a), rel(b)] for a, b in tr["fetch"]],
                "product_ms": [[rel(a), rel(b)] for a, b in tr["product"]],
                "end_ms": rel(tr["end"]), "rows_per_fetch": [c[1] for c in self.chunk_plan]}

    def _forward_copy_engine(self, B_shard, out):
        import torch.distributed as dist

        K, W, cr = self.row_chunks, self.world, self.chunk_rows
        rows, dim = B_shard.shape
        src, peers, fence = self._peer_blocks(dim, B_shard)
        full = self._receive_buffer(K * W * cr, dim, B_shard)
        main = torch.cuda.current_stream()
        events = []
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            if B_shard.data_ptr() != src.data_ptr():
                src[:rows].copy_(B_shard)
            dist.all_reduce(fence, group=self.group)  # every block is in place
            # Pulls from different peers go to different streams, so several copy engines (and
            # NVLink paths) are busy at once; a chunk is complete when all of them are.
            lanes = [self._side] + self._pull_streams
            for st in self._pull_streams:
                st.wait_stream(self._side)
            for kk in range(K):
                for i in range(W):
                    q = (self.rank + i) % W  # own chunk first, then the peers round-robin
                    with torch.cuda.stream(lanes[i % len(lanes)]):
                        full[(kk * W + q) * cr: (kk * W + q + 1) * cr].copy_(peers[q][kk * cr: (kk + 1) * cr])
                for st in self._pull_streams:
                    self._side.wait_stream(st)
                ev = torch.cuda.Event()
                ev.record(self._side)
                events.append(ev)
            dist.all_reduce(fence, group=self.group)  # every peer has finished reading this block
        B_shard.record_stream(self._side)
        for kk in range(K):
            main.wait_event(events[kk])
            rp, ci, v = self.blocks[kk]
            self.block_spmm[kk](out, full, rp, ci, v, accumulate=kk > 0)
        # a producer on the main stream may overwrite the block only after the closing fence
        main.wait_stream(self._side)
        return out

    def _forward_pipelined(self, B_shard, out):
        import torch.distributed as dist

        if self.transport == "copy_engine":
            if self._side is None or self.world == 1:
                raise ValueError("the copy-engine transport needs CUDA devices and at least two ranks")
            return self._forward_copy_engine(B_shard, out)

        K, W, cr = self.row_chunks, self.world, self.chunk_rows
        rows, dim = B_shard.shape
        full = self._receive_buffer(K * W * cr, dim, B_shard)
        cuda = self._side is not None
        main = torch.cuda.current_stream() if cuda else None
        events = []

        def gather(kk):
            lo, hi = min(kk * cr, rows), min((kk + 1) * cr, rows)
            piece = B_shard[lo:hi]
            if hi - lo != cr:  # the ragged end of a block (or a block shorter than the longest one)
                padded = torch.zeros(cr, dim, dtype=B_shard.dtype, device=B_shard.device)
                padded[: hi - lo] = piece
                piece = padded
            dst = full[kk * W * cr: (kk + 1) * W * cr]
            if W == 1:
                dst.copy_(piece)
            else:
                dist.all_gather_into_tensor(dst, piece, group=self.group)

        if cuda:
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                for kk in range(K):
                    gather(kk)
                    ev = torch.cuda.Event()
                    ev.record(self._side)
                    events.append(ev)
            B_shard.record_stream(self._side)
        for kk in range(K):
            if cuda:
                main.wait_event(events[kk])
            else:
                gather(kk)
            rp, ci, v = self.blocks[kk]
            self.block_spmm[kk](out, full, rp, ci, v, accumulate=kk > 0)
        return out

    def _plan_needed_rows(self, cols_global):
        """Set-up of the sparse exchange: which rows this rank needs from every owner, which rows
        every other rank needs from this one, and the local column ids renumbered to positions in
        the receive buffer (rows arrive grouped by owner, ascending inside a group, i.e. in the
        order of the sorted distinct column ids)."""
        import torch.distributed as dist

        dev = cols_global.device
        need = torch.unique(cols_global.long())  # sorted distinct global column ids
        cb = self.col_bounds.to(dev)
        cuts = torch.searchsorted(need, cb)  # need[cuts[q]:cuts[q+1]] is owned by rank q
        recv_counts = (cuts[1:] - cuts[:-1]).cpu()
        owner = torch.repeat_interleave(torch.arange(self.world, device=dev), recv_counts.to(dev))
        wanted = (need - cb[owner]).to(torch.int64)  # row ids inside the owners' shards
        self.colIdx = torch.searchsorted(need, cols_global.long()).to(torch.int32)
        self.n_needed = int(need.numel())
        self.recv_splits = [int(x) for x in recv_counts]
        if self.transport == "pull":  # the reader addresses the owners' blocks itself: nothing to request
            self.chunk_rows = self.max_rows
            self.chunk_plan = [(0, self.n_needed, self.recv_splits, None, wanted.to(torch.int32))]
            return
        if self.world == 1:
            self.send_splits, self.send_rows = list(self.recv_splits), wanted
            return
        counts_out = torch.empty(self.world, dtype=torch.int64, device=dev)
        dist.all_to_all_single(counts_out, recv_counts.to(dev), group=self.group)
        self.send_splits = [int(x) for x in counts_out.cpu()]
        self.send_rows = torch.empty(sum(self.send_splits), dtype=torch.int64, device=dev)
        dist.all_to_all_single(self.send_rows, wanted, output_split_sizes=self.send_splits,
                               input_split_sizes=self.recv_splits, group=self.group)

    def _exchange_needed(self, B_shard):
        """Rows of the dense operand this rank's columns reference, in receive-buffer order."""
        import torch.distributed as dist

        send = B_shard.index_select(0, self.send_rows)
        if self.world == 1:
            return send
        recv = torch.empty(self.n_needed, B_shard.shape[1], dtype=B_shard.dtype, device=B_shard.device)
        dist.all_to_all_single(recv, send, output_split_sizes=self.recv_splits,
                               input_split_sizes=self.send_splits, group=self.group)
        return recv

    def local_block(self):
        """(rowPtr, global column ids, values) of this rank's rows, for building further operators
        over the same shard without extracting it again (needs keep_global_columns())."""
        return self.rowPtr, self._colIdx_global, self.val

    def pull_lists(self):
        """Per chunk of the pull transport: (position of the chunk in the compact operand, list
        positions where each owner's rows start, row ids inside the owners' blocks)."""
        out = []
        for base, cnt, recv_splits, _, want_rows in self.chunk_plan:
            first = [0]
            for c in recv_splits:
                first.append(first[-1] + c)
            out.append((base, first, want_rows))
        return out

    def _planned_spmm(self, rowPtr=None):
        """The CUDA operator with the configuration the decider picks for the row-length statistics
        of this shard (or of one column block of it) and the (slice of the) dense width; a split
        layout, when chosen, is built once on the device from the row pointer and kept."""
        from . import decider

        stats = decider.row_stats(self.rowPtr if rowPtr is None else rowPtr)
        bound = {}

        def local_spmm(out, B, rowPtr, colIdx, val, accumulate=False):
            p = decider.choose(stats, B.shape[1])
            # (a bucketed plan permutes the entries, so it belongs to one column / value array pair)
            key = (int(p["if_split"]), p.get("granularity"), int(p.get("bucketed", 0)), colIdx.data_ptr(), val.data_ptr())
            if key not in bound:  # layout arrays of this plan, built once on the device and kept
                bound[key] = decider.PlannedSpMM(p, rowPtr, colIdx, val)
            op = bound[key]
            op.plan = p
            return op(out, B, accumulate=accumulate)

        return local_spmm

    @property
    def local_rows(self):
        return self.hi - self.lo

    def _gather(self, shard_slice):
        """Padded all-gather of one [rows, d] block of the dense operand -> [world*max_rows, d]."""
        import torch.distributed as dist

        rows, d = shard_slice.shape
        padded = shard_slice
        if rows != self.max_rows or not shard_slice.is_contiguous():
            padded = torch.zeros(self.max_rows, d, dtype=shard_slice.dtype, device=shard_slice.device)
            padded[:rows] = shard_slice
        full = torch.empty(self.world * self.max_rows, d, dtype=shard_slice.dtype, device=shard_slice.device)
        if self.world == 1:
            full.copy_(padded)
        else:
            dist.all_gather_into_tensor(full, padded, group=self.group)
        return full

    def forward(self, B_shard, out=None):
        """B_shard: this rank's rows [col_bounds[rank], col_bounds[rank+1]) of the dense operand.
        Returns this rank's rows of C = A B."""
        if B_shard.shape[0] != self.my_cols[1] - self.my_cols[0]:
            raise ValueError("dense shard has %d rows, expected %d" % (B_shard.shape[0], self.my_cols[1] - self.my_cols[0]))
        dim = B_shard.shape[1]
        if out is None:
            out = torch.empty(self.local_rows, dim, dtype=B_shard.dtype, device=B_shard.device)
        if self.transport == "pull":
            if dim % 4 != 0 or self._side is None:
                raise ValueError("the pull transport needs CUDA devices and a dim that is a multiple of 4")
            return self._forward_pull(B_shard, out)
        if self.exchange == "needed":
            self.local_spmm(out, self._exchange_needed(B_shard), self.rowPtr, self.colIdx, self.val)
            return out
        if self.exchange in ("pipelined", "needed_pipelined"):
            if dim % 4 != 0:
                raise ValueError("the pipelined exchange adds into C with 128-bit accesses: dim must be a multiple of 4")
            if self.exchange == "pipelined":
                return self._forward_pipelined(B_shard, out)
            return self._forward_needed_pipelined(B_shard, out)
        k = max(1, min(self.dim_chunks, dim // 4)) if self.dim_chunks > 1 else 1
        if k == 1:
            self.local_spmm(out, self._gather(B_shard), self.rowPtr, self.colIdx, self.val)
            return out
        # dim slices, multiples of 4 columns so that 128-bit loads stay possible
        step = ((dim + k - 1) // k + 3) // 4 * 4
        slices = [(c0, min(dim, c0 + step)) for c0 in range(0, dim, step)]
        main = torch.cuda.current_stream()
        gathered, events = [None] * len(slices), [None] * len(slices)

        def issue(i):
            c0, c1 = slices[i]
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                gathered[i] = self._gather(B_shard[:, c0:c1])
                events[i] = torch.cuda.Event()
                events[i].record(self._side)

        issue(0)
        for i, (c0, c1) in enumerate(slices):
            if i + 1 < len(slices):
                issue(i + 1)
            main.wait_event(events[i])
            self.local_spmm(out[:, c0:c1], gathered[i], self.rowPtr, self.colIdx, self.val)
            gathered[i].record_stream(main)
        return out

    def forward_replicated(self, B_full, out=None):
        """SpMM against a dense operand every rank already holds in full (no exchange)."""
        if out is None:
            out = torch.empty(self.local_rows, B_full.shape[1], dtype=B_full.dtype, device=B_full.device)
        if not hasattr(self, "_colIdx_global"):
            raise RuntimeError("call keep_global_columns() at set-up to use a replicated operand")
        self.local_spmm(out, B_full, self.rowPtr, self._colIdx_global, self.val)
        return out

    def keep_global_columns(self, colIdx_global_shard):
        self._colIdx_global = colIdx_global_shard.to(self.device)
        return self
