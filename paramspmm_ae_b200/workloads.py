"""Timed runs of the secondary benchmark configurations (the primary one, the dim sweep on
10^6-row matrices, lives in bench.py).  Each function builds its seeded synthetic input on the
device, checks the result against an independent computation, and returns a dict of timings.

* ``agnn_layer``   232,965-node power-law graph with ~114.6 M stored entries (average degree ~490),
                   64 L2-normalised features: SDDMM on the pattern, scale by beta, SpMM with the
                   edge scores as values.  The reference's layer (gnn_conv.py:130-151) has no edge
                   softmax; ``softmax=True`` adds the per-row softmax the configuration text
                   describes, computed with torch segment ops between the two kernels.
* ``gcn_forward_backward``  3-layer GCN (100 -> 256 -> 256 -> 47) forward and backward on a
                   2,449,029-node power-law graph through the drop-in ParamSpCONV operators.
"""
from __future__ import annotations

import sys
import time

import torch

from . import baselines, decider, ops, synth


def _time_ms(fn, warmup=3, iters=10):
    for _ in range(warmup):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b) / iters


def sample_rows(rowPtr, count=32, seed=0):
    """Row ids worth checking: the longest rows (hubs), the last rows that hold entries (largest
    output offsets), the first row, and a seeded random draw."""
    rp = rowPtr.long()
    ln = rp[1:] - rp[:-1]
    n = ln.numel()
    k = max(1, count // 4)
    g = torch.Generator(device="cpu").manual_seed(seed)
    nonempty = torch.nonzero(ln > 0).flatten()
    picks = [torch.topk(ln, min(k, n)).indices.cpu(), nonempty[-k:].cpu(), torch.tensor([0, n - 1]),
             torch.randint(0, n, (count - 2 * k,), generator=g)]
    return torch.unique(torch.cat(picks))


def check_rows_fp64(rowPtr, colIdx, val, B, out, rows, what="spmm"):
    """Compare the sampled rows of out = A B with dense fp64 algebra (one gather and one matrix-vector
    product per row, 64-bit indices throughout, nothing shared with the kernels).  Tolerance: 1e-5
    relative plus an absolute floor of 1e-4 that grows with the row's length beyond 256 entries
    (fp32 re-association over L terms).  Returns the largest error in units of the bound."""
    worst = 0.0
    for r in rows.tolist():
        a, b = int(rowPtr[r]), int(rowPtr[r + 1])
        want = (val[a:b].double()[None, :] @ B[colIdx[a:b].long()].double())[0]
        got = out[r].double()
        bound = 1e-5 * want.abs() + 1e-4 * max(1.0, (b - a) / 256.0)
        ratio = float(((got - want).abs() / bound).max()) if b > a else float(got.abs().max())
        if not ratio <= 1.0:
            raise AssertionError("%s: row %d (%d entries) is off by %.3g times the bound" % (what, r, b - a, ratio))
        worst = max(worst, ratio)
    return worst


def agnn_layer(n=232_965, pairs=57_180_000, dim=64, seed=41, iters=10, grans=(0, 128, 512, 1024, 2048, 4096), device="cuda:0"):
    dev = torch.device(device)
    t0 = time.time()
    g = synth.powerlaw_graph(n, pairs, seed=seed, device=dev, normalize=False)
    gen_s = time.time() - t0
    X = synth.dense_normal(n, dim, seed + 1, dev)
    X = X / X.norm(dim=1, keepdim=True)
    beta = 1.0
    nnz = g.nnz
    out = {"n": n, "nnz": nnz, "dim": dim, "avg_degree": nnz / n, "generate_s": round(gen_s, 1)}

    # correctness on a row sample against dense algebra in fp64
    rows = torch.randint(0, n, (64,), device=dev)
    e_full = ops.csr_sddmm(X, X, g.rowPtr, g.colIdx, g.val, 2, 8)
    for r in rows.tolist()[:16]:
        a, b = int(g.rowPtr[r]), int(g.rowPtr[r + 1])
        want = (X[g.colIdx[a:b].long()].double() @ X[r].double())
        torch.testing.assert_close(e_full[a:b].double(), want, rtol=1e-5, atol=1e-4)

    layouts = {}
    for gran in grans:
        if gran:
            rps, tr = ops.split_csr(g.rowPtr.cpu(), gran)
            layouts[gran] = (rps.to(dev), tr.to(dev))
    res = []
    for gran in grans:
        rp, tr = (g.rowPtr, None) if not gran else layouts[gran]
        cf = (dim + 31) // 32
        if tr is None:
            sd = lambda: ops.csr_sddmm(X, X, rp, g.colIdx, g.val, cf, 8)
        else:
            sd = lambda: ops.csr_split_sddmm(X, X, rp, g.colIdx, g.val, tr, cf, 8)
        ms_sd = _time_ms(sd, iters=iters)
        e = sd() * beta
        C = torch.empty(n, dim, device=dev)
        sp = lambda: ops.spmm_into(C, X, rp, g.colIdx, e, target_row=tr, n_out_rows=n)
        ms_sp = _time_ms(sp, iters=iters)
        res.append({"granularity": gran or None, "sddmm_ms": round(ms_sd, 4), "spmm_ms": round(ms_sp, 4),
                    "sddmm_gflops": round(2.0 * nnz * dim / ms_sd / 1e6, 1),
                    "spmm_gflops": round(2.0 * nnz * dim / ms_sp / 1e6, 1)})
    out["kernels"] = res
    best_sd = min(r["sddmm_ms"] for r in res)
    best_sp = min(r["spmm_ms"] for r in res)
    by_sd = 4 * (n + 1) + 8 * nnz + 8 * dim * n
    by_sp = 4 * (n + 1) + 8 * nnz + 8 * dim * n
    out["bytes_model"] = {"sddmm": by_sd, "spmm": by_sp, "sddmm_gbs": round(by_sd / best_sd / 1e6, 1),
                          "spmm_gbs": round(by_sp / best_sp / 1e6, 1),
                          "gather_bytes": 4 * dim * nnz,
                          "sddmm_gather_gbs": round(4 * dim * nnz / best_sd / 1e6, 1),
                          "spmm_gather_gbs": round(4 * dim * nnz / best_sp / 1e6, 1)}
    # comparators
    try:
        vals = g.val.clone()
        plan = baselines.sddmm_plan(X, X, g.rowPtr, g.colIdx, vals)
        out["cusparse_sddmm_ms"] = round(baselines.time_plan_ms(plan, 2, iters), 4)
        plan.close()
        torch.testing.assert_close(vals, e_full, rtol=1e-4, atol=1e-4)
        C2 = torch.empty(n, dim, device=dev)
        plan = baselines.spmm_plan(0, g.rowPtr, g.colIdx, e_full, X, C2)
        out["cusparse_spmm_ms"] = round(baselines.time_plan_ms(plan, 2, iters), 4)
        plan.close()
        Cn = torch.empty(n, dim, device=dev)
        ops.spmm_into(Cn, X, g.rowPtr, g.colIdx, e_full)
        scale = float(C2.abs().max())
        torch.testing.assert_close(Cn, C2, rtol=1e-4, atol=1e-5 * max(1.0, scale))
    except Exception as ex:  # comparator trouble must not hide the kernel numbers
        out["cusparse_error"] = "%s: %s" % (type(ex).__name__, ex)
    # the full layer (SDDMM, scale by beta, SpMM) on the fastest split layout
    gbest = min((r for r in res if r["granularity"]), key=lambda r: r["sddmm_ms"] + r["spmm_ms"])["granularity"]
    rps, tr = layouts[gbest]
    Cl = torch.empty(n, dim, device=dev)
    layer = lambda: ops.spmm_into(Cl, X, rps, g.colIdx,
                                  ops.csr_split_sddmm(X, X, rps, g.colIdx, g.val, tr, 2, 8) * beta,
                                  target_row=tr, n_out_rows=n)
    out["layer_granularity"] = gbest
    out["layer_sddmm_scale_spmm_ms"] = round(_time_ms(layer, iters=iters), 4)
    # the same layer as ONE kernel (scores, optional edge softmax and aggregation in a single pass)
    fused = []
    want = Cl.clone()
    for gran in grans:
        if not gran:
            continue
        rps, tr = layouts[gran]
        Cf = torch.empty(n, dim, device=dev)
        for vw, lanes, batch in ((4, 16, 8), (4, 4, 4), (8, 8, 4), (8, 8, 8), (8, 4, 4), (0, 0, 0)):
            if gran != 2048 and (vw, lanes, batch) != (0, 0, 0):
                continue  # the shape comparison on one partition length only
            f_plain = lambda: ops.agnn_fused(X, X, rps, g.colIdx, beta, False, target_row=tr, n_out_rows=n,
                                             out=Cf, batch=batch, lanes_per_row=lanes, vec_width=vw)
            ms_plain = _time_ms(f_plain, iters=iters)
            f_plain()
            scale = float(want.abs().max())
            torch.testing.assert_close(Cf, want, rtol=1e-4, atol=1e-5 * max(1.0, scale))
            f_soft = lambda: ops.agnn_fused(X, X, rps, g.colIdx, beta, True, target_row=tr, n_out_rows=n,
                                            out=Cf, batch=batch, lanes_per_row=lanes, vec_width=vw)
            ms_soft = _time_ms(f_soft, iters=iters)
            fused.append({"granularity": gran, "vec_width": vw, "lanes_per_row": lanes, "batch": batch, "fused_ms": round(ms_plain, 4),
                          "fused_softmax_ms": round(ms_soft, 4)})
    out["fused"] = fused
    out["fused_best_ms"] = min(f["fused_ms"] for f in fused)
    out["fused_softmax_best_ms"] = min(f["fused_softmax_ms"] for f in fused)
    # One training step of the layer (projection, propagation, backward to the input, the weights and
    # the attention weight): the reference's three-kernel composition, which writes the attention
    # values and the score gradient per edge, against the fused function, which writes neither.
    from . import gnn_conv, pcsr
    gfast = min((f for f in fused if (f["vec_width"], f["lanes_per_row"], f["batch"]) == (0, 0, 0)),
                key=lambda f: f["fused_ms"])["granularity"]
    rps, tr = layouts[gfast]
    P = pcsr.pcsr_sddmm(None, 1, True, n, nnz, rps, g.colIdx, g.val, tr, CF=(dim + 31) // 32, blkWarpNum=8)
    torch.manual_seed(seed + 5)
    conv = gnn_conv.AGNNConv(dim, dim).to(dev)
    col = g.colIdx.unsqueeze(-1)
    Gup = synth.dense_normal(n, dim, seed + 6, dev)
    Xin = X.clone().requires_grad_(True)

    def train_step():
        for p_ in conv.parameters():
            p_.grad = None
        Xin.grad = None
        conv(Xin, {dim: P}, col).backward(Gup)

    steps = {}
    old = gnn_conv.FUSE_AGNN_TRAINING
    try:
        for label, flag in (("three_kernels", False), ("fused", True)):
            gnn_conv.FUSE_AGNN_TRAINING = flag
            torch.cuda.reset_peak_memory_stats()
            base = torch.cuda.memory_allocated()
            steps[label + "_ms"] = round(_time_ms(train_step, warmup=2, iters=iters), 4)
            steps[label + "_peak_extra_bytes"] = int(torch.cuda.max_memory_allocated() - base)
            steps[label + "_grads"] = [Xin.grad.clone(), conv.weights.grad.clone()]
    finally:
        gnn_conv.FUSE_AGNN_TRAINING = old
    for a_, b_ in zip(steps.pop("three_kernels_grads"), steps.pop("fused_grads")):
        scale = float(a_.abs().max())
        torch.testing.assert_close(b_, a_, rtol=1e-4, atol=1e-5 * max(1.0, scale))
    # the backward product alone (scores recomputed, gradient rows gathered) at both load widths
    Xp = torch.mm(X, conv.weights.detach())
    Dout = torch.empty(n, dim, device=dev)
    for vw in (4, 8):
        steps["backward_product_vw%d_ms" % vw] = round(_time_ms(
            lambda: ops.agnn_fused(Xp, Xp, rps, g.colIdx, beta, False, target_row=tr, n_out_rows=n, out=Dout, V=Gup,
                                   vec_width=vw), iters=iters), 4)
    Tout = torch.empty(n, dim, device=dev)
    steps["pattern_spmm_ms"] = round(_time_ms(lambda: ops.spmm_into(Tout, Gup, rps, g.colIdx, None, target_row=tr,
                                                                    n_out_rows=n), iters=iters), 4)
    out["layer_training_step"] = dict(steps, granularity=gfast)
    return out


def gcn_forward_backward(n=2_449_029, pairs=61_900_000, feats=100, hidden=256, classes=47, seed=31, iters=3,
                         device="cuda:0"):
    """3-layer GCN forward + backward through ParamSpCONV's operators (fp32, random weights and labels)."""
    from . import gnn_conv, pcsr
    dev = torch.device(device)
    t0 = time.time()
    g = synth.powerlaw_graph(n, pairs, seed=seed, device=dev)
    gen_s = time.time() - t0
    stats = decider.row_stats(g.rowPtr, g.colIdx)
    dims = [hidden, hidden, classes]
    # Two sets of operators: the legacy tuple form the reference's GNN.py builds (layout chosen by
    # the decider, library-default kernel parameters), and operators bound to the decider's plan
    # (the table's kernel parameters and the length-bucketed plan where it names it).
    legacy_by_dim, ops_by_dim = {}, {}
    for d in set(dims):
        plan = decider.choose(stats, d)
        if plan["if_split"]:
            rps, tr = ops.split_csr(g.rowPtr.cpu(), plan["granularity"])
            legacy_by_dim[d] = pcsr.pcsr_spmm(None, 1, True, n, g.nnz, rps, g.colIdx, g.val, tr, CF=1, blkWarpNum=8)
        else:
            legacy_by_dim[d] = pcsr.pcsr_spmm(None, 1, False, n, g.nnz, g.rowPtr, g.colIdx, g.val, None, CF=1, blkWarpNum=8)
        ops_by_dim[d] = pcsr.pcsr_spmm.from_plan(plan, g.rowPtr, g.colIdx, g.val)
    torch.manual_seed(seed + 2)
    layers = [gnn_conv.GCNConv(a, b).to(dev) for a, b in zip([feats, hidden, hidden], dims)]
    X = synth.dense_normal(n, feats, seed + 1, dev)
    y = torch.randint(0, classes, (n,), device=dev, generator=torch.Generator(device=dev).manual_seed(seed + 3))

    def step(operators=None):
        h = X
        for i, l in enumerate(layers):
            h = l(h, operators or ops_by_dim)
            if i < 2:
                h = torch.relu(h)
        loss = torch.nn.functional.cross_entropy(h, y)
        for l in layers:
            l.weights.grad = None
        loss.backward()
        return loss

    # Independent check before timing: sampled rows (hub rows, the last rows, random ones) of the
    # aggregation at every width the step uses, and of the first layer's output A (X W1), against
    # dense fp64 algebra.
    rows = sample_rows(g.rowPtr, 32, seed)
    checked = {}
    for d in sorted(set(dims)):
        Z = synth.dense_normal(n, d, seed + 7 + d, dev)
        checked["spmm_dim%d" % d] = round(check_rows_fp64(g.rowPtr, g.colIdx, g.val, Z, ops_by_dim[d].GIN_spmm(Z)[:n],
                                                          rows, "aggregation at width %d" % d), 3)
    with torch.no_grad():
        out1 = layers[0](X, ops_by_dim)
        XW = (X.double() @ layers[0].weights.detach().double())
        checked["layer1"] = round(check_rows_fp64(g.rowPtr, g.colIdx, g.val, XW, out1, rows, "first GCN layer"), 3)
        del XW, out1

    def timed(reorder, operators=None):
        old = gnn_conv.REORDER_NARROW_FIRST
        gnn_conv.REORDER_NARROW_FIRST = reorder
        try:
            run = lambda: step(operators)
            return _time_ms(run, warmup=1, iters=iters), float(run())
        finally:
            gnn_conv.REORDER_NARROW_FIRST = old

    ms_legacy, loss_legacy = timed(False, legacy_by_dim)  # the reference's operation order, A (H W), legacy operators
    ms, loss = timed(False)            # the same order on the plan-bound operators
    ms_reorder, loss_reorder = timed(True)   # widening layers aggregate first, (A H) W

    # Where a step's time goes: the aggregation alone at each width (legacy and plan-bound), the
    # class-count width with and without the padding to a multiple of 4, and the dense products.
    parts = {}
    for d in sorted(set(dims)):
        Z = synth.dense_normal(n, d, seed + 7 + d, dev)
        parts["spmm_dim%d_legacy_ms" % d] = round(_time_ms(lambda: legacy_by_dim[d].GIN_spmm(Z), warmup=2, iters=5), 3)
        parts["spmm_dim%d_planned_ms" % d] = round(_time_ms(lambda: ops_by_dim[d].GIN_spmm(Z), warmup=2, iters=5), 3)
        if d % 4:
            Zp = torch.nn.functional.pad(Z, (0, -d % 4))
            parts["spmm_dim%d_legacy_padded_ms" % d] = round(_time_ms(lambda: legacy_by_dim[d].GIN_spmm(Zp), warmup=2, iters=5), 3)
        del Z
    H1 = synth.dense_normal(n, hidden, seed + 5, dev)

    def dense_products():
        for a, b in zip([feats, hidden, hidden], dims):
            w = torch.empty(a, b, device=dev)
            h = X if a == feats else H1
            torch.mm(h, w)                                   # forward H W
            gz = H1[:, :b] if b != hidden else H1
            if a != feats:
                torch.mm(gz, w.t())                          # dH = AG W^T (not formed for the first layer)
            torch.mm(h.t(), gz)                              # dW = H^T AG
    parts["dense_products_ms"] = round(_time_ms(dense_products, warmup=1, iters=3), 3)
    del H1
    spmm_flops = 2.0 * g.nnz * (sum(dims) * 2)  # one SpMM per layer forward, one backward
    return {"n": n, "nnz": g.nnz, "generate_s": round(gen_s, 1), "ms_per_step": round(ms, 2),
            "ms_per_step_legacy_operators": round(ms_legacy, 2), "loss_legacy_operators": loss_legacy,
            "ms_per_step_narrow_first": round(ms_reorder, 2), "loss": loss, "loss_narrow_first": loss_reorder,
            "parts": parts,
            "spmm_gflop_per_step": round(spmm_flops / 1e9, 1), "regime": decider.regime(stats),
            "fp64_row_checks_worst_error_over_bound": checked, "rows_checked": int(rows.numel())}


def scaleout_spmm(scale=24, nnz=512_000_000, dim=128, seed=51, iters=5, warmup=2, rank=0, world=1,
                  device="cuda:0", dim_chunks=4, row_chunks=4):
    """Row-sharded SpMM of one global R-MAT matrix (strong scaling): every rank holds a contiguous,
    nnz-balanced row block of A and the matching row block of the dense operand.

    Timings per rank (CUDA events on the launching stream, maximum over ranks):
    the local SpMM against a replicated dense operand (no exchange), the all-gather of the dense
    row blocks followed by the SpMM, the exchange of only the rows each shard references (one
    all-to-all) followed by the SpMM on the compact operand, the all-gather in `row_chunks` row
    chunks with the product of column block k running while chunk k+1 is on the wire (for all rows
    over NCCL, for all rows pulled by the copy engines from peer-mapped memory, and for the referenced
    rows only), and the
    all-gather with the dense columns cut into `dim_chunks` slices so that the gather of slice s+1
    overlaps the SpMM of slice s.
    Every rank generates the same global matrix from the seed and keeps only its rows.
    """
    import torch.distributed as dist
    from .shard import ShardedSpMM

    dev = torch.device(device)
    t0 = time.time()
    m = synth.rmat(scale, nnz, seed=seed, device=dev)
    gen_s = time.time() - t0
    n = m.n_rows
    sh = ShardedSpMM(m.rowPtr, m.colIdx, m.val, n, rank, world, device=dev, dim_chunks=1)
    a, b = int(m.rowPtr[sh.lo]), int(m.rowPtr[sh.hi])
    sh.keep_global_columns(m.colIdx[a:b].clone())
    sh_needed = ShardedSpMM(m.rowPtr, m.colIdx, m.val, n, rank, world, device=dev, exchange="needed")
    sh_pipe = ShardedSpMM(m.rowPtr, m.colIdx, m.val, n, rank, world, device=dev, exchange="pipelined",
                          row_chunks=row_chunks)
    sh_ce = None
    if world > 1:
        sh_ce = ShardedSpMM(m.rowPtr, m.colIdx, m.val, n, rank, world, device=dev, exchange="pipelined",
                            row_chunks=row_chunks, transport="copy_engine")
    sh_np = ShardedSpMM(m.rowPtr, m.colIdx, m.val, n, rank, world, device=dev, exchange="needed_pipelined",
                        row_chunks=row_chunks)
    nnz_total, nnz_local = m.nnz, b - a
    del m
    torch.cuda.empty_cache()
    B_full = synth.dense_uniform(n, dim, seed + 1, dev)
    c0, c1 = sh.my_cols
    B_shard = B_full[c0:c1].clone()
    out_rep = torch.empty(sh.local_rows, dim, device=dev)
    out_ag = torch.empty(sh.local_rows, dim, device=dev)

    def timed(fn, label):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:  # progress on stderr: a later step that fails does not take these along
            print("scaleout_spmm world %d: %s %.4f ms" % (world, label, float(t.item())), file=sys.stderr, flush=True)
        return float(t.item())

    ms_rep = timed(lambda: sh.forward_replicated(B_full, out_rep), "replicated")
    # Independent check of the product every other form is compared with: sampled local rows (the
    # shard's hub rows, its last rows, whose output offsets are the largest, random ones) against
    # dense fp64 algebra with 64-bit indexing.  At 2^24 rows and dim 128 the output holds 2^31
    # elements: the last rows sit at byte offsets beyond 2^32 and at element offsets up to 2^31 - 1.
    rows = sample_rows(sh.rowPtr, 40, seed)
    fp64_worst = check_rows_fp64(sh.rowPtr, sh._colIdx_global, sh.val, B_full, out_rep, rows,
                                 "row shard %d of %d" % (rank, world))
    fp64_max_offset = int(rows.max()) * dim
    ms_ag = timed(lambda: sh.forward(B_shard, out_ag), "allgather")
    # Hub rows of this matrix sum 10^5 and more terms, and the pieces of a split row arrive in a
    # different order on every launch (REDs): the comparison allows for fp32 re-association.
    tol = dict(rtol=1e-4, atol=2e-3)
    torch.testing.assert_close(out_ag, out_rep, **tol)
    out_ag.fill_(float("nan"))
    ms_needed = timed(lambda: sh_needed.forward(B_shard, out_ag), "needed rows")
    torch.testing.assert_close(out_ag, out_rep, **tol)
    # the three legs of that form alone: pack (gather into a send buffer), all-to-all, product
    legs = {}
    legs["pack_ms"] = timed(lambda: B_shard.index_select(0, sh_needed.send_rows), "  needed: pack alone")
    send_buf = B_shard.index_select(0, sh_needed.send_rows)
    recv_buf = torch.empty(sh_needed.n_needed, dim, device=dev)
    if world > 1:
        legs["all_to_all_ms"] = timed(lambda: dist.all_to_all_single(recv_buf, send_buf, output_split_sizes=sh_needed.recv_splits,
                                                                     input_split_sizes=sh_needed.send_splits), "  needed: all-to-all alone")
    else:
        recv_buf.copy_(send_buf)
    legs["product_ms"] = timed(lambda: sh_needed.local_spmm(out_ag, recv_buf, sh_needed.rowPtr, sh_needed.colIdx, sh_needed.val),
                               "  needed: product alone")
    legs["bytes_received"] = int(sh_needed.n_needed) * dim * 4
    del send_buf, recv_buf
    out_ag.fill_(float("nan"))
    ms_pipe = timed(lambda: sh_pipe.forward(B_shard, out_ag), "pipelined row chunks")
    torch.testing.assert_close(out_ag, out_rep, **tol)
    sh.dim_chunks = dim_chunks
    sh._side = torch.cuda.Stream()
    out_ag.fill_(float("nan"))
    ms_ov = timed(lambda: sh.forward(B_shard, out_ag), "dim slices")
    torch.testing.assert_close(out_ag, out_rep, **tol)
    out_ag.fill_(float("nan"))
    ms_np = timed(lambda: sh_np.forward(B_shard, out_ag), "needed rows in pipelined row chunks")
    torch.testing.assert_close(out_ag, out_rep, **tol)
    ms_ce = None
    if sh_ce is not None:
        B_sym = sh_ce.symmetric_input(dim)  # the dense block lives in peer-mapped memory, as a producer would leave it
        B_sym.copy_(B_shard)
        out_ag.fill_(float("nan"))
        ms_ce = timed(lambda: sh_ce.forward(B_sym, out_ag), "pipelined row chunks, copy engines")
        torch.testing.assert_close(out_ag, out_rep, **tol)
    gf = lambda ms: 2.0 * nnz_total * dim / ms / 1e6
    by = 4 * (n + 1) + 8 * nnz_total + 4 * dim * n * 2
    return {"n": n, "nnz": nnz_total, "nnz_local": nnz_local, "rows_local": sh.local_rows, "dim": dim,
            "generate_s": round(gen_s, 1), "world": world,
            "spmm_replicated_ms": round(ms_rep, 4), "allgather_spmm_ms": round(ms_ag, 4),
            "allgather_overlapped_ms": round(ms_ov, 4), "dim_chunks": dim_chunks,
            "allgather_pipelined_ms": round(ms_pipe, 4), "row_chunks": row_chunks,
            "allgather_pipelined_gflops": round(gf(ms_pipe), 1),
            "copy_engine_pipelined_ms": None if ms_ce is None else round(ms_ce, 4),
            "copy_engine_pipelined_gflops": 0.0 if ms_ce is None else round(gf(ms_ce), 1),
            "needed_rows_pipelined_ms": round(ms_np, 4), "needed_rows_pipelined_gflops": round(gf(ms_np), 1),
            "needed_rows_exchange_spmm_ms": round(ms_needed, 4),
            "needed_rows_exchange_spmm_gflops": round(gf(ms_needed), 1),
            "needed_rows_fraction": round(sh_needed.n_needed / n, 4), "needed_legs": {k: round(v, 4) for k, v in legs.items()},
            "spmm_replicated_gflops": round(gf(ms_rep), 1), "allgather_spmm_gflops": round(gf(ms_ag), 1),
            "allgather_overlapped_gflops": round(gf(ms_ov), 1),
            "compulsory_bytes_global": by, "spmm_replicated_gbs_global": round(by / ms_rep / 1e6, 1),
            "fp64_rows_checked": int(rows.numel()), "fp64_worst_error_over_bound": round(fp64_worst, 3),
            "fp64_largest_checked_element_offset": fp64_max_offset}


def scaleout_brief(scale=24, nnz=512_000_000, dim=128, seed=51, iters=5, warmup=2, rank=0, world=1,
                   device="cuda:0", row_chunks=(8, 16), labels="natural", legs=True):
    """The three strong-scaling curves of the row-sharded SpMM that the benchmark line carries at
    every GPU count (same global R-MAT matrix and dense operand as :func:`scaleout_spmm`):

    * ``replicated``  every rank already holds the whole dense operand: the local SpMM alone;
    * ``allgather``   one NCCL all-gather of the dense row blocks, then the SpMM;
    * ``exchange``    only the rows a shard references, fetched by the pull kernel from the owners'
                      peer-mapped blocks: in one piece followed by the product (``needed`` / ``pull``),
                      and in ``row_chunks`` fetches ordered by the row group that first needs a row,
                      the product of a row group running beside the next fetch
                      (``needed_rowgroups`` / ``pull``, once per group count given); the fastest is
                      the figure, all of them and the two legs of the first alone are reported.

    ``labels="scattered"`` relabels the nodes by a seeded random permutation first
    (``shard.scattered_labels``, a symmetric permutation P A P^T: the same product up to the order
    of rows): every rank then holds the same mix of rows instead of rank 0 the hubs and the last rank
    most of the rows, and no rank's outgoing link carries more than its share of the exchange.
    ``legs=False`` leaves out the timings of the separate legs.

    Times are CUDA-event times on the launching stream, maximum over ranks.  The replicated product
    is checked on sampled rows against fp64 dense algebra, the other forms against it.
    """
    import torch.distributed as dist
    from . import shard
    from .shard import ShardedSpMM

    dev = torch.device(device)
    m = synth.rmat(scale, nnz, seed=seed, device=dev)
    n = m.n_rows
    if labels == "scattered":
        m.rowPtr, m.colIdx, m.val = shard.relabel_symmetric(m.rowPtr, m.colIdx, m.val, shard.scattered_labels(n, seed))
        torch.cuda.empty_cache()
    elif labels != "natural":
        raise ValueError("labels is 'natural' or 'scattered'")
    sh = ShardedSpMM(m.rowPtr, m.colIdx, m.val, n, rank, world, device=dev)
    a, b = int(m.rowPtr[sh.lo]), int(m.rowPtr[sh.hi])
    cols_global = m.colIdx[a:b].clone()
    sh.keep_global_columns(cols_global)
    common = dict(row_bounds=sh.row_bounds, device=dev, local_block=(sh.rowPtr, cols_global, sh.val))
    notes = {}
    group_counts = [int(k) for k in (row_chunks if isinstance(row_chunks, (tuple, list)) else (row_chunks,))]
    try:
        sh_pull = ShardedSpMM(m.rowPtr, m.colIdx, m.val, n, rank, world, exchange="needed", transport="pull", **common)
        pipes = [ShardedSpMM(m.rowPtr, m.colIdx, m.val, n, rank, world, exchange="needed_rowgroups",
                             transport="pull", row_chunks=k, **common) for k in group_counts]
        src = sh_pull.symmetric_input(dim)  # peer-mapped blocks, where a producer would leave its rows
        src_pipes = [p.symmetric_input(dim) for p in pipes]
        transport = "pull"
    except Exception as ex:  # peer-mapped memory unavailable: the NCCL all-to-all forms stand in
        notes["pull_unavailable"] = "%s: %s" % (type(ex).__name__, ex)
        sh_pull = ShardedSpMM(m.rowPtr, m.colIdx, m.val, n, rank, world, exchange="needed", **common)
        group_counts = group_counts[:1]
        pipes = [ShardedSpMM(m.rowPtr, m.colIdx, m.val, n, rank, world, exchange="needed_pipelined",
                             row_chunks=group_counts[0], **common)]
        transport = "nccl"
    nnz_total = m.nnz
    del m
    torch.cuda.empty_cache()
    B_full = synth.dense_uniform(n, dim, seed + 1, dev)
    c0, c1 = sh.my_cols
    B_shard = B_full[c0:c1].clone()
    out_rep = torch.empty(sh.local_rows, dim, device=dev)
    out = torch.empty(sh.local_rows, dim, device=dev)

    def timed(fn):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    res = {"world": world, "n": n, "nnz": nnz_total, "dim": dim, "row_chunks": group_counts, "transport": transport,
           "labels": labels, "local_rows": int(sh.local_rows)}
    res["replicated_ms"] = timed(lambda: sh.forward_replicated(B_full, out_rep))
    rows = sample_rows(sh.rowPtr, 40, seed)
    res["fp64_worst_error_over_bound"] = round(check_rows_fp64(sh.rowPtr, cols_global, sh.val, B_full, out_rep, rows,
                                                               "row shard %d of %d" % (rank, world)), 3)
    res["fp64_rows_checked"] = int(rows.numel())
    res["fp64_largest_checked_element_offset"] = int(rows.max()) * dim
    del B_full
    tol = dict(rtol=1e-4, atol=2e-3)  # hub rows: 1e5 terms, pieces added in a different order per launch
    res["allgather_ms"] = timed(lambda: sh.forward(B_shard, out))
    torch.testing.assert_close(out, out_rep, **tol)
    if transport == "pull":
        src.copy_(B_shard)
        for sp in src_pipes:
            sp.copy_(B_shard)
    else:
        src, src_pipes = B_shard, [B_shard]
    out.fill_(float("nan"))
    res["exchange_one_piece_ms"] = timed(lambda: sh_pull.forward(src, out))
    torch.testing.assert_close(out, out_rep, **tol)
    # every group count with the load/store fetch kernel and, for the fetches that run beside a
    # product, with the bulk-copy one (one warp per thread block: it takes fewer warp slots and
    # registers from the product); a failure of the second form is recorded, not raised
    by_groups = {}
    for k, p, sp in zip(group_counts, pipes, src_pipes):
        for bulk in ((0, 1) if transport == "pull" else (0,)):
            label = "%d%s" % (k, "_bulk" if bulk else "")
            try:
                p.pull_bulk = bulk
                out.fill_(float("nan"))
                t = timed(lambda: p.forward(sp, out))
                torch.testing.assert_close(out, out_rep, **tol)
                by_groups[label] = t
            except Exception as ex:
                if not bulk:
                    raise
                notes["bulk_fetch_failed_%d_groups" % k] = "%s: %s" % (type(ex).__name__, str(ex)[:200])
            finally:
                p.pull_bulk = 0
    if transport == "pull":
        notes["bulk_fetch_status"] = ops.pull_rows_status()
    best = min(by_groups, key=by_groups.get)
    best_k = int(best.split("_")[0])
    res["exchange_pipelined_ms"] = by_groups[best]
    res["exchange_pipelined_ms_by_groups"] = {k: round(v, 4) for k, v in by_groups.items()}
    if transport == "pull":
        # where the time of one call of the best pipeline goes: every fetch and every row-group product
        # bracketed by timing events (this rank's own clock, ms from the start of the call)
        try:
            p, sp = pipes[group_counts.index(best_k)], src_pipes[group_counts.index(best_k)]
            p.pull_bulk, p.trace = int(best.endswith("_bulk")), True
            p.forward(sp, out)
            res["timeline_of_best_pipeline"] = p.trace_result()
        except Exception as ex:
            notes["timeline_failed"] = "%s: %s" % (type(ex).__name__, str(ex)[:200])
        finally:
            p.pull_bulk, p.trace = 0, False
    res["exchange_ms"] = min(res["exchange_one_piece_ms"], res["exchange_pipelined_ms"])
    res["exchange_form"] = ("one fetch, then the product" if res["exchange_ms"] == res["exchange_one_piece_ms"]
                            else "%d fetches ordered by first use, products of row groups overlapped%s"
                            % (best_k, ", later fetches by bulk asynchronous copies" if best.endswith("_bulk") else ""))
    if transport == "pull":
        res["first_fetch_share"] = {str(k): round(p.chunk_plan[0][1] / max(1, p.n_needed), 4)
                                    for k, p in zip(group_counts, pipes)}
    res["needed_rows_fraction"] = round(sh_pull.n_needed / n, 4)
    if transport == "pull":
        # rows every owner sends (summed over the ranks that fetch from it) against rows every rank
        # receives: the busiest outgoing link bounds the exchange
        first_all = sh_pull.pull_lists()[0][1]
        mine = torch.tensor([first_all[p + 1] - first_all[p] if p != rank else 0 for p in range(world)],
                            device=dev, dtype=torch.int64)
        sent = mine.clone()
        if world > 1:
            dist.all_reduce(sent)
        res["rows_received_by_this_rank"] = int(mine.sum())
        res["rows_sent_per_owner"] = [int(x) for x in sent.tolist()]
        res["busiest_sender_over_mean"] = round(float(sent.max()) / max(1.0, float(sent.double().mean())), 3)
    if transport == "pull" and legs:
        # the two legs of the one-piece form alone: the fetch, and the product on the compact operand
        base, first, want_rows = sh_pull.pull_lists()[0]
        _, peers, _ = sh_pull._peer_blocks(dim, B_shard)
        recv = sh_pull._receive_buffer(max(1, sh_pull.n_needed), dim, B_shard)
        rot = first[(rank + 1) % world] % max(1, sh_pull.n_needed)
        res["fetch_alone_ms"] = timed(lambda: ops.pull_rows(recv, peers, first, want_rows, rotate=rot, ctas=sh_pull.pull_ctas))
        for c in (32, 128, 256):
            res["fetch_alone_%d_ctas_ms" % c] = timed(lambda: ops.pull_rows(recv, peers, first, want_rows, rotate=rot, ctas=c))
        res["fetch_alone_all_sms_ms"] = timed(lambda: ops.pull_rows(recv, peers, first, want_rows, rotate=rot, ctas=1184))
        res["pull_ctas"] = sh_pull.pull_ctas
        res["fetched_bytes"] = int(sh_pull.n_needed) * dim * 4
        res["spmm_on_fetched_rows_ms"] = timed(lambda: sh_pull.local_spmm(out, recv, sh_pull.rowPtr, sh_pull.colIdx, sh_pull.val))
        if world > 1:
            # the same copy kernel with the roles swapped: local rows gathered and WRITTEN into the next rank's
            # peer-mapped block (nothing reads that block any more), same row count as one owner's share of a fetch
            nxt = (rank + 1) % world
            cnt = min(first[nxt + 1] - first[nxt], peers[nxt].shape[0], B_shard.shape[0])
            if cnt > 0:
                rows_local = torch.sort(torch.randperm(B_shard.shape[0], device=dev)[:cnt]).values.to(torch.int32)
                res["remote_write_rows"] = int(cnt)
                res["remote_write_ms"] = timed(lambda: ops.pull_rows(peers[nxt][:cnt], [B_shard], [0, cnt], rows_local,
                                                                     ctas=sh_pull.pull_ctas))
                res["remote_read_same_rows_ms"] = timed(lambda: ops.pull_rows(recv[:cnt], [peers[nxt]], [0, cnt], rows_local,
                                                                              ctas=sh_pull.pull_ctas))
    res.update(notes)
    for k in list(res):
        if k.endswith("_ms"):
            res[k] = round(res[k], 4)
    return res
