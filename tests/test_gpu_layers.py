"""GPU tests of the GCN / GIN / AGNN layers (mirror of the reference's gnn_conv.py) against dense
fp64 algebra with torch autograd.  Tolerance: |got - want| <= 1e-4 + 1e-5 |want|, the bound the
SpMM tests use."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _graph(dev, n=257, pairs=1500):
    from paramspmm_ae_b200 import synth
    g = synth.powerlaw_graph(n, pairs, seed=3)  # symmetric, self loops, D^-1/2 (A+I) D^-1/2
    rp, ci, v = g.numpy()
    dense = np.zeros((n, n))
    for r in range(n):
        dense[r, ci[rp[r]:rp[r + 1]]] = v[rp[r]:rp[r + 1]]
    return g, torch.tensor(dense, dtype=torch.float64, device=dev)


def _operator(g, dev, split):
    from paramspmm_ae_b200 import decider, ops, pcsr
    if split in ("plan", "plan_split", "plan_bucketed"):  # operators bound to a decider plan
        plan = decider.Plan(vec_size=1, lanes_per_row=0, vec_width=0, cta_threads=0, rows_per_group=0, gather_batch=0,
                            col_tile=0, if_split=int(split != "plan"), granularity=8,
                            bucketed=int(split == "plan_bucketed"))
        return pcsr.pcsr_spmm.from_plan(plan, g.rowPtr.to(dev), g.colIdx.to(dev), g.val.to(dev))
    if split:
        rps, tr = ops.split_csr(g.rowPtr, 8)
        return pcsr.pcsr_spmm(None, 1, True, g.n_rows, g.nnz, rps, g.colIdx, g.val, tr, CF=1, blkWarpNum=8)
    return pcsr.pcsr_spmm(None, 1, False, g.n_rows, g.nnz, g.rowPtr, g.colIdx, g.val, None, CF=1, blkWarpNum=8)


def _close(got, want):
    torch.testing.assert_close(got.double(), want.double(), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("split", [False, True, "plan", "plan_split", "plan_bucketed"])
@pytest.mark.parametrize("fin,fout", [(12, 32), (32, 12), (16, 16), (32, 47), (7, 10)])
@pytest.mark.parametrize("reorder", [True, False])
@pytest.mark.parametrize("input_grad", [True, False])
def test_gcn_layer_forward_and_gradients(split, fin, fout, reorder, input_grad):
    from paramspmm_ae_b200 import gnn_conv
    dev = torch.device("cuda:0")
    g, A = _graph(dev)
    P = _operator(g, dev, split)
    torch.manual_seed(5)
    layer = gnn_conv.GCNConv(fin, fout).to(dev)
    H = torch.randn(g.n_rows, fin, device=dev, requires_grad=input_grad)
    old = gnn_conv.REORDER_NARROW_FIRST
    gnn_conv.REORDER_NARROW_FIRST = reorder
    try:
        out = layer(H, {fout: P})
        G = torch.randn_like(out)
        out.backward(G)
    finally:
        gnn_conv.REORDER_NARROW_FIRST = old
    W64 = layer.weights.detach().double().requires_grad_(True)
    H64 = H.detach().double().requires_grad_(True)
    ref = A @ (H64 @ W64)
    ref.backward(G.double())
    _close(out.detach(), ref.detach())
    _close(layer.weights.grad, W64.grad)
    if input_grad:
        _close(H.grad, H64.grad)
    else:
        assert H.grad is None


def test_gin_and_agnn_layers_match_dense_algebra():
    from paramspmm_ae_b200 import gnn_conv, pcsr, ops
    dev = torch.device("cuda:0")
    g, A = _graph(dev)
    P = _operator(g, dev, False)
    torch.manual_seed(6)
    X = torch.randn(g.n_rows, 16, device=dev)
    gin = gnn_conv.GINConv(16, 24).to(dev)
    _close(gin(X, {24: P}).detach(), (A @ X.double()) @ gin.weights.detach().double())
    agnn = gnn_conv.AGNNConv(16, 32).to(dev)
    Ps = pcsr.pcsr_sddmm(None, 1, False, g.n_rows, g.nnz, g.rowPtr, g.colIdx, g.val, None, CF=1, blkWarpNum=8)
    out = agnn(X, {32: Ps}, g.colIdx.to(dev))
    Xp = X.double() @ agnn.weights.detach().double()
    mask = (A != 0).double()
    E = (Xp @ Xp.t()) * mask * float(agnn.attention_w.detach().reshape(()))
    _close(out.detach(), E @ Xp)
    # inference (no gradient): the layer itself switches to the fused kernel
    with torch.no_grad():
        _close(agnn(X, {32: Ps}, g.colIdx.to(dev)), E @ Xp)
        rps, tr = ops.split_csr(g.rowPtr, 8)
        Pss = pcsr.pcsr_sddmm(None, 1, True, g.n_rows, g.nnz, rps, g.colIdx, g.val, tr, CF=1, blkWarpNum=8)
        _close(agnn(X, {32: Pss}, g.colIdx.to(dev)), E @ Xp)
    # the one-kernel form of the same forward
    fused = ops.agnn_fused(Xp.float().contiguous(), Xp.float().contiguous(), g.rowPtr.to(dev), g.colIdx.to(dev),
                           float(agnn.attention_w.detach().reshape(())), softmax=False)
    _close(fused, E @ Xp)


@pytest.mark.parametrize("kind", ["plan", "plan_bucketed"])
def test_plan_bound_operator_products(kind):
    """pcsr_spmm.from_plan: aggregation at an odd width, more input rows than the matrix has, the
    result method, and the methods that keep using the CSR arrays."""
    dev = torch.device("cuda:0")
    g, A = _graph(dev)
    P = _operator(g, dev, kind)
    X = torch.randn(g.n_rows + 1, 15, device=dev, generator=torch.Generator(device=dev).manual_seed(8))
    out = P.GIN_spmm(X)
    assert out.shape == (g.n_rows + 1, 15) and out.is_contiguous()
    _close(out[: g.n_rows], A @ X[: g.n_rows].double())
    assert float(out[g.n_rows].abs().max()) == 0.0
    with pytest.raises(RuntimeError):
        P.GIN_spmm(X[: g.n_rows - 1])
    P.get_spmm_result(dim=16)
    _close(P.result.to(dev), A.sum(1, keepdim=True).expand(-1, 16))
    e = torch.rand(g.nnz, device=dev)
    Ae = torch.zeros_like(A)
    rp, ci, _ = g.numpy()
    rows = torch.repeat_interleave(torch.arange(g.n_rows), torch.from_numpy(np.diff(rp)).long()).to(dev)
    Ae[rows, torch.from_numpy(ci).long().to(dev)] = e.double()
    _close(P.AGNN_spmm(e, X[: g.n_rows, :12].contiguous()), Ae @ X[: g.n_rows, :12].double())


@pytest.mark.parametrize("split", [False, True])
def test_agnn_layer_trains_without_edge_arrays(split):
    """AGNNConv with gradients enabled runs AGNNFusedFunction (forward and backward recompute the
    scores in the kernel): output, input and weight gradients against dense fp64 algebra with the
    edge values held constant in the backward, as the reference's layer defines it
    (gnn_conv.py:153-180); the attention gradient against the reference's expression evaluated in
    fp64; and everything against the three-kernel composition on the same parameters."""
    from paramspmm_ae_b200 import gnn_conv, ops, pcsr
    dev = torch.device("cuda:0")
    g, A = _graph(dev)
    n = g.n_rows
    if split:
        rps, tr = ops.split_csr(g.rowPtr, 8)
        P = pcsr.pcsr_sddmm(None, 1, True, n, g.nnz, rps, g.colIdx, g.val, tr, CF=1, blkWarpNum=8)
    else:
        P = pcsr.pcsr_sddmm(None, 1, False, n, g.nnz, g.rowPtr, g.colIdx, g.val, None, CF=1, blkWarpNum=8)
    colIdx = g.colIdx.to(dev).unsqueeze(-1)
    torch.manual_seed(8)
    layer = gnn_conv.AGNNConv(16, 32).to(dev)
    X = torch.randn(n, 16, device=dev) * 0.5
    G = torch.randn(n, 32, device=dev)

    def run(fused):
        old = gnn_conv.FUSE_AGNN_TRAINING
        gnn_conv.FUSE_AGNN_TRAINING = fused
        try:
            for p in layer.parameters():
                p.grad = None
            x = X.clone().requires_grad_(True)
            out = layer(x, {32: P}, colIdx)
            assert (type(out.grad_fn).__name__ == "AGNNFusedFunctionBackward") == fused
            out.backward(G)
            return out.detach(), x.grad, layer.weights.grad.clone(), layer.attention_w.grad.clone()
        finally:
            gnn_conv.FUSE_AGNN_TRAINING = old

    out, gx, gw, ga = run(True)
    out_u, gx_u, gw_u, ga_u = run(False)
    beta = float(layer.attention_w.detach().reshape(()))
    W64 = layer.weights.detach().double()
    Xp = X.double() @ W64
    mask = (A != 0).double()
    E = (Xp @ Xp.t()) * mask * beta
    D = E @ G.double()
    _close(out, E @ Xp)
    _close(gx, D @ W64.t())
    _close(gw, X.double().t() @ D)
    cols = torch.arange(n, device=dev, dtype=torch.float64)
    want_ga = (((G.double() @ G.double().t()) * mask) * cols[None, :]).sum()
    scale = ((((G.double() @ G.double().t()) * mask).abs()) * cols[None, :]).sum()
    assert abs(float(ga) - float(want_ga)) <= 1e-5 * float(scale)      # a signed sum of ~3000 products times ids
    assert abs(float(ga_u) - float(want_ga)) <= 1e-5 * float(scale)
    assert ga.shape == ga_u.shape == (1, 1)
    _close(out, out_u)
    _close(gx, gx_u)
    _close(gw, gw_u)
