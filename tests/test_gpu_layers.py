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
    from paramspmm_ae_b200 import ops, pcsr
    if split:
        rps, tr = ops.split_csr(g.rowPtr, 8)
        return pcsr.pcsr_spmm(None, 1, True, g.n_rows, g.nnz, rps, g.colIdx, g.val, tr, CF=1, blkWarpNum=8)
    return pcsr.pcsr_spmm(None, 1, False, g.n_rows, g.nnz, g.rowPtr, g.colIdx, g.val, None, CF=1, blkWarpNum=8)


def _close(got, want):
    torch.testing.assert_close(got.double(), want.double(), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("fin,fout", [(12, 32), (32, 12), (16, 16)])
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
