"""The reference's OWN Python layers, unmodified, running on a GPU on top of the drop-in
extension modules (``ParamSpMM``, ``ParamSDDMM``, ``ParamSpCONV`` resolved to this package).

``oracle/build_oracle.py::stage_reference_python`` copies ``PCSR.py``, ``SDDMM.py``,
``gnn_conv.py``, ``graph_input.py``, ``verification.py``, ``decider.py`` and the toy matrix of the
reference as they are into the git-ignored ``baseline/_ref`` (the same arrangement as the compiled
checkers in ``oracle/_ref``); the tests import them from there and are skipped where that
directory is absent.  What runs is the reference's code path: its loader, its operator objects
(``pcsr_spmm`` / ``pcsr_sddmm`` / ``coo_spmm`` / ``csc_spmm``), its acceptance checks
(``SpMM_verification.compare``, ``SDDMM.compare`` / ``compare_2d``) and its autograd layers; every
extension call underneath lands in libpspmm.  A signature, shape or dtype that the drop-in gets
wrong shows up here as an exception inside the reference's own code.

The pickled random forests of the reference's decider are not loaded (they are replaced by the
measured table); every ``<if_split, vec_size>`` combination the forests can return is exercised
instead.
"""
import math
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

DIMS = [16, 32, 48, 64, 100, 128]


@pytest.fixture(scope="module")
def ref():
    """The reference's modules, imported from the staged copy with the drop-in on sys.path."""
    from oracle import build_oracle
    stage = build_oracle.staged_reference_python()
    if stage is None:
        pytest.skip("baseline/_ref does not hold the reference's Python layers (staged where the reference is mounted)")
    import paramspmm_ae_b200
    from paramspmm_ae_b200 import _lib
    _lib.lib()  # no CUDA library, no test
    paramspmm_ae_b200.install_dropin()
    for name in ("graph_input", "verification", "PCSR", "SDDMM", "gnn_conv", "decider"):
        sys.modules.pop(name, None)  # a copy imported from elsewhere must not shadow the staged one
    sys.path.insert(0, stage)
    try:
        import PCSR as r_pcsr
        import SDDMM as r_sddmm
        import decider as r_decider
        import gnn_conv as r_conv
        import graph_input as r_gi
        import verification as r_veri
    finally:
        sys.path.remove(stage)
    for m in (r_pcsr, r_sddmm, r_decider, r_conv, r_gi, r_veri):
        assert os.path.realpath(m.__file__).startswith(os.path.realpath(stage)), m.__file__
    import ParamSpMM
    assert "paramspmm_ae_b200" in os.path.realpath(ParamSpMM.__file__)

    class Mods:
        pcsr, sddmm, decider, conv, gi, veri = r_pcsr, r_sddmm, r_decider, r_conv, r_gi, r_veri
        path = os.path.join(stage, "toy_dataset") + os.sep
    return Mods


def _load(ref, **kw):
    g = ref.gi.graph_input(mtx_name="pubmed", path=ref.path)
    g.load(load_from_mtx=True, **kw)
    return g


@pytest.fixture(scope="module")
def graph(ref):
    return _load(ref, if_mask=True)


def test_reference_decider_loop_on_the_dropin(ref, graph, capsys):
    """decider.py:126-156 of the reference: for every dim build the operator the decider asks for,
    run it, and pass SpMM_verification.compare (1e-4 relative against torch.sparse.mm); then the
    timing calls of :157-172 (profiling, COO, CSC, cuSPARSE, GE-SpMM)."""
    c = graph.csr_data
    veri = ref.veri.SpMM_verification(1, c.rowPtr, c.colIdx, c.val, baseline=True)
    coo, csc = ref.pcsr.coo_spmm(graph), ref.pcsr.csc_spmm(graph)
    dec = ref.decider.SpMMDecider("unused/")  # decode_tree only: the pickles stay closed
    for dim in DIMS:
        veri.reference(dim)
        d16 = math.ceil(dim / 16) * 16
        for code in range(4):  # <if_split, vec_size> in every combination the forests can return
            if_split, vec_size, CF, W = dec.decode_tree(code, d16)
            assert (if_split, vec_size) == (code % 2, [1, 2][code // 2])
            op = ref.pcsr.pcsr_spmm(graph=graph, vec_size=vec_size, if_split=if_split, CF=CF, blkWarpNum=W)
            op.get_spmm_result(dim)
            assert op.result.shape == (graph.mtx_nodes, dim) and op.result.device.type == "cpu"
            veri.compare(op.result, "pubmed")
        # the comparators of the same loop agree with the same reference result
        veri.compare(coo.get_spmm_result(dim), "pubmed-coo")
        veri.compare(csc.get_spmm_result(dim), "pubmed-csc")
        p10 = ref.pcsr.pcsr_spmm(graph, vec_size=1, if_split=False)
        veri.compare(p10.cusparse_ref(dim), "pubmed-cusparse")
        veri.compare(p10.cusparse_csr_alg2_ref(dim), "pubmed-cusparse-alg2")
        veri.compare(p10.gespmm_ref(dim), "pubmed-gespmm")
    for dim in (32, 100):
        for vec_size, if_split in ((1, False), (1, True), (2, False), (2, True)):
            op = ref.pcsr.pcsr_spmm(graph, vec_size=vec_size, if_split=if_split, CF=1, blkWarpNum=8)
            assert op.profiling(dim) > 0 and op.cf_warpnum_profiling(1, 4, dim) > 0
        assert coo.profiling(dim) > 0 and csc.profiling(dim) > 0
        assert p10.cusparse_ref(dim, is_profiling=True) > 0 and p10.gespmm_ref(dim, is_profiling=True) > 0
    capsys.readouterr()


def test_reference_vec_size_3_operator(ref, graph, capsys):
    """vec_size = 3: the reference's loader builds 2 x 1 blocks only and its raw-tensor constructor
    rejects every 2-D value array (PCSR.py:165-166), so the branch of get_spmm_result that calls
    vec_spmm / vec_split_spmm (:226-240) is reached here by handing 3 x 1 arrays to an operator
    object built from the graph."""
    from paramspmm_ae_b200 import ops
    c = graph.csr_data
    rpb, cb, vb = ops.bcsr_from_csr(c.rowPtr, c.colIdx, c.val, graph.mtx_nodes, 3)
    with pytest.raises(ValueError):
        ref.pcsr.pcsr_spmm(None, 3, False, graph.mtx_nodes, graph.mtx_edges, rpb, cb, vb, None)
    veri = ref.veri.SpMM_verification(1, c.rowPtr, c.colIdx, c.val)
    rps, tr = ops.split_csr(rpb, 32)
    for dim in (32, 100):
        veri.reference(dim)
        for if_split, rp, t in ((False, rpb, None), (True, rps, tr)):
            op = ref.pcsr.pcsr_spmm(graph, vec_size=2, if_split=if_split, CF=1, blkWarpNum=4)
            op.vec_size, op.rowPtr, op.colIdx, op.val = 3, rp.cuda(), cb.cuda(), vb.cuda()
            op.target_row = t.cuda() if t is not None else None
            op.get_spmm_result(dim)
            veri.compare(op.result, "pubmed-vec3")
    capsys.readouterr()


def test_reference_sddmm_engine_on_the_dropin(ref, graph, capsys):
    """SDDMM.py:270-340 of the reference (profile_engine's body): the four operator objects, both
    warp counts, compared with cusparse_ref through the reference's compare / compare_2d, and the
    profiling call of each."""
    S = ref.sddmm
    ops4 = [S.pcsr_sddmm(graph, vec_size=1, if_split=False), S.pcsr_sddmm(graph, vec_size=1, if_split=True),
            S.pcsr_sddmm(graph, vec_size=2, if_split=False), S.pcsr_sddmm(graph, vec_size=2, if_split=True)]
    for dim in (32, 64, 100, 128):
        want = ops4[0].cusparse_ref(dim)
        for W in (4, 8):
            for i, op in enumerate(ops4):
                op.get_sddmm_result(dim=dim, blkWarpNum=W)
                torch.cuda.synchronize()
                if i < 2:
                    S.compare(op.result, want)
                else:
                    S.compare_2d(op.result, want, op.mask)
        for op in ops4:
            assert op.profiling(8, dim) > 0
    assert ops4[0].cusparse_ref(64, is_profiling=True) > 0
    capsys.readouterr()


def _dense_adjacency(g, dev):
    import numpy as np
    rp, ci, v = g.csr_data.rowPtr.numpy(), g.csr_data.colIdx.numpy(), g.csr_data.val.numpy()
    rows = np.repeat(np.arange(g.mtx_nodes), rp[1:] - rp[:-1])
    A = torch.zeros(g.mtx_nodes, g.mtx_nodes, dtype=torch.float64)
    A[torch.from_numpy(rows), torch.from_numpy(ci.astype("int64"))] = torch.from_numpy(v).double()
    return A.to(dev)


def _close_strict(got, want, what):
    # fp32 sums over a node's neighbours against fp64: 1e-5 relative, 1e-4 absolute
    torch.testing.assert_close(got.double(), want, rtol=1e-5, atol=1e-4, msg=lambda m: what + ": " + m)


def _close_reduction(got, want, what):
    # Weight gradients are dense fp32 products that sum over all 19,717 nodes, done by cuBLAS
    # (torch.mm) in the reference's layers and in this package's alike: the absolute floor follows
    # the size of the result (1e-5 of its largest element) instead of being fixed at 1e-4.
    torch.testing.assert_close(got.double(), want, rtol=1e-5, atol=1e-5 * max(10.0, float(want.abs().max())),
                               msg=lambda m: what + ": " + m)


@pytest.mark.parametrize("vec_size,if_split", [(1, False), (1, True), (2, False), (2, True)])
def test_reference_gcn_and_gin_layers_forward_backward(ref, vec_size, if_split, capsys):
    """GCNConv and GINConv of the reference's gnn_conv.py (:13-107, :205-238), stacked as GNN.py
    stacks them (widths 32 -> 48 -> 16), forward and backward: equal to dense fp64 algebra and to
    this package's own layers on the same weights."""
    from paramspmm_ae_b200 import gnn_conv as mine
    from paramspmm_ae_b200 import pcsr as my_pcsr
    dev = torch.device("cuda:0")
    for net, kw in (("gcn", dict(is_normalize=True)), ("gin", dict(GIN_epsilon=0.5))):
        g = _load(ref, **kw)
        A = _dense_adjacency(g, dev)
        n = g.mtx_nodes
        dims = [32, 48, 16]
        spmm = {d: ref.pcsr.pcsr_spmm(graph=g, vec_size=vec_size, if_split=bool(if_split), CF=1, blkWarpNum=8)
                for d in dims[1:]}
        mine_spmm = {d: my_pcsr.pcsr_spmm(g, vec_size, bool(if_split), CF=1, blkWarpNum=8) for d in dims[1:]}
        Conv, MyConv = (ref.conv.GCNConv, mine.GCNConv) if net == "gcn" else (ref.conv.GINConv, mine.GINConv)
        torch.manual_seed(11)
        layers = [Conv(a, b).to(dev) for a, b in zip(dims[:-1], dims[1:])]
        my_layers = [MyConv(a, b).to(dev) for a, b in zip(dims[:-1], dims[1:])]
        for l, m in zip(layers, my_layers):
            m.weights.data.copy_(l.weights.data)
        rows = n if vec_size == 1 else (n + 1) // 2 * 2  # GNN.py pads the features for the block layouts
        X = torch.randn(rows, dims[0], device=dev)
        X[n:] = 0
        G = torch.randn(n, dims[-1], device=dev)

        def run(ls, sp):
            x = X.clone().requires_grad_(True)
            h = x
            for i, l in enumerate(ls):
                h = l(h, sp)
                if i + 1 < len(ls):
                    h = torch.relu(h)
            h[:n].backward(G) if h.shape[0] != n else h.backward(G)
            return h.detach()[:n], x.grad[:n], [l.weights.grad for l in ls]

        out, gx, gw = run(layers, spmm)
        out2, gx2, gw2 = run(my_layers, mine_spmm)
        # dense fp64 algebra
        Ws = [l.weights.detach().double().requires_grad_(True) for l in layers]
        x64 = X[:n].double().requires_grad_(True)
        h = x64
        for i, W in enumerate(Ws):
            h = A @ (h @ W) if net == "gcn" else (A @ h) @ W
            if i + 1 < len(Ws):
                h = torch.relu(h)
        h.backward(G.double())
        # GIN aggregates with unnormalised weights (1 per edge, 1 + epsilon on the diagonal): three
        # layers grow the activations to the thousands and elements that cancel to small values carry
        # the rounding of their large terms, so its floor follows the result's size as well
        _close = _close_strict if net == "gcn" else _close_reduction
        _close(out, h.detach(), net + " forward")
        _close(gx, x64.grad, net + " input gradient")
        for a, b in zip(gw, Ws):
            _close_reduction(a, b.grad, net + " weight gradient")
        _close(out2, h.detach(), net + " forward (package layer)")
        _close(gx2, x64.grad, net + " input gradient (package layer)")
        for a, b in zip(gw2, Ws):
            _close_reduction(a, b.grad, net + " weight gradient (package layer)")
    capsys.readouterr()


@pytest.mark.parametrize("vec_size,if_split", [(1, False), (1, True), (2, False), (2, True)])
def test_reference_agnn_layer_forward_backward(ref, vec_size, if_split, capsys):
    """AGNNConv of the reference (gnn_conv.py:110-202) as GNN.py:226-240 drives it (features padded
    to an even row count, colIdx as an [nnz, 1] column): forward, and the gradients it defines,
    equal to this package's layer on the same parameters; forward and the input / weight gradients
    also equal to dense fp64 algebra."""
    from paramspmm_ae_b200 import gnn_conv as mine
    from paramspmm_ae_b200 import pcsr as my_pcsr
    dev = torch.device("cuda:0")
    g = _load(ref, is_normalize=True, if_mask=True)
    n = g.mtx_nodes
    A = _dense_adjacency(g, dev)
    mask = (A != 0).double()
    hid = 32
    op = ref.pcsr.pcsr_spmm(graph=g, vec_size=vec_size, if_split=bool(if_split), CF=1, blkWarpNum=8)
    my_op = my_pcsr.pcsr_spmm(g, vec_size, bool(if_split), CF=1, blkWarpNum=8)
    colIdx = g.csr_data.colIdx.to(dev).unsqueeze(-1)
    torch.manual_seed(12)
    layer = ref.conv.AGNNConv(24, hid).to(dev)
    my_layer = mine.AGNNConv(24, hid).to(dev)
    my_layer.weights.data.copy_(layer.weights.data)
    my_layer.attention_w.data.copy_(layer.attention_w.data)
    rows = (n + 1) // 2 * 2
    X = torch.randn(rows, 24, device=dev) * 0.3
    X[n:] = 0
    G = torch.randn(rows, hid, device=dev)
    G[n:] = 0

    def run(l, o):
        x = X.clone().requires_grad_(True)
        out = l(x, {hid: o}, colIdx)
        assert out.shape == (rows, hid)  # one output row per input row, as zeros_like(input) gives
        out.backward(G)
        return out.detach()[:n], x.grad[:n], l.weights.grad, l.attention_w.grad

    out, gx, gw, ga = run(layer, op)
    out2, gx2, gw2, ga2 = run(my_layer, my_op)
    beta = float(layer.attention_w.detach().reshape(()))
    W64 = layer.weights.detach().double()
    Xp = X[:n].double() @ W64
    E = (Xp @ Xp.t()) * mask * beta
    _close = _close_strict
    _close(out, E @ Xp, "agnn forward")
    _close(out2, E @ Xp, "agnn forward (package layer)")
    # the layer's own backward treats the edge values as constants (gnn_conv.py:153-180)
    d_prime = E @ G[:n].double()
    _close(gx, d_prime @ W64.t(), "agnn input gradient")
    _close_reduction(gw, X[:n].double().t() @ d_prime, "agnn weight gradient")
    torch.testing.assert_close(gx2, gx, rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(gw2, gw, rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(ga2, ga, rtol=1e-4, atol=1e-2)  # a sum over all edges times column ids (~1e7)
    capsys.readouterr()
