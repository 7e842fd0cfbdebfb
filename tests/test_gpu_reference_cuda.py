"""GPU parity against the reference's OWN CUDA kernels for SpMM, SDDMM and genmask.

oracle/build_oracle.py::build_ref_sddmm compiles the reference's SDDMM extension (sddmm.cpp,
sddmm_kernel.cu, sddmm_baseline_kernel.cu) unmodified for sm_100a into oracle/_ref/; these tests
run it next to the oracle's restatement (which this pins) and next to this library's kernels.
They are skipped when that file is absent (it is built only where the reference tree is mounted and
travels with the tree as a binary).

The reference kernels are called inside the domain their launchers support (read from
SDDMM/sddmm_kernel.cu:144-185, 249-290): CF = ceil(dim / 32) <= 4, so that the launch has one
column tile, contiguous fp32 operands, int32 indices, A with one row per (block-)row."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-4


@pytest.fixture(scope="module")
def ref():
    from oracle import build_oracle
    mod = build_oracle.load_ref_sddmm()
    if mod is None:
        pytest.skip("oracle/_ref/ParamSDDMM_ref.so is not there (built only where the reference tree is mounted)")
    return mod


@pytest.fixture(scope="module")
def graphs():
    from paramspmm_ae_b200 import synth
    return {"powerlaw": synth.powerlaw_graph(3001, 24000, seed=1),
            "rmat": synth.with_empty_rows(synth.rmat(12, 60000, seed=23), every=5)}


def _close(got, want):
    np.testing.assert_allclose(got.detach().cpu().numpy(), np.asarray(want), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("name", ["powerlaw", "rmat"])
@pytest.mark.parametrize("dim", [32, 48, 64, 100, 128])
def test_csr_sddmm_against_reference_cuda(ref, graphs, name, dim):
    from oracle import oracle as orc
    from paramspmm_ae_b200 import ops, synth
    dev = torch.device("cuda:0")
    m = graphs[name]
    d = m.to(dev)
    A = synth.dense_uniform(m.n_rows, dim, 700 + dim).to(dev)
    B = synth.dense_uniform(m.n_cols, dim, 800 + dim).to(dev)
    CF = (dim + 31) // 32
    theirs = ref.csr_sddmm(A, B, d.rowPtr, d.colIdx, d.val, CF, 8)
    torch.cuda.synchronize()
    # the restatement is pinned by the reference's kernel ...
    want = orc.sddmm_csr(*m.numpy()[:2], A.cpu().numpy(), B.cpu().numpy())
    _close(theirs, want)
    # ... and this library's kernel agrees with it
    _close(ops.csr_sddmm(A, B, d.rowPtr, d.colIdx, d.val, CF, 8), theirs.cpu().numpy())
    rps, tr = ops.split_csr(m.rowPtr, 32)
    rps, tr = rps.to(dev), tr.to(dev)
    theirs_split = ref.csr_split_sddmm(A, B, rps, d.colIdx, d.val, tr, CF, 8)
    torch.cuda.synchronize()
    _close(theirs_split, want)
    _close(ops.csr_split_sddmm(A, B, rps, d.colIdx, d.val, tr, CF, 8), theirs_split.cpu().numpy())


@pytest.mark.parametrize("name", ["powerlaw", "rmat"])
def test_genmask_and_block_sddmm_against_reference_cuda(ref, graphs, name):
    from oracle import oracle as orc
    from paramspmm_ae_b200 import ops, synth
    dev = torch.device("cuda:0")
    m = graphs[name]
    rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, m.n_cols, 2)
    rpb_d, cb_d, vb_d, rp_d = rpb.to(dev), cb.to(dev), vb.to(dev), m.rowPtr.to(dev)
    theirs = ref.genmask(rpb_d, rp_d, vb_d, m.nnz)
    torch.cuda.synchronize()
    want = orc.genmask(rpb.numpy(), m.rowPtr.numpy(), vb.numpy(), m.nnz)
    assert np.array_equal(theirs.cpu().numpy(), want)                      # pins the restatement, bit for bit
    assert torch.equal(ops.genmask(rpb_d, rp_d, vb_d, m.nnz), theirs)      # and this library's kernel
    nbr = rpb.shape[0] - 1
    for dim in (64, 100):
        A = synth.dense_uniform(nbr * 2, dim, 500 + dim).to(dev)
        B = synth.dense_uniform(m.n_cols, dim, 600 + dim).to(dev)
        CF = (dim + 31) // 32
        theirs_b = ref.bcsr_sddmm(A, B, rpb_d, cb_d, vb_d, CF, 8)
        torch.cuda.synchronize()
        want_b = orc.sddmm_bcsr(rpb.numpy(), cb.numpy(), vb.numpy(), A.cpu().numpy(), B.cpu().numpy())
        _close(theirs_b, want_b)
        _close(ops.bcsr_sddmm(A, B, rpb_d, cb_d, vb_d, CF, 8), theirs_b.cpu().numpy())


# ----------------------------------------------------------------------------- SpMM
@pytest.fixture(scope="module")
def ref_spmm():
    from oracle import build_oracle
    mod = build_oracle.load_ref_spmm_cuda()
    if mod is None:
        pytest.skip("oracle/_ref/ParamSpMM_cuda_ref.so is not there (built only where the reference tree is mounted)")
    return mod


@pytest.mark.parametrize("name", ["powerlaw", "rmat"])
@pytest.mark.parametrize("dim", [16, 47, 64, 100, 128, 256])
def test_spmm_against_reference_cuda(ref_spmm, graphs, name, dim):
    """The reference's own csr / csr_split / bcsr / bcsr_split SpMM kernels (SpMM/SpMM_kernel.cu,
    compiled unmodified) next to the restatement and to this library's kernels.  The reference's
    split kernels add their pieces with atomics, so their hub rows differ from run to run in the
    last bits: the comparison uses the tolerance the project states (1e-5 relative, 1e-4 absolute)."""
    from oracle import oracle as orc
    from paramspmm_ae_b200 import ops, synth
    dev = torch.device("cuda:0")
    m = graphs[name]
    d = m.to(dev)
    X = synth.dense_uniform(m.n_cols, dim, 300 + dim).to(dev)
    CF = min(8, (dim + 31) // 32)
    want = orc.spmm_csr(*m.numpy(), X.cpu().numpy())
    theirs = ref_spmm.csr_spmm(X, d.rowPtr, d.colIdx, d.val, CF, 8)
    torch.cuda.synchronize()
    _close(theirs, want)                                                   # pins the restatement
    _close(ops.csr_spmm(X, d.rowPtr, d.colIdx, d.val, CF, 8), theirs.cpu().numpy())
    rps, tr = ops.split_csr(m.rowPtr, 32)
    rps, tr = rps.to(dev), tr.to(dev)
    theirs_split = ref_spmm.csr_split_spmm(X, rps, d.colIdx, d.val, tr, CF, 8)
    torch.cuda.synchronize()
    _close(theirs_split, want)
    _close(ops.csr_split_spmm(X, rps, d.colIdx, d.val, tr, CF, 8), theirs_split.cpu().numpy())
    # 2 x 1 block layout
    rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, m.n_cols, 2)
    rpb_d, cb_d, vb_d = rpb.to(dev), cb.to(dev), vb.to(dev)
    theirs_b = ref_spmm.bcsr_spmm(X, rpb_d, cb_d, vb_d, CF, 8)
    torch.cuda.synchronize()
    _close(theirs_b[: m.n_rows], want)
    ours_b = ops.bcsr_spmm(X, rpb_d, cb_d, vb_d, CF, 8)
    assert ours_b.shape == theirs_b.shape
    _close(ours_b, theirs_b.cpu().numpy())


@pytest.mark.parametrize("name", ["powerlaw", "rmat"])
@pytest.mark.parametrize("dim", [16, 47, 64, 100, 128, 256])
def test_split_block_and_vec_spmm_against_reference_cuda(ref_spmm, graphs, name, dim):
    """bcsr_split_spmm (2 x 1 blocks, row-split), vec_spmm and vec_split_spmm (3 x 1 blocks) of the
    reference (SpMM/SpMM.cpp:273-480) next to the restatement and to this library's kernels.
    The block-rows are split at 32 blocks, the reference's own partition length for short rows
    (graph_input.py:101), so each piece is one staging window of its kernels."""
    from oracle import oracle as orc
    from paramspmm_ae_b200 import ops, synth
    dev = torch.device("cuda:0")
    m = graphs[name]
    X = synth.dense_uniform(m.n_cols, dim, 300 + dim).to(dev)
    CF = min(8, (dim + 31) // 32)
    want = orc.spmm_csr(*m.numpy(), X.cpu().numpy())
    for V, plain, split in ((2, None, ref_spmm.bcsr_split_spmm), (3, ref_spmm.vec_spmm, ref_spmm.vec_split_spmm)):
        rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, m.n_cols, V)
        rps, tr = ops.split_csr(rpb, 32)
        rpb_d, cb_d, vb_d, rps_d, tr_d = (t.to(dev) for t in (rpb, cb, vb, rps, tr))
        ours_plain = ops.bcsr_spmm if V == 2 else ops.vec_spmm
        ours_split = ops.bcsr_split_spmm if V == 2 else ops.vec_split_spmm
        if plain is not None:
            theirs = plain(X, rpb_d, cb_d, vb_d, CF, 8)
            torch.cuda.synchronize()
            _close(theirs[: m.n_rows], want)                               # pins the restatement
            ours = ours_plain(X, rpb_d, cb_d, vb_d, CF, 8)
            assert ours.shape == theirs.shape
            _close(ours, theirs.cpu().numpy())
        theirs_s = split(X, rps_d, cb_d, vb_d, tr_d, CF, 8)
        torch.cuda.synchronize()
        _close(theirs_s[: m.n_rows], want)
        ours_s = ours_split(X, rps_d, cb_d, vb_d, tr_d, CF, 8)
        assert ours_s.shape == theirs_s.shape
        _close(ours_s, theirs_s.cpu().numpy())


@pytest.mark.parametrize("name", ["powerlaw", "rmat"])
def test_split_block_sddmm_against_reference_cuda(ref, graphs, name):
    """bcsr_split_sddmm of the reference (SDDMM/sddmm.cpp:169-219) inside the domain its launcher
    supports (one column tile: CF = ceil(dim / 32) <= 4; A padded to an even row count, as the
    reference's own callers pad it).  The 3 x 1 SDDMM kernels of the reference are not run: read as
    text they index shared memory with a hard-coded factor 2 and guard the wrong loop variable
    (sddmm_kernel.cu:1303, 1339), so they stay checked against the restatement only."""
    from oracle import oracle as orc
    from paramspmm_ae_b200 import ops, synth
    dev = torch.device("cuda:0")
    m = graphs[name]
    rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, m.n_cols, 2)
    rps, tr = ops.split_csr(rpb, 32)
    cb_d, vb_d, rps_d, tr_d = (t.to(dev) for t in (cb, vb, rps, tr))
    nbr = rpb.shape[0] - 1
    for dim in (32, 64, 100, 128):
        A = synth.dense_uniform(nbr * 2, dim, 500 + dim).to(dev)
        B = synth.dense_uniform(m.n_cols, dim, 600 + dim).to(dev)
        CF = (dim + 31) // 32
        theirs = ref.bcsr_split_sddmm(A, B, rps_d, cb_d, vb_d, tr_d, CF, 8)
        torch.cuda.synchronize()
        want = orc.sddmm_bcsr(rpb.numpy(), cb.numpy(), vb.numpy(), A.cpu().numpy(), B.cpu().numpy())
        _close(theirs, want)
        _close(ops.bcsr_split_sddmm(A, B, rps_d, cb_d, vb_d, tr_d, CF, 8), theirs.cpu().numpy())
    # an A that stops inside the last block-row (odd row count, not padded): nothing is read past it
    if m.n_rows % 2 == 1:
        A = synth.dense_uniform(m.n_rows, 64, 9).to(dev)
        B = synth.dense_uniform(m.n_cols, 64, 10).to(dev)
        Apad = torch.cat([A, torch.zeros(1, 64, device=dev)])
        want = orc.sddmm_bcsr(rpb.numpy(), cb.numpy(), vb.numpy(), Apad.cpu().numpy(), B.cpu().numpy())
        _close(ops.bcsr_sddmm(A, B, rpb.to(dev), cb_d, vb_d, 2, 8), want)
        _close(ops.bcsr_split_sddmm(A, B, rps_d, cb_d, vb_d, tr_d, 2, 8), want)
