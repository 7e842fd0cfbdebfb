"""CPU tests: the oracle against the golden vectors and against live third-party code."""
import json
import os

import numpy as np
import pytest
import scipy.sparse as sp


def _cases(path):
    z = np.load(path)
    return z, int(z["n_cases"])


def test_split_matches_reference_golden(oracle, golden_dir):
    z, n = _cases(os.path.join(golden_dir, "split_ref.npz"))
    for i in range(n):
        rps, tr = oracle.split_csr(z["rowPtr_%d" % i], int(z["gran_%d" % i]))
        assert np.array_equal(rps, z["rowPtr_split_%d" % i])
        assert np.array_equal(tr, z["target_row_%d" % i])
        rps2, tr2 = oracle.split_csr_numpy(z["rowPtr_%d" % i], int(z["gran_%d" % i]))
        assert np.array_equal(rps2, rps) and np.array_equal(tr2, tr)


def test_split_matches_live_reference_when_mounted(oracle):
    from oracle import build_oracle
    if not build_oracle.ref_available():
        pytest.skip("reference tree not mounted")
    import torch
    build_oracle.build_ref()
    ref = build_oracle.load_ref()
    rng = np.random.default_rng(5)
    for gran in (1, 3, 32, 96):
        ln = rng.integers(0, 200, size=500)
        ln[rng.random(500) < 0.2] = 0
        rp = np.concatenate([[0], np.cumsum(ln)]).astype(np.int32)
        a, b = ref.split_csr(torch.from_numpy(rp), gran)
        rps, tr = oracle.split_csr(rp, gran)
        assert np.array_equal(a.numpy(), rps) and np.array_equal(b.numpy(), tr)


def test_bcsr_matches_scipy_golden(oracle, golden_dir):
    z, n = _cases(os.path.join(golden_dir, "bcsr_scipy.npz"))
    for i in range(n):
        rp, ci, v, V = z["rowPtr_%d" % i], z["colIdx_%d" % i], z["val_%d" % i], int(z["V_%d" % i])
        rpb, cb, vb = oracle.bcsr_build(rp, ci, v, n_cols=rp.shape[0] - 1, V=V)
        assert np.array_equal(rpb, z["rowPtr_b_%d" % i])
        assert np.array_equal(cb, z["colIdx_b_%d" % i])
        assert np.array_equal(vb, z["val_b_%d" % i])


def test_bcsr_matches_live_scipy(oracle):
    rng = np.random.default_rng(3)
    n = 200
    a = sp.random_array((n, n), density=0.05, rng=rng, format="csr", dtype=np.float32)
    a.sort_indices()
    b = a.tobsr(blocksize=(2, 1))
    rpb, cb, vb = oracle.bcsr_build(a.indptr, a.indices, a.data, n_cols=n, V=2)
    assert np.array_equal(rpb, b.indptr) and np.array_equal(cb, b.indices)
    assert np.array_equal(vb, b.data.reshape(-1, 2))


def test_spmm_matches_torch_and_scipy_golden(oracle, golden_dir):
    z = np.load(os.path.join(golden_dir, "spmm_torch.npz"))
    rp, ci, v, B = z["rowPtr"], z["colIdx"], z["val"], z["B"]
    for acc64 in (True, False):
        C = oracle.spmm_csr(rp, ci, v, B, acc64=acc64)
        np.testing.assert_allclose(C, z["C_scipy"], rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(C, z["C_torch"], rtol=1e-5, atol=1e-5)
        assert oracle.verification_compare(z["C_torch"], C, rel=1e-4) or acc64 is False
    np.testing.assert_allclose(oracle.spmm_torch_cpu(rp, ci, v, B), z["C_torch"], rtol=0, atol=0)


def test_split_and_block_spmm_agree_with_plain(oracle, golden_dir):
    z = np.load(os.path.join(golden_dir, "spmm_torch.npz"))
    rp, ci, v, B = z["rowPtr"], z["colIdx"], z["val"], z["B"]
    n = rp.shape[0] - 1
    C = oracle.spmm_csr(rp, ci, v, B)
    rps, tr = oracle.split_csr(rp, 4)
    np.testing.assert_allclose(oracle.spmm_csr_split(rps, tr, ci, v, B, n), C, rtol=1e-6, atol=1e-6)
    for V in (2, 3):
        rpb, cb, vb = oracle.bcsr_build(rp, ci, v, n_cols=n, V=V)
        nbr = rpb.shape[0] - 1
        Cb = oracle.spmm_bcsr(rpb, cb, vb, B, nbr)
        assert Cb.shape[0] == nbr * V
        np.testing.assert_allclose(Cb[:n], C, rtol=1e-6, atol=1e-6)
        assert not Cb[n:].any()
        s_rpb, s_tr = oracle.split_csr(rpb, 3)
        Cs = oracle.spmm_bcsr(s_rpb, cb, vb, B, nbr, target_row=s_tr)
        np.testing.assert_allclose(Cs[:n], C, rtol=1e-6, atol=1e-6)


def test_sddmm_matches_dense_product(oracle, golden_dir):
    z = np.load(os.path.join(golden_dir, "spmm_torch.npz"))
    rp, ci, v = z["rowPtr"], z["colIdx"], z["val"]
    n = rp.shape[0] - 1
    rng = np.random.default_rng(0)
    A = rng.standard_normal((n + 1, 24)).astype(np.float32)
    Bm = rng.standard_normal((n, 24)).astype(np.float32)
    full = A.astype(np.float64) @ Bm.astype(np.float64).T
    rows = np.repeat(np.arange(n), np.diff(rp))
    want = full[rows, ci].astype(np.float32)
    got = oracle.sddmm_csr(rp, ci, A, Bm)
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)
    rps, tr = oracle.split_csr(rp, 5)
    np.testing.assert_allclose(oracle.sddmm_csr(rps, ci, A, Bm, target_row=tr), want, rtol=1e-6, atol=1e-6)
    rpb, cb, vb = oracle.bcsr_build(rp, ci, v, n_cols=n, V=2)
    ob = oracle.sddmm_bcsr(rpb, cb, vb, A, Bm)
    brow = np.repeat(np.arange(rpb.shape[0] - 1), np.diff(rpb))
    for u in (0, 1):
        w = np.where(vb[:, u] != 0, full[np.minimum(brow * 2 + u, n), cb], 0.0).astype(np.float32)
        np.testing.assert_allclose(ob[:, u], w, rtol=1e-6, atol=1e-6)


def test_genmask_hand_worked(oracle):
    # rows: 0 -> cols [1,5]; 1 -> cols [0,5,7]; 2 -> []; 3 -> [2]   (n = 4, 2 block rows)
    rp = np.array([0, 2, 5, 5, 6], dtype=np.int32)
    ci = np.array([1, 5, 0, 5, 7, 2], dtype=np.int32)
    v = np.arange(1, 7, dtype=np.float32)
    rpb, cb, vb = oracle.bcsr_build(rp, ci, v, n_cols=8, V=2)
    # first-encounter block order: block-row 0 -> [1,5,0,7], block-row 1 -> [2]
    assert cb.tolist() == [1, 5, 0, 7, 2]
    assert vb.tolist() == [[1, 0], [2, 4], [0, 3], [0, 5], [0, 6]]
    mask = oracle.genmask(rpb, rp, vb, nnz=6)
    # row 0 entries -> flat 0, 2; row 1 entries in block order (col 5, 0, 7) -> flat 3, 5, 7;
    # row 3 -> flat 9.  (The map follows block order, not column order, inside odd rows.)
    assert mask.tolist() == [0, 2, 3, 5, 7, 9]


def test_genmask_is_a_permutation_onto_nonzero_lanes(oracle):
    rng = np.random.default_rng(11)
    n = 301  # odd: exercises the padded last block row
    a = sp.random_array((n, n), density=0.03, rng=rng, format="csr", dtype=np.float32)
    a.sort_indices()
    a.data[:] = rng.random(a.nnz).astype(np.float32) + 0.5
    rpb, cb, vb = oracle.bcsr_build(a.indptr, a.indices, a.data, n_cols=n, V=2)
    mask = oracle.genmask(rpb, a.indptr, vb, nnz=a.nnz)
    flat = vb.reshape(-1)
    assert np.array_equal(np.sort(mask), np.flatnonzero(flat))
    # even rows keep column order, so gathering through the mask returns their CSR values
    rows = np.repeat(np.arange(n), np.diff(a.indptr))
    even = rows % 2 == 0
    assert np.array_equal(flat[mask][even], a.data[even])
    # every position maps into the block row and lane of its own CSR row
    blk_row = np.repeat(np.arange(rpb.shape[0] - 1), np.diff(rpb))
    assert np.array_equal(blk_row[mask // 2] * 2 + mask % 2, rows)


def test_decider_decode_rules(oracle):
    # PCSR.py:19-42 worked by hand
    assert oracle.dynamic_CF_prompter(64) == [1, 2]
    assert oracle.dynamic_CF_prompter(128) == [1, 2, 4]
    assert oracle.dynamic_CF_prompter(256) == [1, 2, 4, 8]
    assert oracle.dynamic_CF_prompter(96) == [1, 3]
    assert oracle.dynamic_CF_prompter(160) == [1, 5]
    assert oracle.dynamic_CF_prompter(224) == [1, 7]
    assert oracle.dynamic_CF_prompter(16) == [1]
    assert oracle.gap_calculator(80, 2) == 48 and oracle.gap_calculator(80, 3) == 0
    assert oracle.dynamic_CF_prompter(80) == [1, 3]
    # decider.py:52-55
    assert [oracle.model_dim_for(d) for d in (16, 32, 47, 48, 64, 100, 128, 200)] == \
        [16, 32, 48, 48, 64, 112, 128, 208]
    # decider.py:63-80: code layout = split + 2*vec + 4*cf_index + 4*len(cf)*warp_index
    assert oracle.decode_tree(0, 64) == (0, 1, 1, 4)
    assert oracle.decode_tree(1, 64) == (1, 1, 1, 4)
    assert oracle.decode_tree(2, 64) == (0, 2, 1, 4)
    assert oracle.decode_tree(7, 64) == (1, 2, 2, 4)
    assert oracle.decode_tree(8, 64) == (0, 1, 1, 8)
    assert oracle.decode_tree(15, 64) == (1, 2, 2, 8)
    assert oracle.decode_tree(23, 128) == (1, 2, 4, 8)


def test_pubmed_statistics(oracle, golden_dir):
    """The oracle's restatement of init_info reproduces the aggregates of the reference's toy
    matrix (read in place when the reference tree is mounted)."""
    stats = json.load(open(os.path.join(golden_dir, "pubmed_stats.json")))
    assert stats[0]["n"] == 19717 and stats[0]["nnz"] == 88651 and stats[0]["segments"] == 20005
    assert stats[0]["bcsr_blocks"] == 88469 and stats[1]["bcsr_blocks"] == 81018
    from oracle import build_oracle
    if not build_oracle.ref_available():
        pytest.skip("reference tree not mounted")
    from scipy.io import mmread
    import warnings
    for st in stats:
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            m = mmread(os.path.join(build_oracle.REF_ROOT, "toy_dataset", st["file"]))
        m.data = np.ones_like(m.data)
        csr = m.tocsr()
        info = oracle.csr_info(csr.indptr, csr.indices)
        assert info["max_row_nnz"] == st["max_deg"]
        assert info["split_granularity"] == st["split_granularity"]
        assert info["split_rows"] == st["segments"]
        assert abs(info["split_ratio"] - st["split_ratio"]) < 1e-12
        assert info["max_bw"] == st["max_bw"]
        assert abs(info["avg_bw"] - st["avg_bw"]) < 1e-2
        assert abs(info["COV"] - st["COV"]) < 1e-5
        rps, tr = oracle.split_csr(csr.indptr, info["split_granularity"])
        assert int(rps.astype(np.int64).sum()) == st["rowPtr_split_sum"]
        assert int(tr.astype(np.int64).sum()) == st["target_row_sum"]
        rpb, cb, vb = oracle.bcsr_build(csr.indptr, csr.indices, csr.data.astype(np.float32), csr.shape[0], 2)
        assert cb.shape[0] == st["bcsr_blocks"] and rpb.shape[0] == st["len_rowPtr_bcsr"]
        assert abs(csr.nnz / (2 * cb.shape[0]) - st["pack_rate"]) < 1e-12


def test_agnn_aggregate_restatement_is_the_sddmm_spmm_composition():
    """softmax=False must equal SDDMM -> * beta -> SpMM of the oracle's own pieces; softmax=True is
    checked on a case worked by hand."""
    import numpy as np
    from oracle import oracle as orc
    rng = np.random.default_rng(5)
    n, dim = 37, 12
    lens = rng.integers(0, 6, size=n)
    rowPtr = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    colIdx = rng.integers(0, n, size=int(rowPtr[-1])).astype(np.int32)
    X = rng.standard_normal((n, dim)).astype(np.float32)
    e = orc.sddmm_csr(rowPtr, colIdx, X, X) * np.float32(0.6)
    want = orc.spmm_csr(rowPtr, colIdx, e, X)
    got = orc.agnn_aggregate(rowPtr, colIdx, X, X, 0.6, softmax=False)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    # two entries with scores 0 and ln 3: weights 1/4 and 3/4
    A = np.array([[1.0, 0.0]], dtype=np.float32)
    B = np.array([[0.0, 2.0], [np.log(3.0), 4.0]], dtype=np.float32)
    out = orc.agnn_aggregate(np.array([0, 2]), np.array([0, 1]), A, B, 1.0, softmax=True)
    np.testing.assert_allclose(out, [[0.75 * np.log(3.0), 0.25 * 2.0 + 0.75 * 4.0]], rtol=1e-6)
