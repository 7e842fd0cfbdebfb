"""The library's MatrixMarket reader and binary CSR container (host only).

Oracle: scipy's ``mmread(...).tocsr()``, which is what the reference's loader runs
(graph_input.py:226-232) -- row pointers and column indices must be identical, values
bit-identical after the cast to float32.
"""
import os

import numpy as np
import pytest
import torch

scipy_io = pytest.importorskip("scipy.io")
import scipy.sparse as sp  # noqa: E402

from paramspmm_ae_b200 import _lib, ops  # noqa: E402
from paramspmm_ae_b200.graph_input import graph_input  # noqa: E402

pytestmark = pytest.mark.filterwarnings("ignore")


def scipy_csr(path, ones):
    m = scipy_io.mmread(path)
    if ones:
        m.data = np.ones_like(m.data)  # graph_input.py:227
    c = sp.csr_matrix(m.tocsr())
    c.sum_duplicates()
    c.sort_indices()
    return c


def same_as_scipy(path):
    for ones in (True, False):
        rp, ci, v, nr, nc = ops.mtx_read_csr(path, force_ones=ones)
        want = scipy_csr(path, ones)
        assert (nr, nc) == want.shape
        assert rp.dtype == torch.int32 and ci.dtype == torch.int32 and v.dtype == torch.float32
        assert np.array_equal(rp.numpy(), want.indptr)
        assert np.array_equal(ci.numpy(), want.indices)
        assert np.array_equal(v.numpy(), want.data.astype(np.float32))


HAND_WRITTEN = {
    "general_real": "%%MatrixMarket matrix coordinate real general\n% comment\n\n%another\n 4 5 7\n"
                    "1 1 1.5\n4 5 -2e-3\n2 3 7\n2 3 1\n\n3 1 .5\n1 5 1E2\n  4   1\t3.25  \n",
    "symmetric_pattern_no_final_newline": "%%MatrixMarket matrix coordinate pattern symmetric\n3 3 4\n1 1\n2 1\n3 1\n3 3",
    "skew_integer_crlf_mixed_case": "%%MatrixMarket MATRIX Coordinate Integer Skew-Symmetric\r\n3 3 2\r\n2 1 4\r\n3 2 -5\r\n",
    "no_entries": "%%MatrixMarket matrix coordinate real general\n5 7 0\n",
    "no_rows": "%%MatrixMarket matrix coordinate real general\n0 0 0\n",
    "rectangular_pattern": "%%MatrixMarket matrix coordinate pattern general\n2 9 3\n2 9\n1 1\n2 1\n",
}


@pytest.mark.parametrize("name", sorted(HAND_WRITTEN))
def test_hand_written_files_match_scipy(tmp_path, name):
    path = str(tmp_path / (name + ".mtx"))
    with open(path, "w", newline="") as f:
        f.write(HAND_WRITTEN[name])
    same_as_scipy(path)


def test_random_files_match_scipy(tmp_path):
    rng = np.random.default_rng(5)
    n, k = 3000, 200_000  # dense enough that many coordinates repeat: exercises the summation
    A = sp.coo_matrix((rng.standard_normal(k), (rng.integers(0, n, k), rng.integers(0, n, k))), shape=(n, n))
    path = str(tmp_path / "general.mtx")
    scipy_io.mmwrite(path, A)
    info = ops.mtx_info(path)
    assert info["stored"] == k and info["symmetric"] == 0 and info["field"] == 1
    rp, ci, v, _, _ = ops.mtx_read_csr(path, force_ones=True)
    want = scipy_csr(path, True)
    assert want.nnz < k and want.data.max() >= 2.0  # repeated coordinates were present
    assert np.array_equal(rp.numpy(), want.indptr) and np.array_equal(ci.numpy(), want.indices)
    assert np.array_equal(v.numpy(), want.data.astype(np.float32))
    # real values: sums of repeated coordinates may differ in the last bit of the double sum
    rp, ci, v, _, _ = ops.mtx_read_csr(path, force_ones=False)
    want = scipy_csr(path, False)
    assert np.array_equal(ci.numpy(), want.indices)
    np.testing.assert_allclose(v.numpy(), want.data.astype(np.float32), rtol=1e-6, atol=1e-7)
    U = sp.triu(A.tocsr(), 1)
    S = (U + U.T + sp.diags(rng.standard_normal(n))).tocoo()
    path = str(tmp_path / "symmetric.mtx")
    scipy_io.mmwrite(path, S, symmetry="symmetric")
    assert ops.mtx_info(path)["symmetric"] == 1
    same_as_scipy(path)


@pytest.mark.parametrize("text,code", [
    ("%%NotMatrixMarket matrix coordinate real general\n1 1 0\n", _lib.PSPMM_E_FORMAT),
    ("%%MatrixMarket matrix array real general\n1 1\n1.0\n", _lib.PSPMM_E_UNSUPPORTED),
    ("%%MatrixMarket matrix coordinate complex general\n1 1 1\n1 1 1 0\n", _lib.PSPMM_E_UNSUPPORTED),
    ("%%MatrixMarket matrix coordinate real general\n2 2 1\n3 1 1.0\n", _lib.PSPMM_E_FORMAT),   # row out of range
    ("%%MatrixMarket matrix coordinate real general\n2 2 1\n0 1 1.0\n", _lib.PSPMM_E_FORMAT),   # indices are 1-based
    ("%%MatrixMarket matrix coordinate real general\n2 2 2\n1 1 1.0\n", _lib.PSPMM_E_FORMAT),   # fewer lines than announced
    ("%%MatrixMarket matrix coordinate real general\n2 2 1\n1 1 1.0\n2 2 1.0\n", _lib.PSPMM_E_FORMAT),  # more
    ("%%MatrixMarket matrix coordinate real general\n2 2 1\n1 1\n", _lib.PSPMM_E_FORMAT),      # value missing
    ("%%MatrixMarket matrix coordinate real symmetric\n2 3 0\n", _lib.PSPMM_E_FORMAT),         # not square
    ("", _lib.PSPMM_E_FORMAT),
])
def test_malformed_files_are_rejected_with_a_code(tmp_path, text, code):
    path = str(tmp_path / "bad.mtx")
    with open(path, "w") as f:
        f.write(text)
    with pytest.raises(_lib.PspmmError) as e:
        ops.mtx_read_csr(path)
    assert e.value.code == code


def test_missing_file_is_an_io_error(tmp_path):
    with pytest.raises(_lib.PspmmError) as e:
        ops.mtx_info(str(tmp_path / "absent.mtx"))
    assert e.value.code == _lib.PSPMM_E_IO
    with pytest.raises(_lib.PspmmError) as e:
        ops.csr_file_info(str(tmp_path / "absent.bin"))
    assert e.value.code == _lib.PSPMM_E_IO


def random_csr(n, m, k, seed):
    rng = np.random.default_rng(seed)
    c = sp.csr_matrix((rng.random(k).astype(np.float32), (rng.integers(0, n, k), rng.integers(0, m, k))), shape=(n, m))
    c.sum_duplicates()
    c.sort_indices()
    return (torch.from_numpy(c.indptr.astype(np.int32)), torch.from_numpy(c.indices.astype(np.int32)),
            torch.from_numpy(c.data.astype(np.float32)))


def test_container_round_trip_and_damage(tmp_path):
    for n, m, k in ((1000, 700, 20_000), (1, 1, 1), (5, 5, 0)):
        rp, ci, v = random_csr(n, m, k, 3) if k else (torch.zeros(n + 1, dtype=torch.int32),
                                                      torch.empty(0, dtype=torch.int32), torch.empty(0))
        path = str(tmp_path / ("m%d.bin" % n))
        ops.csr_file_write(path, rp, ci, v, m)
        info = ops.csr_file_info(path)
        assert (info["n_rows"], info["n_cols"], info["nnz"]) == (n, m, ci.numel())
        got = ops.csr_file_read(path)
        assert torch.equal(got[0], rp) and torch.equal(got[1], ci) and torch.equal(got[2], v) and got[3:] == (n, m)
        assert not [f for f in os.listdir(tmp_path) if ".tmp." in f]  # written under another name, then renamed
    path = str(tmp_path / "m1000.bin")
    raw = bytearray(open(path, "rb").read())
    assert len(raw) % 4 == 0 and raw[:8] == b"PSPMMCSR"
    damaged = bytearray(raw)
    damaged[-5] ^= 0x40  # one bit of one stored value
    open(path, "wb").write(damaged)
    with pytest.raises(_lib.PspmmError) as e:
        ops.csr_file_read(path, verify=True)
    assert e.value.code == _lib.PSPMM_E_FORMAT
    ops.csr_file_read(path, verify=False)  # the caller may skip the checksum
    open(path, "wb").write(raw[:-8])  # truncated
    with pytest.raises(_lib.PspmmError) as e:
        ops.csr_file_info(path)
    assert e.value.code == _lib.PSPMM_E_FORMAT
    open(path, "wb").write(b"NOTACSR!" + bytes(raw[8:]))
    with pytest.raises(_lib.PspmmError):
        ops.csr_file_info(path)


def test_load_matrix_uses_and_refreshes_the_container(tmp_path):
    rng = np.random.default_rng(9)
    n, k = 500, 4000
    path = str(tmp_path / "g.mtx")
    scipy_io.mmwrite(path, sp.coo_matrix((np.ones(k), (rng.integers(0, n, k), rng.integers(0, n, k))), shape=(n, n)))
    cache = str(tmp_path / "cache")
    first = ops.load_matrix(path, cache)
    files = os.listdir(cache)
    assert len(files) == 1 and files[0].endswith(".pspmmcsr")
    cached = os.path.join(cache, files[0])
    stamp = os.stat(cached).st_mtime_ns
    again = ops.load_matrix(path, cache)
    assert os.stat(cached).st_mtime_ns == stamp  # read, not rewritten
    assert all(torch.equal(a, b) for a, b in zip(first[:3], again[:3])) and first[3:] == again[3:]
    # the text file changes: the container is stale and gets replaced
    scipy_io.mmwrite(path, sp.coo_matrix((np.ones(3), ([0, 1, 2], [2, 1, 0])), shape=(n, n)))
    fresh = ops.load_matrix(path, cache)
    assert fresh[1].numel() == 3 and ops.csr_file_info(cached)["nnz"] == 3
    # a damaged container is parsed over, not trusted
    raw = bytearray(open(cached, "rb").read())
    raw[-1] ^= 0xFF
    open(cached, "wb").write(raw)
    st = os.stat(path)
    os.utime(cached, ns=(st.st_atime_ns, st.st_mtime_ns))
    healed = ops.load_matrix(path, cache)
    assert torch.equal(healed[2], fresh[2]) and ops.csr_file_read(cached)[1].numel() == 3
    # an unwritable cache location still returns the arrays
    blocked = str(tmp_path / "file_not_dir")
    open(blocked, "w").write("x")
    assert ops.load_matrix(path, os.path.join(blocked, "sub"))[1].numel() == 3


def test_graph_input_load_equals_load_csr_of_scipy_arrays(tmp_path):
    rng = np.random.default_rng(2)
    n, k = 301, 2500  # odd row count: the block layout pads
    r, c = rng.integers(0, n, k), rng.integers(0, n, k)
    keep = r > c
    S = sp.coo_matrix((np.ones(keep.sum()), (r[keep], c[keep])), shape=(n, n))
    S.sum_duplicates()
    scipy_io.mmwrite(str(tmp_path / "toy.mtx"), S, symmetry="symmetric")
    for kw in ({}, {"is_normalize": True}, {"GIN_epsilon": 0.5}):
        g = graph_input("toy", str(tmp_path) + "/", cache_dir=str(tmp_path / "c"))
        g.load(**kw)
        m = scipy_io.mmread(str(tmp_path / "toy.mtx"))
        m.data = np.ones_like(m.data)
        if kw.get("is_normalize"):
            m = g.normalize_adj(m)
        elif "GIN_epsilon" in kw:
            m = g.normalize_adj_GIN(m, 0.5)
        want = sp.csr_matrix(m.tocsr())
        want.sort_indices()
        h = graph_input().load_csr(want.indptr, want.indices, want.data, n)
        assert torch.equal(g.csr_data.rowPtr, h.csr_data.rowPtr) and torch.equal(g.csr_data.colIdx, h.csr_data.colIdx)
        torch.testing.assert_close(g.csr_data.val, h.csr_data.val, rtol=1e-6, atol=1e-7)
        assert torch.equal(g.csr_data.rowPtr_split, h.csr_data.rowPtr_split)
        assert torch.equal(g.bcsr_data.colIdx, h.bcsr_data.colIdx) and g.pack_rate == h.pack_rate
        np.testing.assert_allclose(g.get_info(), h.get_info(), rtol=1e-12)
