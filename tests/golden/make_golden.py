#!/usr/bin/env python3
"""Regenerates the golden vectors in this directory.  Run from the repository root:

    python tests/golden/make_golden.py

What each file pins and where its numbers come from:

* ``split_ref.npz``   PCSR partitions produced by the REFERENCE's own compiled host code
  (``split_csr`` and ``split_csr_par`` of SpMM/SpMM.cpp:15-75, built by
  ``oracle/build_oracle.py`` into ``oracle/_ref``) on seeded row-pointer arrays, including
  empty rows, rows that are exact multiples of the granularity and one long row.
* ``bcsr_scipy.npz``  2x1 and 3x1 block layouts produced by scipy's ``tobsr`` through the
  same steps as graph_input.py:245-266 of the reference (odd row counts are padded).
* ``spmm_torch.npz``  a small CSR matrix, a dense operand and ``torch.sparse.mm`` on CPU, the
  reference's acceptance oracle (verification.py:18-46), plus scipy's product.
* ``pubmed_stats.json``  aggregates of the reference's toy matrix
  (toy_dataset/pubmed.mtx and toy_dataset/rabbit/pubmed_rabbit.mtx, read in place, never
  copied): sizes, degree statistics, split counts, block counts and pack rate, computed with
  scipy and the reference's compiled ``split_csr``.

Needs the reference tree to be mounted (location: PSPMM_REFERENCE_ROOT, see oracle/build_oracle.py) because it runs the
reference's code; the tests only read the files written here.
"""
import json
import os
import sys

import numpy as np
import scipy.sparse as sp
import torch
from scipy.io import mmread

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import build_oracle  # noqa: E402

REF_ROOT = build_oracle.REF_ROOT


def random_rowptr(rng, n, mean, heavy=0):
    ln = rng.poisson(mean, size=n)
    ln[rng.random(n) < 0.15] = 0
    ln[rng.integers(0, n, size=max(1, n // 10))] = 32
    ln[rng.integers(0, n, size=max(1, n // 10))] = 64
    if heavy:
        ln[rng.integers(0, n)] = heavy
    return np.concatenate([[0], np.cumsum(ln)]).astype(np.int32)


def make_split(ref):
    rng = np.random.default_rng(1234)
    out = {}
    cases = [(1, 5, 0, 32), (17, 3, 0, 1), (64, 20, 0, 32), (257, 40, 5000, 32), (100, 10, 777, 7),
             (33, 100, 0, 64), (5, 0, 0, 32)]
    for i, (n, mean, heavy, gran) in enumerate(cases):
        rp = random_rowptr(rng, n, mean, heavy) if mean else np.zeros(n + 1, dtype=np.int32)
        rps, tr = ref.split_csr(torch.from_numpy(rp), gran)
        pieces = np.ceil((rp[1:] - rp[:-1]) / gran).astype(np.int64)
        off = torch.from_numpy(np.concatenate([[0], np.cumsum(pieces)]).astype(np.int32))
        rps2, tr2 = ref.split_csr_par(torch.from_numpy(rp), off, gran)
        assert torch.equal(rps, rps2) and torch.equal(tr, tr2)
        out["rowPtr_%d" % i] = rp
        out["gran_%d" % i] = np.int32(gran)
        out["rowPtr_split_%d" % i] = rps.numpy()
        out["target_row_%d" % i] = tr.numpy()
    out["n_cases"] = np.int32(len(cases))
    np.savez_compressed(os.path.join(HERE, "split_ref.npz"), **out)


def scipy_blocks(csr, V):
    """graph_input.py:245-266 of the reference, parameterised by the block height."""
    n, nnz = csr.shape[0], csr.nnz
    if n % V == 0:
        b = csr.tobsr(blocksize=(V, 1))
    else:
        res = V - n % V
        rp = np.concatenate([csr.indptr, [nnz] * res])
        b = sp.csr_array((csr.data, csr.indices, rp), shape=(n + res, n + res)).tobsr(blocksize=(V, 1))
    return b.indptr.astype(np.int32), b.indices.astype(np.int32), b.data.squeeze().astype(np.float32).reshape(-1, V)


def random_csr(rng, n, mean):
    rp = random_rowptr(rng, n, mean)
    cols = np.concatenate([np.sort(rng.choice(n, size=k, replace=False)) for k in np.minimum(rp[1:] - rp[:-1], n)]
                          or [np.zeros(0, dtype=np.int64)])
    rp = np.concatenate([[0], np.cumsum(np.minimum(rp[1:] - rp[:-1], n))]).astype(np.int32)
    val = (rng.random(cols.shape[0]) + 0.25).astype(np.float32)
    return sp.csr_array((val, cols.astype(np.int32), rp), shape=(n, n))


def make_bcsr():
    rng = np.random.default_rng(99)
    out = {}
    cases = [(64, 6, 2), (65, 6, 2), (37, 9, 3), (38, 9, 3), (39, 2, 3), (9, 80, 2)]
    for i, (n, mean, V) in enumerate(cases):
        a = random_csr(rng, n, min(mean, n // 2))
        rpb, cb, vb = scipy_blocks(a, V)
        out["rowPtr_%d" % i] = a.indptr.astype(np.int32)
        out["colIdx_%d" % i] = a.indices.astype(np.int32)
        out["val_%d" % i] = a.data.astype(np.float32)
        out["V_%d" % i] = np.int32(V)
        out["rowPtr_b_%d" % i] = rpb
        out["colIdx_b_%d" % i] = cb
        out["val_b_%d" % i] = vb
    out["n_cases"] = np.int32(len(cases))
    np.savez_compressed(os.path.join(HERE, "bcsr_scipy.npz"), **out)


def make_spmm():
    rng = np.random.default_rng(7)
    n, dim = 96, 20
    a = random_csr(rng, n, 7)
    B = (rng.random((n, dim)) * 2 - 1).astype(np.float32)
    s = torch.sparse_csr_tensor(torch.from_numpy(a.indptr.astype(np.int32)),
                                torch.from_numpy(a.indices.astype(np.int32)),
                                torch.from_numpy(a.data.astype(np.float32)), size=(n, n))
    C_torch = torch.sparse.mm(s, torch.from_numpy(B)).numpy()
    C_scipy = (a.astype(np.float64) @ B.astype(np.float64)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "spmm_torch.npz"), rowPtr=a.indptr.astype(np.int32),
                        colIdx=a.indices.astype(np.int32), val=a.data.astype(np.float32), B=B,
                        C_torch=C_torch, C_scipy=C_scipy)


def pubmed_stats(ref, rel):
    m = mmread(os.path.join(REF_ROOT, "toy_dataset", rel))
    m.data = np.ones_like(m.data)  # graph_input.py:227
    csr = m.tocsr()
    n, nnz = csr.shape[0], csr.nnz
    ln = np.diff(csr.indptr)
    avg = nnz / n
    gran = int(np.ceil(avg / 32) * 32)
    rps, tr = ref.split_csr(torch.from_numpy(csr.indptr.astype(np.int32)), gran)
    rpb, cb, vb = scipy_blocks(csr, 2)
    nz = ln != 0
    bw = csr.indices[csr.indptr[1:][nz] - 1] - csr.indices[csr.indptr[:-1][nz]]
    cov = float(torch.from_numpy(ln).float().std() / avg)
    return {"file": rel, "n": int(n), "nnz": int(nnz), "diag": int((csr.diagonal() != 0).sum()),
            "min_deg": int(ln.min()), "max_deg": int(ln.max()), "avg_deg": avg, "COV": cov,
            "split_granularity": gran, "segments": int(tr.shape[0]),
            "split_ratio": int(tr.shape[0]) / int(nz.sum()),
            "max_bw": int(bw.max()), "avg_bw": float(bw.sum() / nz.sum()),
            "bcsr_blocks": int(cb.shape[0]), "pack_rate": nnz / (2 * cb.shape[0]),
            "len_rowPtr_bcsr": int(rpb.shape[0]),
            "rowPtr_split_sum": int(rps.astype(np.int64).sum() if isinstance(rps, np.ndarray) else rps.long().sum()),
            "target_row_sum": int(tr.long().sum())}


def main():
    build_oracle.build_ref()
    ref = build_oracle.load_ref()
    if ref is None:
        raise SystemExit("the reference tree is not mounted; cannot regenerate golden vectors")
    make_split(ref)
    make_bcsr()
    make_spmm()
    stats = [pubmed_stats(ref, "pubmed.mtx"), pubmed_stats(ref, os.path.join("rabbit", "pubmed_rabbit.mtx"))]
    with open(os.path.join(HERE, "pubmed_stats.json"), "w") as f:
        json.dump(stats, f, indent=1)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
