"""Acceptance check: mirror of the reference's ``SpMM_verification`` (verification.py:10-102).

The reference result is ``torch.sparse.mm`` on a CSR tensor, computed on the CPU here (the
reference defaults to computing it on the GPU, i.e. with cuSPARSE; the CPU result is the
independent one).  ``compare`` applies the reference's rule: no element may differ from the
reference by more than ``1e-4 * |reference|``.
"""
from __future__ import annotations

import time

import torch


class SpMM_verification(object):
    def __init__(self, dim, rowPtr, colIdx, val, baseline=False, baseline_round=100):
        self.baseline, self.baseline_round = baseline, baseline_round
        self.rowPtr, self.colIdx, self.csr_val = rowPtr, colIdx, val
        self.num_nodes = len(rowPtr) - 1
        self.s = torch.sparse_csr_tensor(rowPtr, colIdx, val, size=(self.num_nodes, self.num_nodes))
        self.test_embedding = dim
        self.X = torch.ones(self.num_nodes, dim)
        self.result_ref = None
        self.result = None

    def reference(self, dim=None, device="cpu", x=None):
        if device not in ("cpu", "cuda"):
            raise ValueError("device must be 'cpu' or 'cuda'")
        if x is not None:
            X = x.to(device)
        elif dim is None:
            X = self.X.to(device)
        else:
            X = torch.ones(self.num_nodes, dim, device=device)
        self.result_ref = torch.sparse.mm(self.s.to(device), X).to("cpu")
        return self.result_ref

    def torch_compute(self, device):
        """Times torch.sparse.mm (10 warm-ups, baseline_round timed runs); returns (result, GFLOP/s)."""
        X, s = self.X.to(device), self.s.to(device)
        self.result = torch.sparse.mm(s, X)
        if not self.baseline:
            return self.result, None
        for _ in range(10):
            torch.sparse.mm(s, X)
        if device == "cuda":
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(self.baseline_round):
            self.result = torch.sparse.mm(s, X)
        if device == "cuda":
            torch.cuda.synchronize()
        dur = (time.perf_counter() - t0) / self.baseline_round
        gflop = 2 * int(self.rowPtr[-1]) / 1e9 * self.test_embedding
        return self.result, int(gflop / dur)

    def compare(self, result, mtx_name=""):
        if self.result_ref is None or result is None:
            raise ValueError("MUST compute result and result reference (CPU) first!!")
        bad = (self.result_ref - result).abs() > 1e-4 * self.result_ref.abs()
        if bad.any():
            r, c = [int(i) for i in torch.nonzero(bad)[0]]
            raise ValueError("Verification FAILED in {}: first mismatch at ({}, {}): expected {}, found {}".format(
                mtx_name, r, c, self.result_ref[r, c].item(), result[r, c].item()))
        return True
