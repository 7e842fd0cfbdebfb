"""cuSPARSE comparators behind the names the reference exposes from its extension modules
(SpMM/SpMM.cpp:915-925, SDDMM/sddmm.cpp:696-697).  They call libpspmm_baselines.so, which is
separate from the product library and links cuSPARSE; they are measurement baselines, not
part of the SpMM/SDDMM path.

``gespmm_*``: the reference vendors a third-party kernel (SpMM/Baseline_kernel.cu:601-857); here the
comparator is this library's own restatement of the published GE-SpMM algorithm (coalesced row
caching + coarse-grained warp merging), see csrc/baselines.cu.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib
from .ops import PROFILE_ITERS, PROFILE_WARMUP, _check_cuda, _gflops, _ptr, _stream

_handle = None


def _bl():
    global _handle
    if _handle is None:
        if not os.path.exists(_lib.BASELINES_PATH):
            raise ImportError("%s not found: build it with `python -m paramspmm_ae_b200.build`"
                              % _lib.BASELINES_PATH)
        h = ctypes.CDLL(_lib.BASELINES_PATH)
        h.pspmm_baselines_last_error.restype = ctypes.c_char_p
        _handle = h
    return _handle


def _ok(rc):
    if rc != 0:
        raise RuntimeError("baseline call failed: " + _bl().pspmm_baselines_last_error().decode())


class _Plan:
    def __init__(self, handle):
        self.h = handle

    def run(self):
        _ok(_bl().pspmm_baselines_run(self.h, _stream()))

    def close(self):
        if self.h:
            _bl().pspmm_baselines_plan_destroy(self.h)
            self.h = None

    def __del__(self):
        self.close()


def spmm_plan(fmt, idx0, idx1, val, X, out, n_rows=None):
    """fmt: 0 CSR default algorithm, 1 CSR ALG2, 2 COO, 3 CSC."""
    for t, nm in ((idx0, "idx0"), (idx1, "idx1")):
        _check_cuda(t, nm, torch.int32, 1)
    _check_cuda(val, "values", torch.float32, 1)
    _check_cuda(X, "input", torch.float32, 2)
    n_cols, dim = X.shape
    if n_rows is None:
        n_rows = out.shape[0]
    h = ctypes.c_void_p(0)
    _ok(_bl().pspmm_baselines_spmm_plan(ctypes.byref(h), int(fmt), _ptr(idx0), _ptr(idx1), _ptr(val),
                                        _ptr(X), _ptr(out), ctypes.c_int64(n_rows),
                                        ctypes.c_int64(n_cols), ctypes.c_int64(val.shape[0]),
                                        ctypes.c_int32(dim), ctypes.c_int64(X.stride(0)),
                                        ctypes.c_int64(out.stride(0))))
    return _Plan(h)


def sddmm_plan(A, B, rowPtr, colIdx, val_out):
    _check_cuda(A, "A", torch.float32, 2)
    _check_cuda(B, "B", torch.float32, 2)
    h = ctypes.c_void_p(0)
    _ok(_bl().pspmm_baselines_sddmm_plan(ctypes.byref(h), _ptr(rowPtr), _ptr(colIdx), _ptr(val_out),
                                         _ptr(A), _ptr(B), ctypes.c_int64(rowPtr.shape[0] - 1),
                                         ctypes.c_int64(B.shape[0]), ctypes.c_int64(colIdx.shape[0]),
                                         ctypes.c_int32(A.shape[1]), ctypes.c_int64(A.stride(0)),
                                         ctypes.c_int64(B.stride(0))))
    return _Plan(h)


def time_plan_ms(plan, warmup=PROFILE_WARMUP, iters=PROFILE_ITERS):
    for _ in range(warmup):
        plan.run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        plan.run()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / iters


def _compute(fmt, X, i0, i1, val):
    out = torch.empty_like(X)
    plan = spmm_plan(fmt, i0, i1, val, X, out)
    plan.run()
    torch.cuda.current_stream().synchronize()
    plan.close()
    return out


def _profile(fmt, X, i0, i1, val):
    out = torch.empty_like(X)
    plan = spmm_plan(fmt, i0, i1, val, X, out)
    ms = time_plan_ms(plan)
    plan.close()
    return _gflops(val.shape[0], X.shape[1], ms)


def cusparse_compute(X, rowPtr, colIdx, val):
    return _compute(0, X, rowPtr, colIdx, val)


def cusparse_profile(X, rowPtr, colIdx, val):
    return _profile(0, X, rowPtr, colIdx, val)


def cusparse_compute_csr_alg2(X, rowPtr, colIdx, val):
    return _compute(1, X, rowPtr, colIdx, val)


def cusparse_profile_csr_alg2(X, rowPtr, colIdx, val):
    return _profile(1, X, rowPtr, colIdx, val)


def cusparse_compute_coo_alg4(X, row, col, val):
    return _compute(2, X, row, col, val)


def cusparse_profile_coo_alg4(X, row, col, val):
    return _profile(2, X, row, col, val)


def cusparse_compute_csc(X, colPtr, rowIdx, val):
    return _compute(3, X, colPtr, rowIdx, val)


def cusparse_profile_csc(X, colPtr, rowIdx, val):
    return _profile(3, X, colPtr, rowIdx, val)


def cusparse_sddmm_compute(A, B, rowPtr, colIdx, val):
    """Overwrites `val` in place, as the reference's wrapper does
    (SDDMM/sddmm_baseline_kernel.cu:24-80)."""
    plan = sddmm_plan(A, B, rowPtr, colIdx, val)
    plan.run()
    torch.cuda.current_stream().synchronize()
    plan.close()
    return val


def cusparse_sddmm_profile(A, B, rowPtr, colIdx, val):
    plan = sddmm_plan(A, B, rowPtr, colIdx, val)
    ms = time_plan_ms(plan)
    plan.close()
    return _gflops(colIdx.shape[0], A.shape[1], ms)


def _gespmm(X, rowPtr, colIdx, val, out):
    _check_cuda(X, "input", torch.float32, 2)
    _check_cuda(rowPtr, "rowPtr", torch.int32, 1)
    _check_cuda(colIdx, "colIdx", torch.int32, 1)
    _check_cuda(val, "values", torch.float32, 1)
    _ok(_bl().pspmm_baselines_gespmm(_ptr(rowPtr), _ptr(colIdx), _ptr(val), _ptr(X), _ptr(out),
                                     ctypes.c_int64(rowPtr.shape[0] - 1), ctypes.c_int32(X.shape[1]),
                                     ctypes.c_int64(X.stride(0)), ctypes.c_int64(out.stride(0)), _stream()))
    return out


def gespmm_compute(X, rowPtr, colIdx, val):
    out = torch.empty(rowPtr.shape[0] - 1, X.shape[1], dtype=torch.float32, device=X.device)
    return _gespmm(X, rowPtr, colIdx, val, out)


def gespmm_time_ms(X, rowPtr, colIdx, val, warmup=PROFILE_WARMUP, iters=PROFILE_ITERS):
    out = torch.empty(rowPtr.shape[0] - 1, X.shape[1], dtype=torch.float32, device=X.device)
    for _ in range(warmup):
        _gespmm(X, rowPtr, colIdx, val, out)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        _gespmm(X, rowPtr, colIdx, val, out)
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / iters


def gespmm_profile(X, rowPtr, colIdx, val):
    return _gflops(val.shape[0], X.shape[1], gespmm_time_ms(X, rowPtr, colIdx, val))


def gather_ceiling_ms(colIdx, B, run=64, warmup=3, iters=10):
    """Milliseconds the GPU needs just to fetch B[colIdx[k]] for every k (8 row loads in flight per
    lane, nothing else): the floor of any row-major-gather SpMM over this column stream and dense
    operand (see csrc/baselines.cu).  dim must be a multiple of 4."""
    _check_cuda(colIdx, "colIdx", torch.int32, 1)
    _check_cuda(B, "B", torch.float32, 2)
    nnz, dim = colIdx.shape[0], B.shape[1]
    h = _bl()
    h.pspmm_baselines_gather_sink_bytes.restype = ctypes.c_int64
    nbytes = h.pspmm_baselines_gather_sink_bytes(ctypes.c_int64(nnz), ctypes.c_int32(dim), ctypes.c_int32(run))
    sink = torch.empty(nbytes // 4, dtype=torch.float32, device=B.device)

    def go():
        _ok(h.pspmm_baselines_gather_ceiling(_ptr(colIdx), ctypes.c_int64(nnz), _ptr(B), ctypes.c_int32(dim),
                                             ctypes.c_int64(B.stride(0)), ctypes.c_int32(run), _ptr(sink), _stream()))

    for _ in range(warmup):
        go()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        go()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / iters
