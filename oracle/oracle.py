"""Python face of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this module.  It wraps
``oracle/liboracle.so`` (built from ``oracle/pspmm_oracle.c``) with numpy
arrays and restates, in numpy / plain Python, the small host-side rules of the
reference that are not worth writing in C.  Every function cites the reference
location it follows (path inside the reference project : lines).

Pinning status
--------------
* ``split_csr``: pinned against the reference's own compiled host code
  (``oracle/_ref/ParamSpMM_ref.so``, built from SpMM/SpMM.cpp where it lies)
  and against committed golden vectors generated from it.
* ``bcsr_build``: pinned against scipy's ``tobsr`` (the third-party routine
  the reference calls) and golden vectors.
* ``spmm_*``: pinned against ``torch.sparse.mm`` on CPU, the reference's own
  acceptance oracle (verification.py:18-46), and scipy ``csr @ dense``; on a
  GPU box also against the reference's own CUDA SpMM kernels
  (``oracle/_ref/ParamSpMM_cuda_ref.so``, tests/test_gpu_reference_cuda.py).
* ``genmask``, ``sddmm_*``: the reference holds no golden vectors for them;
  they are pinned on a GPU box against the reference's own CUDA kernels
  (``oracle/_ref/ParamSDDMM_ref.so``, the reference's SDDMM extension compiled
  unmodified for sm_100a, tests/test_gpu_reference_cuda.py: ``genmask`` bit for
  bit, SDDMM within 1e-5 relative).  Without a GPU only hand-worked cases pin
  them.
* decider decode rules: pinned by hand-evaluated cases of decider.py:63-80.
"""
from __future__ import annotations

import ctypes
import math
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)
_i64 = ctypes.c_int64
_i32 = ctypes.c_int32


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            from . import build_oracle

            build_oracle.build_oracle()
        _LIB = ctypes.CDLL(path)
        _LIB.orc_split_csr.restype = _i64
        _LIB.orc_bcsr_build.restype = _i64
        _LIB.orc_num_threads.restype = ctypes.c_int
    return _LIB


def _pi(a):
    return a.ctypes.data_as(_i32p) if a is not None else None


def _pf(a):
    return a.ctypes.data_as(_f32p) if a is not None else None


def _ci(a):
    return np.ascontiguousarray(a, dtype=np.int32)


def _cf(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def num_threads():
    return int(_lib().orc_num_threads())


# --------------------------------------------------------------------------- index builders
def split_csr(rowPtr, gran):
    """PCSR partition (SpMM/SpMM.cpp:15-40): returns (rowPtr_split[S+1], target_row[S])."""
    rowPtr = _ci(rowPtr)
    n = rowPtr.shape[0] - 1
    if gran <= 0:
        raise ValueError("granularity must be positive")
    s = _lib().orc_split_csr(_pi(rowPtr), _i64(n), _i32(gran), None, None)
    rps = np.zeros(s + 1, dtype=np.int32)
    tr = np.zeros(s, dtype=np.int32)
    _lib().orc_split_csr(_pi(rowPtr), _i64(n), _i32(gran), _pi(rps), _pi(tr))
    return rps, tr


def split_csr_numpy(rowPtr, gran):
    """Same arrays as :func:`split_csr`, vectorised (second restatement, used as a cross-check)."""
    rowPtr = np.asarray(rowPtr, dtype=np.int64)
    ln = rowPtr[1:] - rowPtr[:-1]
    pieces = (ln + gran - 1) // gran
    off = np.concatenate([[0], np.cumsum(pieces)])
    s = int(off[-1])
    tr = np.repeat(np.arange(ln.shape[0], dtype=np.int64), pieces)
    idx_in_row = np.arange(s, dtype=np.int64) - off[tr]
    ends = np.minimum(rowPtr[tr] + (idx_in_row + 1) * gran, rowPtr[tr + 1])
    rps = np.concatenate([[0], ends])
    return rps.astype(np.int32), tr.astype(np.int32)


def row_split_counts(rowPtr, gran):
    """ceil(row_nnz / gran) per row as integers (graph_input.py:48-51 computes the same in fp32)."""
    rowPtr = np.asarray(rowPtr, dtype=np.int64)
    ln = rowPtr[1:] - rowPtr[:-1]
    return (ln + gran - 1) // gran


def bcsr_build(rowPtr, colIdx, val, n_cols, V=2):
    """V x 1 block CSR exactly as scipy's ``tobsr`` lays it out (graph_input.py:245-266).

    Returns (rowPtr_b[ceil(n/V)+1], colIdx_b[nblk], val_b[nblk, V]).
    """
    rowPtr, colIdx, val = _ci(rowPtr), _ci(colIdx), _cf(val)
    n = rowPtr.shape[0] - 1
    nbr = (n + V - 1) // V
    scratch = np.full(max(int(n_cols), 1), -1, dtype=np.int32)
    rpb = np.zeros(nbr + 1, dtype=np.int32)
    nblk = _lib().orc_bcsr_build(_pi(rowPtr), _pi(colIdx), _pf(val), _i64(n), _i32(V),
                                 _pi(scratch), _pi(rpb), None, None)
    cb = np.zeros(nblk, dtype=np.int32)
    vb = np.zeros((nblk, V), dtype=np.float32)
    _lib().orc_bcsr_build(_pi(rowPtr), _pi(colIdx), _pf(val), _i64(n), _i32(V), _pi(scratch),
                          _pi(rpb), _pi(cb), _pf(vb))
    return rpb, cb, vb


def genmask(rowPtr_b, rowPtr, val_b, nnz):
    """CSR-order -> flattened BCSR(2x1) index map (SDDMM/sddmm_kernel.cu:78-141)."""
    rowPtr_b, rowPtr, val_b = _ci(rowPtr_b), _ci(rowPtr), _cf(val_b)
    nbr = rowPtr_b.shape[0] - 1
    # The kernel reads rowPtr[2r] and rowPtr[2r+1]; with an odd row count the last
    # index equals n, which the (n+1)-long rowPtr still holds.
    assert rowPtr.shape[0] >= 2 * nbr
    mask = np.zeros(int(nnz), dtype=np.int32)
    _lib().orc_genmask(_pi(rowPtr_b), _pi(rowPtr), _pf(val_b), _i64(nbr), _pi(mask))
    return mask


# --------------------------------------------------------------------------- numeric kernels
def spmm_csr(rowPtr, colIdx, val, B, acc64=True):
    """C = A @ B, A in CSR (SpMM/SpMM_kernel.cu:1157-1243). fp64 accumulation unless acc64=False."""
    rowPtr, colIdx, val, B = _ci(rowPtr), _ci(colIdx), _cf(val), _cf(B)
    n, dim = rowPtr.shape[0] - 1, B.shape[1]
    C = np.empty((n, dim), dtype=np.float32)
    _lib().orc_spmm_csr(_pi(rowPtr), _pi(colIdx), _pf(val), _pf(B), _pf(C), _i64(n), _i32(dim),
                        _i64(B.shape[1]), _i64(dim), _i32(1 if acc64 else 0))
    return C


def spmm_csr_split(rowPtr_split, target_row, colIdx, val, B, n_rows):
    """SpMM over a row-split layout (SpMM/SpMM_kernel.cu:1245-1360)."""
    rps, tr, colIdx, val, B = _ci(rowPtr_split), _ci(target_row), _ci(colIdx), _cf(val), _cf(B)
    dim = B.shape[1]
    C = np.empty((n_rows, dim), dtype=np.float32)
    _lib().orc_spmm_csr_split(_pi(rps), _pi(tr), _i64(tr.shape[0]), _pi(colIdx), _pf(val), _pf(B),
                              _pf(C), _i64(n_rows), _i32(dim), _i64(dim), _i64(dim))
    return C


def spmm_bcsr(rowPtr_b, colIdx_b, val_b, B, n_blk_rows, target_row=None):
    """SpMM with V x 1 blocks, padded output of V*n_blk_rows rows (SpMM/SpMM_kernel.cu:1362-1972)."""
    rpb, cb, vb, B = _ci(rowPtr_b), _ci(colIdx_b), _cf(val_b), _cf(B)
    V, dim = vb.shape[1], B.shape[1]
    tr = _ci(target_row) if target_row is not None else None
    C = np.empty((V * n_blk_rows, dim), dtype=np.float32)
    _lib().orc_spmm_bcsr(_pi(rpb), _pi(tr), _i64(rpb.shape[0] - 1), _pi(cb), _pf(vb), _i32(V),
                         _pf(B), _pf(C), _i64(V * n_blk_rows), _i32(dim), _i64(dim), _i64(dim))
    return C


def sddmm_csr(rowPtr, colIdx, A, B, target_row=None):
    """out[k] = <A[row(k)], B[col[k]]> (SDDMM/sddmm_kernel.cu:917-1057)."""
    rowPtr, colIdx, A, B = _ci(rowPtr), _ci(colIdx), _cf(A), _cf(B)
    tr = _ci(target_row) if target_row is not None else None
    out = np.zeros(colIdx.shape[0], dtype=np.float32)
    _lib().orc_sddmm_csr(_pi(rowPtr), _pi(tr), _i64(rowPtr.shape[0] - 1), _pi(colIdx), _pf(A),
                         _pf(B), _pf(out), _i32(A.shape[1]), _i64(A.shape[1]), _i64(B.shape[1]))
    return out


def sddmm_bcsr(rowPtr_b, colIdx_b, val_b, A, B, target_row=None):
    """Masked SDDMM on V x 1 blocks (SDDMM/sddmm_kernel.cu:1059-1468)."""
    rpb, cb, vb, A, B = _ci(rowPtr_b), _ci(colIdx_b), _cf(val_b), _cf(A), _cf(B)
    tr = _ci(target_row) if target_row is not None else None
    V = vb.shape[1]
    out = np.zeros((cb.shape[0], V), dtype=np.float32)
    _lib().orc_sddmm_bcsr(_pi(rpb), _pi(tr), _i64(rpb.shape[0] - 1), _pi(cb), _pf(vb), _i32(V),
                          _pf(A), _pf(B), _pf(out), _i32(A.shape[1]), _i64(A.shape[1]),
                          _i64(B.shape[1]))
    return out


def agnn_aggregate(rowPtr, colIdx, A, B, beta=1.0, softmax=True, V=None):
    """out_i = sum_j a_ij B_j over the stored pattern, a_ij = softmax_j(beta <A_i, B_j>) or, with
    softmax=False, the raw scaled scores: the composition SDDMM -> ``* attention_w`` -> SpMM of the
    reference's AGNN layer (gnn_conv.py:130-151), with the per-row edge softmax in between when
    asked for.  With ``V`` the aggregated rows are V_j instead of B_j (the layer's backward product
    AGNN_spmm(edge_attentions, d_output), gnn_conv.py:157, for V = d_output); a single row
    ``[1, dim]`` is shared by all columns.  Computed row by row in float64 (numpy), returned as float32."""
    rowPtr, colIdx = np.asarray(rowPtr, dtype=np.int64), np.asarray(colIdx, dtype=np.int64)
    A64, B64 = np.asarray(A, dtype=np.float64), np.asarray(B, dtype=np.float64)
    V64 = B64 if V is None else np.asarray(V, dtype=np.float64)
    if V64.shape[0] == 1 and B64.shape[0] != 1:
        V64 = np.broadcast_to(V64, B64.shape)
    n = rowPtr.shape[0] - 1
    out = np.zeros((n, B64.shape[1]), dtype=np.float64)
    for i in range(n):
        lo, hi = rowPtr[i], rowPtr[i + 1]
        if hi == lo:
            continue
        nb = B64[colIdx[lo:hi]]
        s = beta * (nb @ A64[i])
        if softmax:
            w = np.exp(s - s.max())
            w /= w.sum()
        else:
            w = s
        out[i] = w @ V64[colIdx[lo:hi]]
    return out.astype(np.float32)


def spmm_torch_cpu(rowPtr, colIdx, val, B, n_cols=None):
    """The reference's own acceptance oracle: torch.sparse.mm on a CSR tensor, CPU
    (verification.py:18-23, 44-46)."""
    import torch

    n = len(rowPtr) - 1
    s = torch.sparse_csr_tensor(torch.as_tensor(np.asarray(rowPtr), dtype=torch.int32),
                                torch.as_tensor(np.asarray(colIdx), dtype=torch.int32),
                                torch.as_tensor(np.asarray(val), dtype=torch.float32),
                                size=(n, n if n_cols is None else n_cols))
    return torch.sparse.mm(s, torch.as_tensor(np.asarray(B), dtype=torch.float32)).numpy()


def verification_compare(ref, out, rel=1e-4):
    """The reference's acceptance rule (verification.py:79-83): fails where |ref-out| > rel*|ref|."""
    ref, out = np.asarray(ref), np.asarray(out)
    return not bool(np.any(np.abs(ref - out) > rel * np.abs(ref)))


# --------------------------------------------------------------------------- matrix statistics
def split_granularity_auto(real_avg_degree):
    """graph_input.py:101: ceil(real_avg_degree / 32) * 32."""
    return int(math.ceil(real_avg_degree / 32) * 32)


def csr_info(rowPtr, colIdx, num_edges=None, manual_granularity=None, is_avg_granularity=False):
    """Per-matrix statistics of csr_data.init_info (graph_input.py:53-102) for a CSR matrix.

    Follows the reference's arithmetic: torch's unbiased std on fp32 row lengths, the
    ``nonempty_rate < 0.98`` switch for the "real" averages, bandwidth = last minus first
    stored column of every non-empty row.
    """
    rowPtr = np.asarray(rowPtr, dtype=np.int64)
    colIdx = np.asarray(colIdx, dtype=np.int64)
    n = rowPtr.shape[0] - 1
    nnz = int(rowPtr[-1]) if num_edges is None else num_edges
    ln = rowPtr[1:] - rowPtr[:-1]
    nonempty = ln != 0
    real_nrow = int(nonempty.sum())
    nonempty_rate = np.float32(real_nrow) / np.float32(n)
    avg_degree = nnz / n
    lnf = ln.astype(np.float32)
    cov = float(np.float32(np.std(lnf.astype(np.float64), ddof=1)) / np.float32(avg_degree))
    if nonempty_rate < 0.98:
        real_avg = float(np.float32(nnz) / np.float32(real_nrow))
        real_cov = float(np.float32(np.std(lnf[nonempty].astype(np.float64), ddof=1)) / np.float32(real_avg))
    else:
        real_avg, real_cov = avg_degree, cov
    head = rowPtr[:-1][nonempty]
    tail = (rowPtr[1:] - 1)[nonempty]
    bw = colIdx[tail] - colIdx[head]
    if is_avg_granularity:
        gran = int(real_avg)
    elif manual_granularity is not None:
        gran = int(manual_granularity)
    else:
        gran = split_granularity_auto(real_avg)
    pieces = row_split_counts(rowPtr, gran)
    return {
        "max_row_nnz": int(ln.max()) if n else 0,
        "real_nrow": real_nrow,
        "nonempty_rate": float(nonempty_rate),
        "avg_degree": avg_degree,
        "COV": cov,
        "real_avg_degree": real_avg,
        "real_COV": real_cov,
        "max_bw": int(bw.max()) if bw.size else 0,
        "avg_bw": float(np.float32(bw.sum()) / np.float32(real_nrow)) if real_nrow else 0.0,
        "split_granularity": gran,
        "split_ratio": int(pieces.sum()) / real_nrow if real_nrow else 0.0,
        "split_rows": int(pieces.sum()),
    }


def bcsr_split_info(rowPtr_b, nnzblk, manual_granularity=None, is_avg_granularity=False):
    """csr_data.get_split_info for the block layout (graph_input.py:107-131)."""
    rowPtr_b = np.asarray(rowPtr_b, dtype=np.int64)
    ln = rowPtr_b[1:] - rowPtr_b[:-1]
    real_nrow = int((ln != 0).sum())
    real_avg = float(np.float32(nnzblk) / np.float32(real_nrow))
    if is_avg_granularity:
        gran = int(real_avg)
    elif manual_granularity is not None:
        gran = int(manual_granularity)
    else:
        gran = split_granularity_auto(real_avg)
    pieces = row_split_counts(rowPtr_b, gran)
    return {"real_nrow": real_nrow, "real_avg_degree": real_avg, "split_granularity": gran,
            "split_ratio": int(pieces.sum()) / real_nrow, "split_rows": int(pieces.sum())}


# --------------------------------------------------------------------------- decider decode rules
def gap_calculator(dim, CF, warp_size=32):
    """PCSR.py:19-26: idle lanes in the last column tile for a given coarsening factor."""
    t_norm = min(dim, CF * warp_size)
    t_res = dim % (warp_size * CF)
    return 0 if t_res == 0 else t_norm - t_res


def dynamic_CF_prompter(dim, CF_set=None, warp_size=32):
    """PCSR.py:30-42: coarsening factors whose residue gap is below one warp."""
    if CF_set is None:
        CF_set = [1, 2, 3, 4, 5, 6, 7, 8]
    CF_set = CF_set[: math.ceil(dim / 32)]
    return [cf for cf in CF_set if gap_calculator(dim, cf, warp_size) < 32]


def decode_tree(code, dim, vec_size_list=(1, 2), warpNum_list=(4, 8)):
    """decider.py:63-80: class code -> (if_split, vec_size, CF, blkWarpNum)."""
    if_split = code % 2
    cf_list = dynamic_CF_prompter(dim)
    nv = len(vec_size_list)
    vec_size = vec_size_list[code // 2 % nv]
    ncf = len(cf_list)
    CF = cf_list[code // (nv * 2) % ncf]
    W = warpNum_list[code // (ncf * nv * 2)]
    return if_split, vec_size, CF, W


def model_dim_for(dim):
    """decider.py:52-55: which per-dim model serves an arbitrary dim."""
    return dim if dim % 32 == 0 else (math.ceil(dim / 32) * 2 - 1) * 16
