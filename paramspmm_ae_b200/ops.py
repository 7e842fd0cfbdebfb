"""Torch-tensor level operators over libpspmm's C ABI.

These functions keep the positional signatures, return types and error behaviour of the
reference's three pybind extension modules (``ParamSpMM``: SpMM/SpMM.cpp:891-926,
``ParamSDDMM``: SDDMM/sddmm.cpp:675-701, ``ParamSpCONV``: SpCONV/SpCONV.cpp:496-512); the
modules under ``paramspmm_ae_b200/dropin`` re-export them under the reference's names.

torch is plumbing here: it owns device memory and the current stream.  All arithmetic on
the sparse path runs in libpspmm's CUDA kernels; a missing library or a non-CUDA tensor is
an error, never a reason to fall back to a torch implementation.
"""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib
from ._lib import PspmmError, check, lib, make_cfg

PROFILE_ITERS = 200   # SpMM/SpMM.h:12 (PROFILE)
PROFILE_WARMUP = 20


# ----------------------------------------------------------------------------- argument checks
def _check_cuda(t, name, dtype=None, ndim=None):
    if not isinstance(t, torch.Tensor):
        raise RuntimeError("%s must be a tensor" % name)
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor" % name)
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous" % name)
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError("%s must have dtype %s, got %s" % (name, dtype, t.dtype))
    if ndim is not None and t.dim() != ndim:
        raise RuntimeError("%s must be %d-dimensional" % (name, ndim))


def _check_cpu(t, name, dtype=torch.int32):
    if not isinstance(t, torch.Tensor) or t.is_cuda:
        raise RuntimeError("%s must be a CPU tensor" % name)
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous" % name)
    if t.dtype != dtype:
        raise RuntimeError("%s must have dtype %s, got %s" % (name, dtype, t.dtype))


def _check_legacy(CF, blkWarpNum, max_cf=8):
    # Same domain the reference enforces with TORCH_CHECK (SpMM/SpMM.cpp:110,139).
    if blkWarpNum not in (4, 8):
        raise RuntimeError("blkWarpNum must be 4 or 8")
    if not (isinstance(CF, int) and 1 <= CF <= max_cf):
        raise RuntimeError("CF must be an integer in 1..%d" % max_cf)


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr() if t is not None else 0)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# Kernel parameters chosen per call.  `tuner` (set by paramspmm_ae_b200.decider) maps
# (op, dim, mean entries per segment, V, split) to the non-legacy fields of pspmm_cfg.
tuner = None


def _cfg(op, CF, W, dim, n_entries, n_seg, V, split):
    kw = {}
    if tuner is not None:
        kw = tuner(op, dim, (n_entries / n_seg) if n_seg else 0.0, V, split) or {}
    return make_cfg(CF=CF, blkWarpNum=W, **kw)


# ----------------------------------------------------------------------------- host builders
def split_csr(rowPtr, granularity):
    """PCSR partition of a CPU int32 rowPtr -> [rowPtr_split, target_row] (SpMM/SpMM.cpp:15-40)."""
    _check_cpu(rowPtr, "rowPtr")
    n = rowPtr.shape[0] - 1
    nseg = ctypes.c_int64(0)
    check(lib().pspmm_split_count(_ptr(rowPtr), n, int(granularity), ctypes.byref(nseg)))
    rps = torch.empty(nseg.value + 1, dtype=torch.int32)
    tr = torch.empty(nseg.value, dtype=torch.int32)
    check(lib().pspmm_split_csr(_ptr(rowPtr), n, int(granularity), _ptr(rps), _ptr(tr), nseg.value))
    return [rps, tr]


def mtx_info(path):
    """Banner and size line of a MatrixMarket file -> dict (n_rows, n_cols, stored, nnz_max,
    symmetric, field)."""
    from ._lib import MtxInfo
    info = MtxInfo()
    check(lib().pspmm_mtx_info_read(os.fsencode(path), ctypes.byref(info)))
    return {k: int(getattr(info, k)) for k, _ in MtxInfo._fields_}


def mtx_read_csr(path, force_ones=True):
    """MatrixMarket coordinate file -> (rowPtr, colIdx, val, n_rows, n_cols) as CPU tensors in
    canonical CSR: what ``scipy.io.mmread(path).tocsr()`` gives in the reference's loader
    (graph_input.py:226-232), with every stored value replaced by 1 first when ``force_ones``
    (graph_input.py:227).  Parsed by the library's parallel reader."""
    info = mtx_info(path)
    rowPtr = torch.empty(info["n_rows"] + 1, dtype=torch.int32)
    colIdx = torch.empty(info["nnz_max"], dtype=torch.int32)
    val = torch.empty(info["nnz_max"], dtype=torch.float32)
    nnz = ctypes.c_int64(0)
    check(lib().pspmm_mtx_read_csr(os.fsencode(path), 1 if force_ones else 0, _ptr(rowPtr), _ptr(colIdx),
                                   _ptr(val), info["nnz_max"], ctypes.byref(nnz)))
    k = nnz.value
    if k != info["nnz_max"]:  # duplicates or a diagonal in a symmetric file: give the surplus back
        colIdx, val = colIdx[:k].clone(), val[:k].clone()
    return rowPtr, colIdx, val, info["n_rows"], info["n_cols"]


def csr_file_write(path, rowPtr, colIdx, val, n_cols, source=None):
    """Write CSR arrays (CPU tensors) as a binary container; ``source`` = the text file they were
    parsed from, whose size and modification time are recorded for staleness checks."""
    _check_cpu(rowPtr, "rowPtr")
    _check_cpu(colIdx, "colIdx")
    if val.dtype != torch.float32 or val.is_cuda or not val.is_contiguous() or val.shape != colIdx.shape:
        raise RuntimeError("values must be a contiguous CPU float32 tensor with one entry per column index")
    size = mtime = 0
    if source is not None:
        st = os.stat(source)
        size, mtime = st.st_size, st.st_mtime_ns
    check(lib().pspmm_csr_file_write(os.fsencode(path), rowPtr.shape[0] - 1, int(n_cols), colIdx.shape[0],
                                     _ptr(rowPtr), _ptr(colIdx), _ptr(val), size, mtime))


def csr_file_info(path):
    from ._lib import CsrFileInfo
    info = CsrFileInfo()
    check(lib().pspmm_csr_file_info(os.fsencode(path), ctypes.byref(info)))
    return {k: int(getattr(info, k)) for k, _ in CsrFileInfo._fields_}


def csr_file_read(path, verify=True, info=None):
    """Binary container -> (rowPtr, colIdx, val, n_rows, n_cols) as CPU tensors."""
    info = info or csr_file_info(path)
    rowPtr = torch.empty(info["n_rows"] + 1, dtype=torch.int32)
    colIdx = torch.empty(info["nnz"], dtype=torch.int32)
    val = torch.empty(info["nnz"], dtype=torch.float32)
    check(lib().pspmm_csr_file_read(os.fsencode(path), _ptr(rowPtr), _ptr(colIdx), _ptr(val), info["n_rows"],
                                    info["nnz"], 1 if verify else 0))
    return rowPtr, colIdx, val, info["n_rows"], info["n_cols"]


def load_matrix(mtx_path, cache_dir=None, force_ones=True, verify=True):
    """CSR arrays of a MatrixMarket file, through a binary container in ``cache_dir`` when one is
    given: a container whose recorded size and modification time match the text file is read
    instead of parsing; otherwise the file is parsed and the container (re)written.  A cache
    directory that cannot be written to is not an error, the arrays are still returned."""
    if cache_dir is None:
        return mtx_read_csr(mtx_path, force_ones)
    st = os.stat(mtx_path)
    tag = "ones" if force_ones else "vals"
    cached = os.path.join(cache_dir, "%s.%s.pspmmcsr" % (os.path.basename(mtx_path), tag))
    if os.path.exists(cached):
        try:
            info = csr_file_info(cached)
            if info["source_size"] == st.st_size and info["source_mtime_ns"] == st.st_mtime_ns:
                return csr_file_read(cached, verify, info)
        except PspmmError:
            pass  # unreadable or damaged container: parse again and replace it
    out = mtx_read_csr(mtx_path, force_ones)
    try:
        os.makedirs(cache_dir, exist_ok=True)
        csr_file_write(cached, out[0], out[1], out[2], out[4], source=mtx_path)
    except (OSError, PspmmError):
        pass
    return out


def split_csr_par(rowPtr, row_split_offset, granularity):
    """Same result as :func:`split_csr` (SpMM/SpMM.cpp:42-75).

    The reference takes per-row piece offsets computed by the caller through an fp32
    cumulative sum; they are validated for type only and recomputed here with 64-bit integer
    arithmetic, which agrees with them wherever the fp32 sum was exact.
    """
    _check_cpu(row_split_offset, "row_split_offset")
    if row_split_offset.shape[0] != rowPtr.shape[0]:
        raise RuntimeError("row_split_offset must have as many entries as rowPtr")
    return split_csr(rowPtr, granularity)


def split_csr_device(rowPtr, granularity):
    """PCSR partition of a CUDA int32 rowPtr, built on the device -> [rowPtr_split, target_row]
    (CUDA tensors; bit-exact with :func:`split_csr`).  Reads the piece count back, so it
    synchronises the current stream once."""
    _check_cuda(rowPtr, "rowPtr", torch.int32, 1)
    n = rowPtr.shape[0] - 1
    need = ctypes.c_size_t(0)
    check(lib().pspmm_split_device_scratch_bytes(n, ctypes.byref(need)))
    scratch = torch.empty((need.value + 7) // 8, dtype=torch.int64, device=rowPtr.device)
    nseg = ctypes.c_int64(0)
    check(lib().pspmm_split_count_device(_ptr(rowPtr), n, int(granularity), _ptr(scratch), need.value,
                                         ctypes.byref(nseg), _stream()))
    rps = torch.empty(nseg.value + 1, dtype=torch.int32, device=rowPtr.device)
    tr = torch.empty(nseg.value, dtype=torch.int32, device=rowPtr.device)
    check(lib().pspmm_split_csr_device(_ptr(rowPtr), n, int(granularity), _ptr(rps), _ptr(tr), nseg.value,
                                       _ptr(scratch), need.value, _stream()))
    return [rps, tr]


SEG_MULTI, SEG_FIRST, SEG_ROW_MASK = 0x80000000, 0x40000000, 0x3FFFFFFF


def bucket_pcsr(rowPtr, colIdx, val, granularity):
    """Length-bucketed plan of a (block-)CSR matrix for ``pspmm_cfg.bucketed``: the rows are cut into
    pieces of at most ``granularity`` entries exactly as :func:`split_csr` cuts them, the pieces are
    then ordered by length, longest first (a stable sort: pieces of one row stay together and in
    order), rows without entries follow as empty pieces, and the entries are permuted to match.
    Returns ``(segPtr, colIdx_p, val_p, target)``; ``target`` carries the row in its low 30 bits,
    bit 31 on every piece of a row that has several, bit 30 on the first of those.

    This is an internal layout of the sm_100a kernels (the lane groups of a warp then walk equally
    long pieces and no batch of gathers is cut short by a neighbouring row's end); the arrays the
    reference defines, ``split_csr``'s, are untouched by it.  Built with torch ops on the device the
    inputs live on; it is set-up work, done once per matrix and partition length."""
    rp = rowPtr.long()
    n = rp.numel() - 1
    if n >= SEG_FIRST:
        raise RuntimeError("the bucketed plan holds row ids in 30 bits")
    dev = rp.device
    ln = rp[1:] - rp[:-1]
    g = int(granularity)
    pieces = torch.div(ln + g - 1, g, rounding_mode="floor")          # per row; 0 for empty rows
    S = int(pieces.sum())
    tr = torch.repeat_interleave(torch.arange(n, device=dev), pieces)   # row of every piece (non-decreasing)
    first_piece = torch.cumsum(pieces, 0) - pieces                      # index of each row's first piece
    k = torch.arange(S, device=dev) - first_piece[tr]                   # position of the piece inside its row
    start = rp[:-1][tr] + k * g
    plen = torch.minimum(rp[1:][tr], start + g) - start
    multi = pieces[tr] > 1
    order = torch.argsort(plen, descending=True, stable=True)
    empty = torch.nonzero(pieces == 0).flatten()
    flags = multi.long() * SEG_MULTI + (multi & (k == 0)).long() * SEG_FIRST
    target = torch.cat([(tr | flags)[order], empty])
    plen_b = torch.cat([plen[order], torch.zeros_like(empty)])
    seg = torch.zeros(target.numel() + 1, dtype=torch.long, device=dev)
    seg[1:] = torch.cumsum(plen_b, 0)
    # entries: piece `order[i]` moves to segment i
    new_start = torch.empty(S, dtype=torch.long, device=dev)
    new_start[order] = seg[:S]
    piece_of_entry = torch.repeat_interleave(torch.arange(S, device=dev), plen)
    # entries are stored piece after piece in the original arrays, so entry e belongs to piece_of_entry[e]
    pos = new_start[piece_of_entry] + (torch.arange(piece_of_entry.numel(), device=dev) + int(rp[0]) - start[piece_of_entry])
    lo = int(rp[0])
    src_c, src_v = colIdx[lo: lo + pos.numel()], val[lo: lo + pos.numel()]
    ci_p = torch.empty_like(src_c)
    v_p = torch.empty_like(src_v)
    ci_p[pos] = src_c
    v_p[pos] = src_v
    # values above 2^31 wrap into the sign bit of int32, which is where the kernels look for them
    target32 = torch.where(target >= 2**31, target - 2**32, target).to(torch.int32)
    return seg.to(torch.int32), ci_p, v_p, target32


def bcsr_from_csr(rowPtr, colIdx, val, n_cols, V=2):
    """CSR (CPU tensors) -> V x 1 block CSR laid out as scipy's tobsr((V,1)) does
    (what graph_input.py:245-266 of the reference builds)."""
    _check_cpu(rowPtr, "rowPtr")
    _check_cpu(colIdx, "colIdx")
    _check_cpu(val, "val", torch.float32)
    n = rowPtr.shape[0] - 1
    nbr = (n + V - 1) // V
    rpb = torch.empty(nbr + 1, dtype=torch.int32)
    nblk = ctypes.c_int64(0)
    check(lib().pspmm_bcsr_count(_ptr(rowPtr), _ptr(colIdx), n, int(n_cols), V, _ptr(rpb),
                                 ctypes.byref(nblk)))
    cb = torch.empty(nblk.value, dtype=torch.int32)
    vb = torch.empty((nblk.value, V), dtype=torch.float32)
    check(lib().pspmm_bcsr_fill(_ptr(rowPtr), _ptr(colIdx), _ptr(val), n, int(n_cols), V, _ptr(rpb),
                                _ptr(cb), _ptr(vb)))
    return rpb, cb, vb


# ----------------------------------------------------------------------------- SpMM
def _spmm_inputs(X, rowPtr, colIdx, val, target_row, V):
    _check_cuda(X, "input", torch.float32, 2)
    _check_cuda(rowPtr, "rowPtr", torch.int32, 1)
    _check_cuda(colIdx, "colIdx", torch.int32, 1)
    if val is None and V != 1:
        raise RuntimeError("block layouts need their value array (it also is their mask)")
    if val is not None:
        _check_cuda(val, "values", torch.float32, 1 if V == 1 else 2)
        if V > 1 and val.shape[1] != V:
            raise RuntimeError("values must have %d columns" % V)
    if target_row is not None:
        _check_cuda(target_row, "target_row", torch.int32, 1)
        if target_row.shape[0] != rowPtr.shape[0] - 1:
            raise RuntimeError("target_row must have one entry per split row")


def _check_output(out, rowPtr, split, n_out_rows, V, dim):
    # The kernels index rowPtr and the output by n_out_rows without looking at their sizes.
    # (the output may be a column slice of a wider array: only its row stride is passed on)
    if not out.is_cuda or out.dtype != torch.float32 or out.dim() != 2 or out.stride(1) != 1:
        raise RuntimeError("output must be a 2-D float32 CUDA tensor with unit column stride")
    if out.shape[1] != dim or out.shape[0] < n_out_rows * V:
        raise RuntimeError("output must hold %d rows of %d columns" % (n_out_rows * V, dim))
    if not split and rowPtr.shape[0] - 1 != n_out_rows:
        raise RuntimeError("rowPtr must have one entry per output row plus one")


def spmm_into(out, X, rowPtr, colIdx, val, target_row=None, V=1, n_out_rows=None, CF=0, W=0,
              cfg=None):
    """Launch the SpMM into a caller-provided output (also used by the multi-GPU row shards).

    ``n_out_rows`` counts (block-)rows of the output; it defaults to the number of segments
    when there is no split and must be given for split layouts.  ``val=None`` (CSR layouts)
    multiplies by the pattern itself: every stored entry counts as 1.
    """
    dim = X.shape[1]
    n_seg = rowPtr.shape[0] - 1
    split = target_row is not None
    if n_out_rows is None:
        if split:
            raise RuntimeError("n_out_rows is required for split layouts")
        n_out_rows = n_seg
    _check_output(out, rowPtr, split, n_out_rows, V, dim)
    nent = colIdx.shape[0]
    if cfg is None:
        cfg = _cfg("spmm", CF, W, dim, nent, n_seg, V, split)
    seg_ptr = _ptr(rowPtr)
    null = ctypes.c_void_p(0)
    if V == 1:
        check(lib().pspmm_spmm_csr(null if split else seg_ptr, _ptr(colIdx), _ptr(val), _ptr(X),
                                   _ptr(out), n_out_rows, X.shape[0], nent, dim, X.stride(0),
                                   out.stride(0), ctypes.byref(cfg), seg_ptr if split else null,
                                   _ptr(target_row) if split else null, n_seg if split else 0,
                                   _stream()))
    else:
        check(lib().pspmm_spmm_bcsr(null if split else seg_ptr, _ptr(colIdx), _ptr(val), V, _ptr(X),
                                    _ptr(out), n_out_rows, X.shape[0], nent, dim, X.stride(0),
                                    out.stride(0), ctypes.byref(cfg), seg_ptr if split else null,
                                    _ptr(target_row) if split else null, n_seg if split else 0,
                                    _stream()))
    return out


def _spmm(X, rowPtr, colIdx, val, target_row, V, CF, W):
    _check_legacy(CF, W)
    _spmm_inputs(X, rowPtr, colIdx, val, target_row, V)
    n, dim = X.shape
    # The reference sizes the output from the dense input, zeros_like(input) for CSR
    # (SpMM/SpMM_kernel.cu:136) and the input's row count rounded up to a multiple of V for the
    # block layouts (:281-282, 427-428), and walks as many (block-)rows as the row pointer has.
    # Its own callers hand in inputs with more rows than the matrix (GNN.py:226-240 pads the
    # features to an even row count): those extra output rows stay zero.
    padded = (n + V - 1) // V * V
    n_out = padded // V
    out = torch.empty((padded, dim), dtype=torch.float32, device=X.device)
    if target_row is None:
        n_seg = rowPtr.shape[0] - 1
        if n_seg > n_out:
            raise RuntimeError("rowPtr describes %d (block-)rows, the input only allows %d" % (n_seg, n_out))
        if n_seg < n_out:
            out[n_seg * V:].zero_()
            n_out = n_seg
    return spmm_into(out, X, rowPtr, colIdx, val, target_row, V, n_out, CF, W)


def csr_spmm(X, rowPtr, colIdx, val, CF, blkWarpNum):
    return _spmm(X, rowPtr, colIdx, val, None, 1, CF, blkWarpNum)


def csr_split_spmm(X, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum):
    return _spmm(X, rowPtr_split, colIdx, val, target_row, 1, CF, blkWarpNum)


def bcsr_spmm(X, rowPtr_bcsr, colIdx, val, CF, blkWarpNum):
    return _spmm(X, rowPtr_bcsr, colIdx, val, None, 2, CF, blkWarpNum)


def bcsr_split_spmm(X, rowPtr_bcsr_split, colIdx, val, target_row, CF, blkWarpNum):
    return _spmm(X, rowPtr_bcsr_split, colIdx, val, target_row, 2, CF, blkWarpNum)


def _vec_size(val):
    if val.dim() != 2 or val.shape[1] != 3:
        raise RuntimeError("vec_size must be 3")  # SpMM/SpMM.cpp:352,406
    return 3


def vec_spmm(X, rowPtr_bcsr, colIdx, val, CF, blkWarpNum):
    return _spmm(X, rowPtr_bcsr, colIdx, val, None, _vec_size(val), CF, blkWarpNum)


def vec_split_spmm(X, rowPtr_bcsr_split, colIdx, val, target_row, CF, blkWarpNum):
    return _spmm(X, rowPtr_bcsr_split, colIdx, val, target_row, _vec_size(val), CF, blkWarpNum)


def spmm_time_ms(X, rowPtr, colIdx, val, target_row=None, V=1, CF=0, W=0, cfg=None,
                 warmup=PROFILE_WARMUP, iters=PROFILE_ITERS, out=None, n_out_rows=None):
    """Mean milliseconds per launch over `iters` back-to-back launches (CUDA events).

    ``n_out_rows`` counts (block-)rows of the output; it defaults to the square case
    ceil(input rows / V) that the reference's profile functions assume.
    """
    _spmm_inputs(X, rowPtr, colIdx, val, target_row, V)
    n, dim = X.shape
    n_seg = rowPtr.shape[0] - 1
    split = target_row is not None
    n_out = (n + V - 1) // V if n_out_rows is None else n_out_rows
    if out is None:
        out = torch.empty((n_out * V, dim), dtype=torch.float32, device=X.device)
    _check_output(out, rowPtr, split, n_out, V, dim)
    nent = colIdx.shape[0]
    if cfg is None:
        cfg = _cfg("spmm", CF, W, dim, nent, n_seg, V, split)
    ms = ctypes.c_float(0.0)
    null = ctypes.c_void_p(0)
    check(lib().pspmm_profile_spmm(null if split else _ptr(rowPtr), _ptr(colIdx), _ptr(val), V,
                                   _ptr(X), _ptr(out), n_out, n, nent, dim, X.stride(0),
                                   out.stride(0), ctypes.byref(cfg),
                                   _ptr(rowPtr) if split else null,
                                   _ptr(target_row) if split else null, n_seg if split else 0,
                                   warmup, iters, ctypes.byref(ms), _stream()))
    return ms.value


def _gflops(nnz, dim, ms):
    # int(2*nnz*dim / 1e6 / ms), the figure the reference's *_profile functions return
    # (SpMM/SpMM_kernel.cu:645-656).
    return int(nnz / 1e6 * dim * 2 / ms)


def csr_spmm_profile(X, rowPtr, colIdx, val, CF, blkWarpNum):
    _check_legacy(CF, blkWarpNum)
    return _gflops(colIdx.shape[0], X.shape[1], spmm_time_ms(X, rowPtr, colIdx, val, None, 1, CF, blkWarpNum))


def csr_split_spmm_profile(X, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum):
    _check_legacy(CF, blkWarpNum)
    return _gflops(colIdx.shape[0], X.shape[1],
                   spmm_time_ms(X, rowPtr_split, colIdx, val, target_row, 1, CF, blkWarpNum))


def bcsr_spmm_profile(X, rowPtr, colIdx, val, nnz, CF, blkWarpNum):
    _check_legacy(CF, blkWarpNum)
    return _gflops(nnz, X.shape[1], spmm_time_ms(X, rowPtr, colIdx, val, None, 2, CF, blkWarpNum))


def bcsr_split_spmm_profile(X, rowPtr, colIdx, val, target_row, nnz, CF, blkWarpNum):
    _check_legacy(CF, blkWarpNum)
    return _gflops(nnz, X.shape[1], spmm_time_ms(X, rowPtr, colIdx, val, target_row, 2, CF, blkWarpNum))


def vec_spmm_profile(X, rowPtr, colIdx, val, nnz, CF, blkWarpNum):
    _check_legacy(CF, blkWarpNum)
    return _gflops(nnz, X.shape[1],
                   spmm_time_ms(X, rowPtr, colIdx, val, None, _vec_size(val), CF, blkWarpNum))


def vec_split_spmm_profile(X, rowPtr, colIdx, val, target_row, nnz, CF, blkWarpNum):
    _check_legacy(CF, blkWarpNum)
    return _gflops(nnz, X.shape[1],
                   spmm_time_ms(X, rowPtr, colIdx, val, target_row, _vec_size(val), CF, blkWarpNum))


# ----------------------------------------------------------------------------- SDDMM
def _sddmm(A, B, rowPtr, colIdx, val, target_row, V, CF, W, time_only=False):
    _check_legacy(CF, W, max_cf=4)  # SDDMM/sddmm.cpp:31-43
    _check_cuda(A, "A", torch.float32, 2)
    _check_cuda(B, "B", torch.float32, 2)
    _check_cuda(rowPtr, "rowPtr", torch.int32, 1)
    _check_cuda(colIdx, "colIdx", torch.int32, 1)
    _check_cuda(val, "values", torch.float32, 1 if V == 1 else 2)
    if A.shape[1] != B.shape[1]:
        raise RuntimeError("A and B must have the same number of columns")
    split = target_row is not None
    if split:
        _check_cuda(target_row, "target_row", torch.int32, 1)
    dim = A.shape[1]
    n_seg = rowPtr.shape[0] - 1
    nent = colIdx.shape[0]
    out = torch.empty_like(val)
    cfg = _cfg("sddmm", CF, W, dim, nent, n_seg, V, split)
    null = ctypes.c_void_p(0)
    # (block-)rows of the pattern; A may stop inside the last block-row when the node count is
    # not a multiple of V, and the kernel then reads nothing past A's last row
    n_rows = n_seg if not split else (A.shape[0] + V - 1) // V
    if A.shape[0] <= (n_rows - 1) * V:
        raise RuntimeError("A has %d rows, the pattern needs more than %d" % (A.shape[0], (n_rows - 1) * V))
    args_tail = (ctypes.byref(cfg), _ptr(rowPtr) if split else null,
                 _ptr(target_row) if split else null, n_seg if split else 0)
    if time_only:
        ms = ctypes.c_float(0.0)
        check(lib().pspmm_profile_sddmm(null if split else _ptr(rowPtr), _ptr(colIdx), _ptr(val), V,
                                        _ptr(A), _ptr(B), _ptr(out), n_rows, A.shape[0], nent, dim, A.stride(0),
                                        B.stride(0), *args_tail, PROFILE_WARMUP, PROFILE_ITERS,
                                        ctypes.byref(ms), _stream()))
        return ms.value
    if V == 1:
        check(lib().pspmm_sddmm_csr(null if split else _ptr(rowPtr), _ptr(colIdx), _ptr(A), _ptr(B),
                                    _ptr(out), n_rows, nent, dim, A.stride(0), B.stride(0),
                                    *args_tail, _stream()))
    else:
        check(lib().pspmm_sddmm_bcsr(null if split else _ptr(rowPtr), _ptr(colIdx), _ptr(val), V,
                                     _ptr(A), _ptr(B), _ptr(out), n_rows, A.shape[0], nent, dim, A.stride(0),
                                     B.stride(0), *args_tail, _stream()))
    return out


def csr_sddmm(A, B, rowPtr, colIdx, val, CF, blkWarpNum):
    return _sddmm(A, B, rowPtr, colIdx, val, None, 1, CF, blkWarpNum)


def csr_split_sddmm(A, B, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum):
    return _sddmm(A, B, rowPtr_split, colIdx, val, target_row, 1, CF, blkWarpNum)


def bcsr_sddmm(A, B, rowPtr, colIdx, val, CF, blkWarpNum):
    return _sddmm(A, B, rowPtr, colIdx, val, None, 2, CF, blkWarpNum)


def bcsr_split_sddmm(A, B, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum):
    return _sddmm(A, B, rowPtr_split, colIdx, val, target_row, 2, CF, blkWarpNum)


def vec_sddmm(A, B, rowPtr, colIdx, val, CF, blkWarpNum):
    return _sddmm(A, B, rowPtr, colIdx, val, None, _vec_size(val), CF, blkWarpNum)


def vec_split_sddmm(A, B, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum):
    return _sddmm(A, B, rowPtr_split, colIdx, val, target_row, _vec_size(val), CF, blkWarpNum)


def csr_sddmm_profile(A, B, rowPtr, colIdx, val, CF, blkWarpNum):
    return _gflops(colIdx.shape[0], A.shape[1], _sddmm(A, B, rowPtr, colIdx, val, None, 1, CF, blkWarpNum, True))


def csr_split_sddmm_profile(A, B, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum):
    return _gflops(colIdx.shape[0], A.shape[1],
                   _sddmm(A, B, rowPtr_split, colIdx, val, target_row, 1, CF, blkWarpNum, True))


def bcsr_sddmm_profile(A, B, rowPtr, colIdx, val, nnz, CF, blkWarpNum):
    return _gflops(nnz, A.shape[1], _sddmm(A, B, rowPtr, colIdx, val, None, 2, CF, blkWarpNum, True))


def bcsr_split_sddmm_profile(A, B, rowPtr_split, colIdx, val, target_row, nnz, CF, blkWarpNum):
    return _gflops(nnz, A.shape[1],
                   _sddmm(A, B, rowPtr_split, colIdx, val, target_row, 2, CF, blkWarpNum, True))


def vec_sddmm_profile(A, B, rowPtr, colIdx, val, nnz, CF, blkWarpNum):
    return _gflops(nnz, A.shape[1],
                   _sddmm(A, B, rowPtr, colIdx, val, None, _vec_size(val), CF, blkWarpNum, True))


def vec_split_sddmm_profile(A, B, rowPtr_split, colIdx, val, target_row, nnz, CF, blkWarpNum):
    return _gflops(nnz, A.shape[1],
                   _sddmm(A, B, rowPtr_split, colIdx, val, target_row, _vec_size(val), CF, blkWarpNum, True))


def agnn_fused(A, B, rowPtr, colIdx, beta=1.0, softmax=True, target_row=None, n_out_rows=None, out=None,
               batch=0, lanes_per_row=0, vec_width=0, V=None):
    """out_i = sum_j a_ij B_j with a_ij = softmax_j(beta <A_i, B_j>) (or the raw scaled scores when
    ``softmax`` is false) over the stored pattern, in one pass and without a per-edge array.

    With ``softmax=False`` and ``A is B`` this equals the reference's AGNN forward composition
    csr_sddmm -> ``* attention_w`` -> csr_spmm (gnn_conv.py:130-151).  ``rowPtr`` is the CSR row
    pointer, or the split row pointer when ``target_row`` is given (then ``n_out_rows`` is
    required).  dim must be a multiple of 4, at most 256.

    ``V`` (same shape as ``B``, or a single row ``[1, dim]`` that every column shares) replaces ``B``
    in the aggregation: ``out_i = sum_j a_ij V_j``.  With ``A = B`` = the projected features and
    ``V`` = an upstream gradient this is the layer's backward product from recomputed scores.
    """
    _check_cuda(A, "A", torch.float32, 2)
    _check_cuda(B, "B", torch.float32, 2)
    _check_cuda(rowPtr, "rowPtr", torch.int32, 1)
    _check_cuda(colIdx, "colIdx", torch.int32, 1)
    if A.shape[1] != B.shape[1]:
        raise RuntimeError("A and B must have the same width")
    if A.stride(1) != 1 or B.stride(1) != 1:
        raise RuntimeError("dense operands must be row-major")
    dim = A.shape[1]
    ldV = None
    if V is not None:
        _check_cuda(V, "V", torch.float32, 2)
        if V.shape[1] != dim or V.shape[0] not in (1, B.shape[0]):
            raise RuntimeError("V must be [%d, %d] or a single shared row [1, %d]" % (B.shape[0], dim, dim))
        ldV = 0 if (V.shape[0] == 1 and B.shape[0] != 1) else V.stride(0)
    n_seg = rowPtr.shape[0] - 1
    split = target_row is not None
    if split:
        _check_cuda(target_row, "target_row", torch.int32, 1)
        if n_out_rows is None:
            raise RuntimeError("n_out_rows is required for split layouts")
    else:
        n_out_rows = n_seg
    if A.shape[0] < n_out_rows:
        raise RuntimeError("A has fewer rows than the pattern")
    if out is None:
        out = torch.empty(n_out_rows, dim, dtype=torch.float32, device=A.device)
    null = ctypes.c_void_p(0)
    scratch, sbytes = None, 0
    if split:
        need = ctypes.c_size_t(0)
        check(lib().pspmm_agnn_scratch_bytes(n_seg, dim, ctypes.byref(need)))
        sbytes = need.value
        scratch = torch.empty((sbytes + 15) // 16 * 4, dtype=torch.float32, device=A.device)
    seg_ptr = _ptr(rowPtr)
    tail = (float(beta), 1 if softmax else 0, int(vec_width), int(lanes_per_row), int(batch),
            seg_ptr if split else null, _ptr(target_row) if split else null, n_seg if split else 0,
            _ptr(scratch) if split else null, sbytes, _stream())
    if V is None:
        check(lib().pspmm_agnn_fused_csr(null if split else seg_ptr, _ptr(colIdx), _ptr(A), _ptr(B), _ptr(out),
                                         n_out_rows, colIdx.shape[0], dim, A.stride(0), B.stride(0), out.stride(0),
                                         *tail))
    else:
        check(lib().pspmm_agnn_fused_apply_csr(null if split else seg_ptr, _ptr(colIdx), _ptr(A), _ptr(B), _ptr(V),
                                               _ptr(out), n_out_rows, colIdx.shape[0], dim, A.stride(0), B.stride(0),
                                               ldV, out.stride(0), *tail))
    return out


def pull_rows(dst, sources, first, rows, rotate=0, ctas=0, bulk=False):
    """dst[j] = sources[s][rows[j]] for first[s] <= j < first[s+1]: gathers rows of a dense operand
    that lives in several blocks (this GPU's memory or peer-mapped memory of other GPUs) into one
    compact buffer with a copy kernel that reads the blocks directly (``pspmm_pull_rows``).
    ``sources``: 2-D float32 CUDA tensors with one row stride; ``first``: len(sources)+1
    non-decreasing list positions; ``rows``: int32 CUDA tensor of row ids inside the owning block.
    ``bulk=True`` moves the rows with bulk asynchronous copies through shared memory
    (``pspmm_pull_rows_bulk``: one warp per thread block), the form meant to run beside an SpMM."""
    if not sources or len(sources) > _lib.MAX_ROW_SOURCES or len(first) != len(sources) + 1:
        raise RuntimeError("between 1 and %d sources with len(sources)+1 list positions" % _lib.MAX_ROW_SOURCES)
    _check_cuda(rows, "rows", torch.int32, 1)
    if dst.dtype != torch.float32 or not dst.is_cuda or dst.dim() != 2 or dst.stride(1) != 1:
        raise RuntimeError("dst must be a 2-D float32 CUDA tensor with unit column stride")
    n, dim = dst.shape
    if rows.shape[0] != n or int(first[-1]) != n:
        raise RuntimeError("rows and first must describe exactly dst.shape[0] rows")
    src = _lib.RowSources()
    ld = None
    for s, t in enumerate(sources):
        if t.dtype != torch.float32 or not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.shape[1] != dim:
            raise RuntimeError("every source must be a float32 CUDA tensor [rows, %d] with unit column stride" % dim)
        if ld is None:
            ld = t.stride(0)
        elif t.stride(0) != ld:
            raise RuntimeError("all sources must share one row stride")
        src.base[s] = t.data_ptr()
    for s, f in enumerate(first):
        src.first[s] = int(f)
    src.n_src = len(sources)
    fn = lib().pspmm_pull_rows_bulk if bulk else lib().pspmm_pull_rows
    check(fn(ctypes.byref(src), _ptr(rows), n, _ptr(dst), dim, ld, dst.stride(0), int(rotate), int(ctas), _stream()))
    return dst


def pull_rows_status():
    """1 once a bounded wait inside the bulk fetch kernel has run out on this GPU, else 0
    (synchronises with the device)."""
    v = ctypes.c_int32(0)
    check(lib().pspmm_pull_rows_status(ctypes.byref(v)))
    return int(v.value)


def genmask(rowPtr_bcsr, rowPtr, blkval, nnz):
    """int32[nnz] map from CSR entry order to the flattened [nblk,2] block values
    (SDDMM/sddmm.cpp:663-673)."""
    _check_cuda(rowPtr_bcsr, "rowPtr_bcsr", torch.int32, 1)
    _check_cuda(rowPtr, "rowPtr", torch.int32, 1)
    _check_cuda(blkval, "blkval", torch.float32, 2)
    if blkval.shape[1] != 2:
        raise RuntimeError("blkval must be [nblk, 2]")
    mask = torch.empty(int(nnz), dtype=torch.int32, device=rowPtr.device)
    check(lib().pspmm_genmask(_ptr(rowPtr_bcsr), _ptr(rowPtr), _ptr(blkval),
                              rowPtr_bcsr.shape[0] - 1, rowPtr.shape[0] - 1, int(nnz), _ptr(mask),
                              _stream()))
    return mask


# ----------------------------------------------------------------------------- GCN layer (SpCONV)
def _pad_cols(t, pad):
    return torch.nn.functional.pad(t, (0, pad)) if pad else t


def _conv_forward(V, H, weight, rowPtr, colIdx, val, target_row, CF, W, product=None):
    """A @ (H @ W): dense GEMM (cuBLAS through torch.mm) then SpMM (SpCONV/SpCONV.h:43-193).

    An output width that is not a multiple of 4 (class counts: 47, 41, ...) is carried as the next
    multiple of 4 through both products, by a zero column appended to the weights, so that the
    SpMM runs with 128-bit accesses on 16-byte aligned rows; the extra column is dropped from the
    result.  ``product`` replaces the SpMM launch (an operator bound to a decider plan)."""
    _check_legacy(CF, W, max_cf=4)  # SpCONV/SpCONV.cpp:93-104
    fout = weight.shape[1]
    HW = torch.mm(H, _pad_cols(weight, -fout % 4))
    n = HW.shape[0]
    out = product(HW) if product else _spmm(HW, rowPtr, colIdx, val, target_row, V, CF, W)
    if out.shape[0] != n:
        out = out[:n]  # block variants slice back (SpCONV.h:115-118)
    return out[:, :fout].contiguous() if out.shape[1] != fout else out


def _conv_backward(V, g_out, H, weight, rowPtr, colIdx, val, target_row, CF, W, product=None, input_grad=True):
    """AG = A @ g_out (A itself, the normalised adjacency is symmetric); dH = AG @ W^T;
    dW = H^T @ AG (SpCONV/SpCONV.h:57-72).  Odd widths are padded as in the forward.
    ``input_grad=False`` leaves dH out (None): the first layer of a network has no use for it."""
    _check_legacy(CF, W, max_cf=4)
    fout = g_out.shape[1]
    pad = -fout % 4
    g_out = _pad_cols(g_out, pad).contiguous()
    n = g_out.shape[0]
    AG = product(g_out) if product else _spmm(g_out, rowPtr, colIdx, val, target_row, V, CF, W)
    if AG.shape[0] != n:
        AG = AG[:n]
    d_weight = torch.mm(H.t(), AG)
    d_input = torch.mm(AG, _pad_cols(weight, pad).t()) if input_grad else None
    return [d_input, d_weight[:, :fout].contiguous() if pad else d_weight]


def csr_spmm_forward(H, weight, rowPtr, colIdx, val, CF, blkWarpNum):
    return _conv_forward(1, H, weight, rowPtr, colIdx, val, None, CF, blkWarpNum)


def csr_spmm_backward(g_out, H, weight, rowPtr, colIdx, val, CF, blkWarpNum):
    return _conv_backward(1, g_out, H, weight, rowPtr, colIdx, val, None, CF, blkWarpNum)


def csr_split_spmm_forward(H, weight, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum):
    return _conv_forward(1, H, weight, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum)


def csr_split_spmm_backward(g_out, H, weight, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum):
    return _conv_backward(1, g_out, H, weight, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum)


def bcsr_spmm_forward(H, weight, rowPtr, colIdx, val, CF, blkWarpNum):
    return _conv_forward(2, H, weight, rowPtr, colIdx, val, None, CF, blkWarpNum)


def bcsr_spmm_backward(g_out, H, weight, rowPtr, colIdx, val, CF, blkWarpNum):
    return _conv_backward(2, g_out, H, weight, rowPtr, colIdx, val, None, CF, blkWarpNum)


def bcsr_split_spmm_forward(H, weight, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum):
    return _conv_forward(2, H, weight, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum)


def bcsr_split_spmm_backward(g_out, H, weight, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum):
    return _conv_backward(2, g_out, H, weight, rowPtr_split, colIdx, val, target_row, CF, blkWarpNum)
