"""ctypes binding of libpspmm.so (the C ABI declared in include/pspmm.h).

There is no fallback: if the shared library is missing or a call fails, an exception is
raised.  Build it with ``python -m paramspmm_ae_b200.build``.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libpspmm.so")
BASELINES_PATH = os.path.join(_PKG, "libpspmm_baselines.so")

PSPMM_OK = 0
PSPMM_E_ARG = -1
PSPMM_E_CONFIG = -2
PSPMM_E_CUDA = -3
PSPMM_E_UNSUPPORTED = -4
PSPMM_E_RANGE = -5
PSPMM_E_IO = -6
PSPMM_E_FORMAT = -7
PSPMM_E_NOMEM = -8

_i32 = ctypes.c_int32
_i64 = ctypes.c_int64
_vp = ctypes.c_void_p


class PspmmCfg(ctypes.Structure):
    """Mirror of ``pspmm_cfg``; zero fields mean "library's choice"."""

    _fields_ = [("lanes_per_row", _i32), ("vec_width", _i32), ("cta_threads", _i32),
                ("rows_per_group", _i32), ("gather_batch", _i32), ("col_tile", _i32), ("hint_CF", _i32),
                ("hint_blkWarpNum", _i32), ("bucketed", _i32), ("accumulate", _i32)]


class MtxInfo(ctypes.Structure):
    """Mirror of ``pspmm_mtx_info``."""

    _fields_ = [("n_rows", _i64), ("n_cols", _i64), ("stored", _i64), ("nnz_max", _i64),
                ("symmetric", _i32), ("field", _i32)]


class CsrFileInfo(ctypes.Structure):
    """Mirror of ``pspmm_csr_file_info_t``."""

    _fields_ = [("n_rows", _i64), ("n_cols", _i64), ("nnz", _i64), ("source_size", _i64),
                ("source_mtime_ns", _i64)]


MAX_ROW_SOURCES = 16


class RowSources(ctypes.Structure):
    """Mirror of ``pspmm_row_sources``."""

    _fields_ = [("base", _vp * MAX_ROW_SOURCES), ("first", _i64 * (MAX_ROW_SOURCES + 1)), ("n_src", _i32)]


class PspmmError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("libpspmm: %s (code %d)" % (text, code))
        self.code = code


_cfgp = ctypes.POINTER(PspmmCfg)

# name -> argument types, exactly as declared in include/pspmm.h
_SIGNATURES = {
    "pspmm_resolve_cfg": [_cfgp, _i32, _i64, _i64, _i32, _vp, _vp],
    "pspmm_spmm_csr": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i64, _i64, _cfgp, _vp, _vp,
                       _i64, _vp],
    "pspmm_spmm_bcsr": [_vp, _vp, _vp, _i32, _vp, _vp, _i64, _i64, _i64, _i32, _i64, _i64, _cfgp,
                        _vp, _vp, _i64, _vp],
    "pspmm_sddmm_csr": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i64, _i64, _cfgp, _vp, _vp, _i64,
                        _vp],
    "pspmm_sddmm_bcsr": [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i64, _i64, _cfgp,
                         _vp, _vp, _i64, _vp],
    "pspmm_genmask": [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp],
    "pspmm_split_count": [_vp, _i64, _i32, ctypes.POINTER(_i64)],
    "pspmm_split_csr": [_vp, _i64, _i32, _vp, _vp, _i64],
    "pspmm_split_device_scratch_bytes": [_i64, ctypes.POINTER(ctypes.c_size_t)],
    "pspmm_split_count_device": [_vp, _i64, _i32, _vp, ctypes.c_size_t, ctypes.POINTER(_i64), _vp],
    "pspmm_split_csr_device": [_vp, _i64, _i32, _vp, _vp, _i64, _vp, ctypes.c_size_t, _vp],
    "pspmm_split_csr_device_static": [_vp, _i64, _i32, _vp, _vp, _i64, _vp],
    "pspmm_agnn_scratch_bytes": [_i64, _i32, ctypes.POINTER(ctypes.c_size_t)],
    "pspmm_agnn_fused_apply_csr": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i64, _i64, _i64, _i64,
                                   ctypes.c_float, _i32, _i32, _i32, _i32, _vp, _vp, _i64, _vp, ctypes.c_size_t, _vp],
    "pspmm_agnn_fused_csr": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i64, _i64, _i64, ctypes.c_float, _i32,
                             _i32, _i32, _i32, _vp, _vp, _i64, _vp, ctypes.c_size_t, _vp],
    "pspmm_pull_rows": [ctypes.POINTER(RowSources), _vp, _i64, _vp, _i32, _i64, _i64, _i64, _i32, _vp],
    "pspmm_pull_rows_bulk": [ctypes.POINTER(RowSources), _vp, _i64, _vp, _i32, _i64, _i64, _i64, _i32, _vp],
    "pspmm_pull_rows_status": [ctypes.POINTER(ctypes.c_int32)],
    "pspmm_bcsr_count": [_vp, _vp, _i64, _i64, _i32, _vp, ctypes.POINTER(_i64)],
    "pspmm_bcsr_fill": [_vp, _vp, _vp, _i64, _i64, _i32, _vp, _vp, _vp],
    "pspmm_mtx_info_read": [ctypes.c_char_p, ctypes.POINTER(MtxInfo)],
    "pspmm_mtx_read_csr": [ctypes.c_char_p, _i32, _vp, _vp, _vp, _i64, ctypes.POINTER(_i64)],
    "pspmm_csr_file_write": [ctypes.c_char_p, _i64, _i64, _i64, _vp, _vp, _vp, _i64, _i64],
    "pspmm_csr_file_info": [ctypes.c_char_p, ctypes.POINTER(CsrFileInfo)],
    "pspmm_csr_file_read": [ctypes.c_char_p, _vp, _vp, _vp, _i64, _i64, _i32],
    "pspmm_profile_spmm": [_vp, _vp, _vp, _i32, _vp, _vp, _i64, _i64, _i64, _i32, _i64, _i64, _cfgp,
                           _vp, _vp, _i64, _i32, _i32, ctypes.POINTER(ctypes.c_float), _vp],
    "pspmm_profile_sddmm": [_vp, _vp, _vp, _i32, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i64, _i64, _cfgp,
                            _vp, _vp, _i64, _i32, _i32, ctypes.POINTER(ctypes.c_float), _vp],
}
EXPORTED = ["pspmm_version", "pspmm_strerror", "pspmm_last_cuda_error"] + list(_SIGNATURES)

_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s not found: build it with `python -m paramspmm_ae_b200.build` "
                              "(there is no CPU or PyTorch fallback)" % LIB_PATH)
        handle = ctypes.CDLL(LIB_PATH)
        handle.pspmm_version.restype = ctypes.c_int
        handle.pspmm_strerror.restype = ctypes.c_char_p
        handle.pspmm_strerror.argtypes = [ctypes.c_int]
        handle.pspmm_last_cuda_error.restype = ctypes.c_char_p
        for name, args in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = ctypes.c_int
            fn.argtypes = args
        _lib = handle
    return _lib


def check(code):
    """Raise PspmmError for a non-zero return code."""
    if code == PSPMM_OK:
        return
    handle = lib()
    text = handle.pspmm_strerror(code).decode()
    if code == PSPMM_E_CUDA:
        text += ": " + handle.pspmm_last_cuda_error().decode()
    raise PspmmError(code, text)


def make_cfg(CF=0, blkWarpNum=0, lanes_per_row=0, vec_width=0, cta_threads=0, rows_per_group=0,
             gather_batch=0, col_tile=0, accumulate=0, bucketed=0):
    return PspmmCfg(lanes_per_row, vec_width, cta_threads, rows_per_group, gather_batch, col_tile, CF, blkWarpNum,
                    bucketed, accumulate)
