"""CPU tests of the C-ABI library: it loads, exports what include/pspmm.h declares, its host
builders are bit-exact, and argument errors are reported as codes (no GPU call is made)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "pspmm.h")).read()
    return sorted(set(re.findall(r"PSPMM_API\s+[\w \*]+?\b(pspmm_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pspmm_lib):
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(pspmm_lib, n), "libpspmm.so does not export %s" % n
    from paramspmm_ae_b200 import _lib
    assert sorted(_lib.EXPORTED) == sorted(n for n in names if n in _lib.EXPORTED)
    assert set(_lib.EXPORTED) <= set(names)
    assert pspmm_lib.pspmm_version() >= 100
    assert pspmm_lib.pspmm_strerror(0) == b"ok"
    assert b"CF" in pspmm_lib.pspmm_strerror(-2)


def test_split_csr_bit_exact_with_golden_and_oracle(pspmm_lib, oracle, golden_dir):
    from paramspmm_ae_b200 import ops
    z = np.load(os.path.join(golden_dir, "split_ref.npz"))
    for i in range(int(z["n_cases"])):
        rp = torch.from_numpy(z["rowPtr_%d" % i])
        gran = int(z["gran_%d" % i])
        rps, tr = ops.split_csr(rp, gran)
        assert rps.dtype == torch.int32 and tr.dtype == torch.int32
        assert np.array_equal(rps.numpy(), z["rowPtr_split_%d" % i])
        assert np.array_equal(tr.numpy(), z["target_row_%d" % i])
        pieces = oracle.row_split_counts(z["rowPtr_%d" % i], gran)
        off = torch.from_numpy(np.concatenate([[0], np.cumsum(pieces)]).astype(np.int32))
        rps2, tr2 = ops.split_csr_par(rp, off, gran)
        assert torch.equal(rps, rps2) and torch.equal(tr, tr2)


def test_split_csr_large_random_matches_oracle(pspmm_lib, oracle):
    from paramspmm_ae_b200 import ops
    rng = np.random.default_rng(8)
    ln = rng.zipf(1.8, size=300000).clip(max=50000)
    ln[rng.random(ln.shape[0]) < 0.1] = 0
    rp = np.concatenate([[0], np.cumsum(ln)]).astype(np.int32)
    for gran in (32, 512):
        rps, tr = ops.split_csr(torch.from_numpy(rp), gran)
        o_rps, o_tr = oracle.split_csr(rp, gran)
        assert np.array_equal(rps.numpy(), o_rps) and np.array_equal(tr.numpy(), o_tr)


def test_split_csr_edge_cases(pspmm_lib):
    from paramspmm_ae_b200 import ops
    rps, tr = ops.split_csr(torch.zeros(1, dtype=torch.int32), 32)  # no rows
    assert rps.tolist() == [0] and tr.numel() == 0
    rps, tr = ops.split_csr(torch.zeros(6, dtype=torch.int32), 32)  # only empty rows
    assert rps.tolist() == [0] and tr.numel() == 0
    rps, tr = ops.split_csr(torch.tensor([0, 64], dtype=torch.int32), 32)  # exact multiple
    assert rps.tolist() == [0, 32, 64] and tr.tolist() == [0, 0]
    with pytest.raises(RuntimeError):
        ops.split_csr(torch.tensor([0, 4], dtype=torch.int32), 0)
    with pytest.raises(RuntimeError):
        ops.split_csr(torch.tensor([0, 4], dtype=torch.int64), 2)


def test_bcsr_builder_bit_exact(pspmm_lib, oracle, golden_dir):
    from paramspmm_ae_b200 import ops
    z = np.load(os.path.join(golden_dir, "bcsr_scipy.npz"))
    for i in range(int(z["n_cases"])):
        rp, ci, v, V = z["rowPtr_%d" % i], z["colIdx_%d" % i], z["val_%d" % i], int(z["V_%d" % i])
        rpb, cb, vb = ops.bcsr_from_csr(torch.from_numpy(rp), torch.from_numpy(ci), torch.from_numpy(v),
                                        rp.shape[0] - 1, V)
        assert np.array_equal(rpb.numpy(), z["rowPtr_b_%d" % i])
        assert np.array_equal(cb.numpy(), z["colIdx_b_%d" % i])
        assert np.array_equal(vb.numpy(), z["val_b_%d" % i])


def test_bcsr_builder_matches_scipy_on_power_law(pspmm_lib):
    from paramspmm_ae_b200 import ops, synth
    m = synth.powerlaw_graph(3001, 20000, seed=5)
    rp, ci, v = m.numpy()
    import scipy.sparse as sp
    n = m.n_rows
    pad = np.concatenate([rp, [rp[-1]]])
    b = sp.csr_array((v, ci, pad), shape=(n + 1, n + 1)).tobsr(blocksize=(2, 1))
    rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, n, 2)
    assert np.array_equal(rpb.numpy(), b.indptr) and np.array_equal(cb.numpy(), b.indices)
    assert np.array_equal(vb.numpy(), b.data.reshape(-1, 2))


def test_argument_errors_are_codes_not_crashes(pspmm_lib):
    from paramspmm_ae_b200 import _lib
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)  # never dereferenced: validation fails first
    cfg = _lib.make_cfg()
    # dim <= 0
    assert pspmm_lib.pspmm_spmm_csr(one, one, one, one, one, 4, 4, 4, 0, 8, 8, ctypes.byref(cfg),
                                    null, null, 0, null) == _lib.PSPMM_E_ARG
    # leading dimension smaller than dim
    assert pspmm_lib.pspmm_spmm_csr(one, one, one, one, one, 4, 4, 4, 16, 8, 16, ctypes.byref(cfg),
                                    null, null, 0, null) == _lib.PSPMM_E_ARG
    # null operand
    assert pspmm_lib.pspmm_spmm_csr(one, one, one, null, one, 4, 4, 4, 16, 16, 16, ctypes.byref(cfg),
                                    null, null, 0, null) == _lib.PSPMM_E_ARG
    # split arrays must come together
    assert pspmm_lib.pspmm_spmm_csr(one, one, one, one, one, 4, 4, 4, 16, 16, 16, ctypes.byref(cfg),
                                    one, null, 3, null) == _lib.PSPMM_E_ARG
    # index range
    assert pspmm_lib.pspmm_spmm_csr(one, one, one, one, one, 4, 4, 2 ** 31, 16, 16, 16,
                                    ctypes.byref(cfg), null, null, 0, null) == _lib.PSPMM_E_RANGE
    # legacy hints keep the reference's domain
    for bad in (_lib.make_cfg(CF=9, blkWarpNum=4), _lib.make_cfg(CF=1, blkWarpNum=5),
                _lib.make_cfg(lanes_per_row=3), _lib.make_cfg(vec_width=3), _lib.make_cfg(cta_threads=100),
                _lib.make_cfg(accumulate=2), _lib.make_cfg(accumulate=-1), _lib.make_cfg(col_tile=6)):
        assert pspmm_lib.pspmm_spmm_csr(one, one, one, one, one, 4, 4, 4, 16, 16, 16, ctypes.byref(bad),
                                        null, null, 0, null) == _lib.PSPMM_E_CONFIG
    assert pspmm_lib.pspmm_sddmm_csr(one, one, one, one, one, 4, 4, 16, 16, 16,
                                     ctypes.byref(_lib.make_cfg(CF=5, blkWarpNum=4)), null, null, 0,
                                     null) == _lib.PSPMM_E_CONFIG
    # SDDMM has nothing to add into
    assert pspmm_lib.pspmm_sddmm_csr(one, one, one, one, one, 4, 4, 16, 16, 16,
                                     ctypes.byref(_lib.make_cfg(accumulate=1)), null, null, 0,
                                     null) == _lib.PSPMM_E_CONFIG
    assert pspmm_lib.pspmm_spmm_bcsr(one, one, one, 4, one, one, 4, 4, 4, 16, 16, 16, ctypes.byref(cfg),
                                     null, null, 0, null) == _lib.PSPMM_E_UNSUPPORTED
    with pytest.raises(_lib.PspmmError):
        _lib.check(_lib.PSPMM_E_ARG)


def test_config_resolution_covers_every_dim(pspmm_lib):
    """Every dim 1..1100 and block height resolves to an instantiated kernel shape."""
    from paramspmm_ae_b200 import _lib
    for V in (1, 2, 3):
        for dim in list(range(1, 300)) + [512, 1000, 1024, 1100]:
            cfg = _lib.make_cfg()
            rc = pspmm_lib.pspmm_resolve_cfg(ctypes.byref(cfg), dim, dim, dim, V, ctypes.c_void_p(256),
                                             ctypes.c_void_p(256))
            assert rc == 0
            assert cfg.vec_width == (4 if dim % 4 == 0 else 2 if dim % 2 == 0 else 1)
            assert cfg.lanes_per_row in (1, 2, 4, 8, 16, 32)
    cfg = _lib.make_cfg()
    assert pspmm_lib.pspmm_resolve_cfg(ctypes.byref(cfg), 64, 64, 64, 1, ctypes.c_void_p(256),
                                       ctypes.c_void_p(256)) == 0
    assert (cfg.lanes_per_row, cfg.vec_width) == (16, 4)
    # a misaligned base pointer or odd leading dimension narrows the vector width
    cfg = _lib.make_cfg()
    pspmm_lib.pspmm_resolve_cfg(ctypes.byref(cfg), 64, 64, 64, 1, ctypes.c_void_p(260), ctypes.c_void_p(256))
    assert cfg.vec_width == 1
    cfg = _lib.make_cfg()
    pspmm_lib.pspmm_resolve_cfg(ctypes.byref(cfg), 64, 66, 64, 1, ctypes.c_void_p(256), ctypes.c_void_p(256))
    assert cfg.vec_width == 2


def test_ops_reject_cpu_tensors_and_bad_hints():
    """The torch-level operators never fall back: a CPU tensor or an invalid CF / blkWarpNum is
    an error, as in the reference (SpMM/SpMM.cpp:5-13, 110, 139)."""
    from paramspmm_ae_b200 import ops
    X = torch.zeros(4, 8)
    rp = torch.zeros(5, dtype=torch.int32)
    ci = torch.zeros(0, dtype=torch.int32)
    v = torch.zeros(0)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        ops.csr_spmm(X, rp, ci, v, 1, 4)
    with pytest.raises(RuntimeError, match="blkWarpNum"):
        ops.csr_spmm(X, rp, ci, v, 1, 6)
    with pytest.raises(RuntimeError, match="CF"):
        ops.csr_spmm(X, rp, ci, v, 9, 4)
    with pytest.raises(RuntimeError, match="CF"):
        ops.csr_sddmm(X, X, rp, ci, v, 5, 4)


def test_dropin_modules_expose_reference_names():
    import paramspmm_ae_b200
    paramspmm_ae_b200.install_dropin()
    import ParamSDDMM
    import ParamSpCONV
    import ParamSpMM
    spmm_names = """split_csr split_csr_par csr_spmm csr_split_spmm bcsr_spmm bcsr_split_spmm vec_spmm
        vec_split_spmm csr_spmm_profile csr_split_spmm_profile bcsr_spmm_profile bcsr_split_spmm_profile
        vec_spmm_profile vec_split_spmm_profile cusparse_compute cusparse_profile cusparse_compute_csr_alg2
        cusparse_profile_csr_alg2 cusparse_compute_coo_alg4 cusparse_profile_coo_alg4 cusparse_compute_csc
        cusparse_profile_csc gespmm_compute gespmm_profile""".split()
    sddmm_names = """csr_sddmm csr_split_sddmm bcsr_sddmm bcsr_split_sddmm vec_sddmm vec_split_sddmm
        csr_sddmm_profile csr_split_sddmm_profile bcsr_sddmm_profile bcsr_split_sddmm_profile
        vec_sddmm_profile vec_split_sddmm_profile cusparse_sddmm_compute cusparse_sddmm_profile genmask""".split()
    conv_names = """split_csr split_csr_par csr_spmm_forward csr_spmm_backward csr_split_spmm_forward
        csr_split_spmm_backward bcsr_spmm_forward bcsr_spmm_backward bcsr_split_spmm_forward
        bcsr_split_spmm_backward""".split()
    for mod, names in ((ParamSpMM, spmm_names), (ParamSDDMM, sddmm_names), (ParamSpCONV, conv_names)):
        for n in names:
            assert callable(getattr(mod, n)), "%s.%s missing" % (mod.__name__, n)


def test_table_plans_become_valid_kernel_configurations():
    """Every entry of the measured table decodes into a pspmm_cfg the library accepts (including
    the column-tile field), for every regime and every dim key."""
    import ctypes
    from paramspmm_ae_b200 import _lib, decider
    lib = _lib.lib()
    tab = decider.load_table()
    seen = 0
    for regime, per_dim in tab["entries"]["spmm"].items():
        for dim_key, e in per_dim.items():
            plan = decider.Plan(if_split=0, vec_size=1, granularity=None)
            plan.update(e)
            cfg = _lib.make_cfg(**plan.kernel_cfg())
            assert cfg.col_tile in (0, 32, 64, 128) and cfg.bucketed in (0, 1)
            dim = int(dim_key)
            rc = lib.pspmm_resolve_cfg(ctypes.byref(cfg), dim, dim, dim, 1, ctypes.c_void_p(256), ctypes.c_void_p(256))
            assert rc == _lib.PSPMM_OK, (regime, dim_key, e)
            assert cfg.lanes_per_row in (2, 4, 8, 16, 32) and cfg.cta_threads in (32, 64, 128, 256)
            seen += 1
    assert seen >= 64


def test_table_measures_every_regime_and_the_decider_reaches_them():
    """The committed table holds a measured entry for every regime the fit covers and for every
    dim key; the regime rule sends the generators' matrices where the fit put them; a regime
    without measurements borrows from its nearest measured neighbour."""
    import torch
    from paramspmm_ae_b200 import decider, sweep, synth
    tab = decider.load_table()
    regimes = tab["entries"]["spmm"]
    for r in sweep.ALL_REGIMES:
        assert r in regimes, r
        assert set(regimes[r]) == {str(d) for d in range(16, 257, 16)}, r
    cases = [(synth.uniform_rows(4000, 4, seed=1), "tiny_even"), (synth.uniform_rows(4000, 16, seed=1), "short_even"),
             (synth.banded_rows(4000, 16, 32, seed=1), "short_local"), (synth.uniform_rows(3000, 64, seed=1), "medium_even"),
             (synth.banded_rows(3000, 64, 96, seed=1), "medium_local"), (synth.rmat(12, 4 * 4096, seed=1), "tiny_skewed"),
             (synth.rmat(12, 16 * 4096, seed=1), "short_skewed"), (synth.powerlaw_graph(3000, 75000, seed=1), "medium_skewed")]
    for m, want in cases:
        st = decider.row_stats(m.rowPtr, m.colIdx)
        assert decider.regime(st) == want, (want, st)
        for dim in (16, 100, 256, 300):
            p = decider.choose(st, dim)
            assert p["regime"] == want and p["vec_size"] in (1, 2)
            assert (p["granularity"] is not None) == bool(p["if_split"])
    # without column indices a banded matrix is an even one; long_local borrows (no fit matrix for it)
    b = synth.banded_rows(4000, 16, 32, seed=1)
    assert decider.regime(decider.row_stats(b.rowPtr)) == "short_even"
    st = {"n_rows": 10, "nnz": 3000, "avg": 300.0, "cov": 0.1, "max": 310, "real_avg": 300.0, "near_diag": 1.0}
    assert decider.regime(st) == "long_local" and decider.choose(st, 64)["regime"] == "long_local"


def test_header_is_plain_c_and_declares_what_the_python_shim_binds(tmp_path):
    """include/pspmm.h must compile as C99 and as C++ on its own (it is what a foreign-language
    binding includes), and every function the ctypes shim binds must be declared in it."""
    import os
    import re
    import subprocess
    from paramspmm_ae_b200 import _lib
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hdr = os.path.join(root, "include", "pspmm.h")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-fsyntax-only", "-x", "c", hdr], check=True)
    subprocess.run(["g++", "-std=c++14", "-Wall", "-Werror", "-fsyntax-only", "-x", "c++", hdr], check=True)
    text = open(hdr).read()
    declared = set(re.findall(r"PSPMM_API\s+[\w\s\*]+?\b(pspmm_\w+)\s*\(", text))
    assert set(_lib.EXPORTED) <= declared, sorted(set(_lib.EXPORTED) - declared)
    # a C caller can fill the configuration struct by name
    src = tmp_path / "use.c"
    src.write_text('#include "pspmm.h"\nint main(void) { pspmm_cfg c = {0}; c.col_tile = 128; c.hint_CF = 2; '
                   'return pspmm_version() > 0 && c.col_tile == 128 ? 0 : 1; }\n')
    exe = tmp_path / "use"
    subprocess.run(["gcc", "-std=c99", "-I", os.path.join(root, "include"), str(src), "-o", str(exe),
                    _lib.LIB_PATH, "-Wl,-rpath," + os.path.dirname(_lib.LIB_PATH)], check=True)
    assert subprocess.run([str(exe)]).returncode == 0


def test_new_entry_points_validate_before_touching_the_device(pspmm_lib):
    """pspmm_pull_rows, pspmm_agnn_fused_apply_csr, the bucketed flag and the block SDDMM's row count
    of A: bad arguments come back as codes (no CUDA call is reached with them)."""
    from paramspmm_ae_b200 import _lib
    null, one = ctypes.c_void_p(0), ctypes.c_void_p(16)
    src = _lib.RowSources()
    src.n_src = 1
    src.base[0] = 16
    src.first[0], src.first[1] = 0, 8
    call = lambda n, dim, lds, ldd, rot, s=src: pspmm_lib.pspmm_pull_rows(ctypes.byref(s), one, n, one, dim, lds, ldd, rot, 0, null)
    assert call(8, 0, 16, 16, 0) == _lib.PSPMM_E_ARG            # dim
    assert call(8, 16, 8, 16, 0) == _lib.PSPMM_E_ARG            # row stride smaller than dim
    assert call(8, 16, 16, 16, 8) == _lib.PSPMM_E_ARG           # rotate outside the list
    assert call(9, 16, 16, 16, 0) == _lib.PSPMM_E_ARG           # the sources do not cover the list
    assert call(8, 18, 20, 20, 0) == _lib.PSPMM_E_UNSUPPORTED   # not 128-bit accessible
    assert call(0, 16, 16, 16, 0) == _lib.PSPMM_OK              # nothing to copy
    bad = _lib.RowSources()
    bad.n_src = _lib.MAX_ROW_SOURCES + 1
    assert call(8, 16, 16, 16, 0, bad) == _lib.PSPMM_E_ARG
    # the bulk-copy form checks the same way; its status query wants somewhere to write
    bulk = lambda n, dim, lds, ldd, rot: pspmm_lib.pspmm_pull_rows_bulk(ctypes.byref(src), one, n, one, dim, lds, ldd, rot, 0, null)
    assert bulk(8, 0, 16, 16, 0) == _lib.PSPMM_E_ARG
    assert bulk(8, 16, 16, 16, 8) == _lib.PSPMM_E_ARG
    assert bulk(8, 18, 20, 20, 0) == _lib.PSPMM_E_UNSUPPORTED
    assert bulk(0, 16, 16, 16, 0) == _lib.PSPMM_OK
    assert pspmm_lib.pspmm_pull_rows_status(None) == _lib.PSPMM_E_ARG
    # bucketed is a 0/1 flag of the SpMM only
    assert pspmm_lib.pspmm_spmm_csr(one, one, one, one, one, 4, 4, 4, 16, 16, 16, ctypes.byref(_lib.make_cfg(bucketed=2)),
                                    null, null, 0, null) == _lib.PSPMM_E_CONFIG
    assert pspmm_lib.pspmm_sddmm_csr(one, one, one, one, one, 4, 4, 16, 16, 16, ctypes.byref(_lib.make_cfg(bucketed=1)),
                                     null, null, 0, null) == _lib.PSPMM_E_CONFIG
    # block SDDMM: A must reach into the last block-row
    cfg = _lib.make_cfg()
    assert pspmm_lib.pspmm_sddmm_bcsr(one, one, one, 2, one, one, one, 5, 8, 4, 16, 16, 16, ctypes.byref(cfg),
                                      null, null, 0, null) == _lib.PSPMM_E_ARG
    # fused aggregation with a separate operand: V missing, V's stride too small
    f = pspmm_lib.pspmm_agnn_fused_apply_csr
    assert f(one, one, one, one, null, one, 4, 4, 16, 16, 16, 16, 16, 1.0, 0, 0, 0, 0, null, null, 0, null, 0, null) == _lib.PSPMM_E_ARG
    assert f(one, one, one, one, one, one, 4, 4, 16, 16, 16, 8, 16, 1.0, 0, 0, 0, 0, null, null, 0, null, 0, null) == _lib.PSPMM_E_ARG


def test_block_builder_rejects_bad_columns_and_inconsistent_counts(pspmm_lib):
    """The host block builder range-checks column ids and never writes more blocks than the row
    pointer it is given allows."""
    import numpy as np
    from paramspmm_ae_b200 import _lib
    p = lambda a: ctypes.c_void_p(a.ctypes.data)
    rp = np.array([0, 2, 3, 5], dtype=np.int32)
    ci = np.array([0, 3, 1, 2, 9], dtype=np.int32)    # 9 is outside [0, 4)
    v = np.ones(5, dtype=np.float32)
    rpb = np.zeros(3, dtype=np.int32)
    nblk = ctypes.c_int64(0)
    assert pspmm_lib.pspmm_bcsr_count(p(rp), p(ci), 3, 4, 2, p(rpb), ctypes.byref(nblk)) == _lib.PSPMM_E_ARG
    ci[4] = 3
    assert pspmm_lib.pspmm_bcsr_count(p(rp), p(ci), 3, 4, 2, p(rpb), ctypes.byref(nblk)) == _lib.PSPMM_OK
    assert rpb.tolist() == [0, 3, 5] and nblk.value == 5
    # a row pointer that promises fewer blocks than the rows hold: an error, and the arrays' tails stay untouched
    lie = np.array([0, 1, 2], dtype=np.int32)
    cb = np.full(6, -7, dtype=np.int32)
    vb = np.full(12, -7.0, dtype=np.float32)
    assert pspmm_lib.pspmm_bcsr_fill(p(rp), p(ci), p(v), 3, 4, 2, p(lie), p(cb), p(vb)) == _lib.PSPMM_E_ARG
    assert (cb[2:] == -7).all() and (vb[4:] == -7).all()
