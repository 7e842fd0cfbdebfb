"""GPU parity tests: the CUDA kernels, called through the C ABI (ctypes), against the CPU oracle.

Tolerance for floating-point results: |got - want| <= 1e-4 + 1e-5 * |want| (max relative error
1e-5 with an absolute floor of 1e-4), the bound the project states for fp32 outputs.  Index
arrays must match bit for bit.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-4


def close(got, want):
    got = got.detach().cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got)
    np.testing.assert_allclose(got, np.asarray(want), rtol=RTOL, atol=ATOL)


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    from paramspmm_ae_b200 import _lib
    _lib.lib()  # fails loudly when the CUDA library has not been built
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def mats():
    """Small seeded matrices covering the row-length regimes, each with some empty rows."""
    from paramspmm_ae_b200 import synth
    out = {
        "powerlaw": synth.powerlaw_graph(3001, 24000, seed=1),          # odd n, hub rows, self loops
        "uniform16": synth.uniform_rows(2000, 16, seed=21),              # every row exactly 16
        "banded": synth.banded_rows(1500, 16, 32, seed=22),
        "rmat": synth.with_empty_rows(synth.rmat(12, 60000, seed=23), every=5),
        "tiny": synth.uniform_rows(7, 3, seed=2),
    }
    # one matrix whose row 0 is far longer than any partition length
    hub = synth.uniform_rows(1200, 4, seed=3)
    rp = hub.rowPtr.clone().long()
    g = torch.Generator().manual_seed(4)
    extra_cols = torch.sort(torch.randperm(1200, generator=g)[:900]).values.int()
    ci = torch.cat([extra_cols, hub.colIdx[4:]])
    v = torch.cat([torch.rand(900, generator=g), hub.val[4:]])
    rp[1:] += 900 - 4
    out["hub"] = synth.CSR(rp.int(), ci, v, 1200, 1200)
    return out


def dense(n, dim, seed):
    from paramspmm_ae_b200 import synth
    return synth.dense_uniform(n, dim, seed)


DIMS = [1, 3, 4, 8, 16, 20, 32, 47, 48, 64, 80, 100, 128, 160, 256, 260]


@pytest.mark.parametrize("name", ["powerlaw", "uniform16", "banded", "rmat", "tiny", "hub"])
def test_csr_spmm_matches_oracle(dev, oracle, mats, name):
    from paramspmm_ae_b200 import ops
    m = mats[name]
    rp, ci, v = m.numpy()
    d = m.to(dev)
    for dim in DIMS:
        B = dense(m.n_cols, dim, 100 + dim)
        want = oracle.spmm_csr(rp, ci, v, B.numpy())
        got = ops.csr_spmm(B.to(dev), d.rowPtr, d.colIdx, d.val, 1, 4)
        assert got.shape == (m.n_rows, dim)
        close(got, want)


def test_csr_spmm_meets_the_reference_acceptance_rule(dev, oracle, mats):
    """verification.py:79-102: no element may differ by more than 1e-4 relative from
    torch.sparse.mm (computed here on the CPU)."""
    from paramspmm_ae_b200 import ops
    m = mats["uniform16"]
    rp, ci, v = m.numpy()
    d = m.to(dev)
    B = torch.ones(m.n_cols, 32)  # the operand the reference itself verifies with
    ref = oracle.spmm_torch_cpu(rp, ci, v, B.numpy())
    got = ops.csr_spmm(B.to(dev), d.rowPtr, d.colIdx, d.val, 1, 8).cpu().numpy()
    assert oracle.verification_compare(ref, got, rel=1e-4)


def test_golden_spmm_fixture(dev, golden_dir):
    from paramspmm_ae_b200 import ops
    z = np.load(os.path.join(golden_dir, "spmm_torch.npz"))
    t = lambda k: torch.from_numpy(z[k]).to(dev)
    got = ops.csr_spmm(t("B"), t("rowPtr"), t("colIdx"), t("val"), 1, 4)
    close(got, z["C_torch"])
    close(got, z["C_scipy"])


@pytest.mark.parametrize("name", ["powerlaw", "rmat", "hub", "uniform16"])
@pytest.mark.parametrize("gran", [1, 7, 32, 512])
def test_csr_split_spmm_matches_oracle(dev, oracle, mats, name, gran):
    from paramspmm_ae_b200 import ops
    m = mats[name]
    rp, ci, v = m.numpy()
    rps, tr = ops.split_csr(m.rowPtr, gran)
    o_rps, o_tr = oracle.split_csr(rp, gran)
    assert np.array_equal(rps.numpy(), o_rps) and np.array_equal(tr.numpy(), o_tr)
    d = m.to(dev)
    for dim in (4, 16, 47, 64, 100, 128, 256):
        B = dense(m.n_cols, dim, 200 + dim)
        want = oracle.spmm_csr_split(o_rps, o_tr, ci, v, B.numpy(), m.n_rows)
        got = ops.csr_split_spmm(B.to(dev), rps.to(dev), d.colIdx, d.val, tr.to(dev), 1, 4)
        close(got, want)
        close(got, oracle.spmm_csr(rp, ci, v, B.numpy()))


@pytest.mark.parametrize("V", [2, 3])
@pytest.mark.parametrize("name", ["powerlaw", "rmat", "tiny", "hub"])
def test_block_spmm_matches_oracle(dev, oracle, mats, name, V):
    from paramspmm_ae_b200 import ops
    m = mats[name]
    rp, ci, v = m.numpy()
    rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, m.n_cols, V)
    o = oracle.bcsr_build(rp, ci, v, m.n_cols, V)
    assert np.array_equal(rpb.numpy(), o[0]) and np.array_equal(cb.numpy(), o[1])
    assert np.array_equal(vb.numpy(), o[2])
    nbr = rpb.shape[0] - 1
    fn = ops.bcsr_spmm if V == 2 else ops.vec_spmm
    fn_split = ops.bcsr_split_spmm if V == 2 else ops.vec_split_spmm
    s_rpb, s_tr = ops.split_csr(rpb, 8)
    for dim in (4, 16, 47, 64, 96, 128, 256):
        B = dense(m.n_cols, dim, 300 + dim)
        want = oracle.spmm_bcsr(o[0], o[1], o[2], B.numpy(), nbr)
        got = fn(B.to(dev), rpb.to(dev), cb.to(dev), vb.to(dev), 1, 4)
        assert got.shape == (nbr * V, dim)  # rows padded to a multiple of V
        close(got, want)
        close(got[: m.n_rows], oracle.spmm_csr(rp, ci, v, B.numpy()))
        got = fn_split(B.to(dev), s_rpb.to(dev), cb.to(dev), vb.to(dev), s_tr.to(dev), 2, 8)
        close(got, want)


def test_spmm_explicit_configs(dev, oracle, mats):
    """Every kernel parameter the configuration table can choose gives the same product."""
    from paramspmm_ae_b200 import _lib, ops
    m = mats["rmat"]
    rp, ci, v = m.numpy()
    d = m.to(dev)
    rps, tr = ops.split_csr(m.rowPtr, 32)
    rps, tr = rps.to(dev), tr.to(dev)
    for dim in (16, 48, 64, 96, 128, 256):
        B = dense(m.n_cols, dim, 400 + dim)
        want = oracle.spmm_csr(rp, ci, v, B.numpy())
        Bd = B.to(dev)
        for lpr in (2, 4, 8, 16, 32):
            for vw in (1, 2, 4):
                for thr, rpg, mlp in ((128, 1, 4), (256, 4, 8), (256, 16, 16), (256, 2, 2), (64, 4, 4), (32, 2, 8)):
                    cfg = _lib.make_cfg(lanes_per_row=lpr, vec_width=vw, cta_threads=thr, rows_per_group=rpg,
                                        gather_batch=mlp)
                    out = torch.full((m.n_rows, dim), float("nan"), device=dev)
                    ops.spmm_into(out, Bd, d.rowPtr, d.colIdx, d.val, cfg=cfg)
                    close(out, want)
                    out = torch.full((m.n_rows, dim), float("nan"), device=dev)
                    ops.spmm_into(out, Bd, rps, d.colIdx, d.val, target_row=tr, n_out_rows=m.n_rows, cfg=cfg)
                    close(out, want)


def test_spmm_strided_operands_and_row_shards(dev, oracle, mats):
    """Leading dimensions larger than dim, and an output with fewer rows than B (a row shard)."""
    from paramspmm_ae_b200 import ops
    m = mats["powerlaw"]
    rp, ci, v = m.numpy()
    d = m.to(dev)
    for dim, ld in ((64, 96), (47, 50), (20, 22)):
        wide = dense(m.n_cols, ld, 500 + dim)
        B = wide[:, :dim]
        want = oracle.spmm_csr(rp, ci, v, np.ascontiguousarray(B.numpy()))
        Bd = wide.to(dev)[:, :dim]
        out_wide = torch.zeros(m.n_rows, ld, device=dev)
        ops.spmm_into(out_wide[:, :dim], Bd, d.rowPtr, d.colIdx, d.val)
        close(out_wide[:, :dim], want)
        assert not out_wide[:, dim:].any()  # nothing written past dim
    # rows [lo, hi) of A as a shard with re-based row pointers and global column ids
    lo, hi = 700, 1900
    rp_s = (m.rowPtr[lo: hi + 1] - m.rowPtr[lo]).contiguous()
    a, b = int(m.rowPtr[lo]), int(m.rowPtr[hi])
    B = dense(m.n_cols, 64, 77)
    want = oracle.spmm_csr(rp, ci, v, B.numpy())[lo:hi]
    out = torch.empty(hi - lo, 64, device=dev)
    ops.spmm_into(out, B.to(dev), rp_s.to(dev), d.colIdx[a:b].contiguous(), d.val[a:b].contiguous())
    close(out, want)


def test_spmm_accumulate_over_column_blocks(dev, oracle, mats):
    """cfg.accumulate adds the product to C: summing the products of the column blocks of A, the
    first one in overwrite mode, gives A B; plain and split layouts, empty rows add nothing."""
    from paramspmm_ae_b200 import _lib, ops
    m = mats["rmat"]
    rp, ci, v = m.numpy()
    n = m.n_rows
    rows = np.repeat(np.arange(n), np.diff(rp))
    K = 3
    block = ci * K // m.n_cols  # column block of every entry
    for dim in (16, 64, 100, 256):
        B = dense(m.n_cols, dim, 900 + dim)
        want = oracle.spmm_csr(rp, ci, v, B.numpy())
        Bd = B.to(dev)
        for split in (False, True):
            for lpr in (0, 2, 32):
                out = torch.full((n, dim), float("nan"), device=dev)
                for k in range(K):
                    sel = block == k
                    rp_k = np.concatenate([[0], np.cumsum(np.bincount(rows[sel], minlength=n))]).astype(np.int32)
                    rp_k, ci_k, v_k = (torch.from_numpy(x).to(dev) for x in (rp_k, ci[sel], v[sel]))
                    cfg = _lib.make_cfg(lanes_per_row=lpr, accumulate=1 if k else 0,
                                        col_tile=128 if (dim == 256 and lpr == 32) else 0)
                    if split:
                        rps, tr = ops.split_csr_device(rp_k, 32)
                        ops.spmm_into(out, Bd, rps, ci_k, v_k, target_row=tr, n_out_rows=n, cfg=cfg)
                    else:
                        ops.spmm_into(out, Bd, rp_k, ci_k, v_k, cfg=cfg)
                close(out, want)
    # adding into an existing C, and a matrix without entries adds nothing
    C0 = dense(n, 64, 3).to(dev)
    B = dense(m.n_cols, 64, 4)
    d = m.to(dev)
    out = C0.clone()
    ops.spmm_into(out, B.to(dev), d.rowPtr, d.colIdx, d.val, cfg=_lib.make_cfg(accumulate=1))
    close(out - C0, oracle.spmm_csr(rp, ci, v, B.numpy()))
    out = C0.clone()
    ops.spmm_into(out, B.to(dev), torch.zeros(n + 1, dtype=torch.int32, device=dev), d.colIdx[:0], d.val[:0],
                  cfg=_lib.make_cfg(accumulate=1))
    assert torch.equal(out, C0)
    # built for 128-bit rows only: other widths are refused, not silently overwritten
    with pytest.raises(_lib.PspmmError) as e:
        ops.spmm_into(torch.zeros(n, 18, device=dev), dense(m.n_cols, 18, 1).to(dev), d.rowPtr, d.colIdx, d.val,
                      cfg=_lib.make_cfg(accumulate=1))
    assert e.value.code == _lib.PSPMM_E_UNSUPPORTED
    with pytest.raises(_lib.PspmmError):
        ops.spmm_into(out, B.to(dev), d.rowPtr, d.colIdx, d.val, cfg=_lib.make_cfg(accumulate=2))


def test_spmm_rejects_inconsistent_sizes(dev, mats):
    """A row pointer or an output that does not match the row count raises before any launch
    (the kernels index both by the row count alone)."""
    from paramspmm_ae_b200 import ops
    d = mats["powerlaw"].to(dev)
    n = d.n_rows
    B = dense(d.n_cols, 32, 5).to(dev)
    short_rp = d.rowPtr[: n // 2 + 1].contiguous()
    with pytest.raises(RuntimeError):  # plain CSR: n rows asked for, n/2 + 1 row pointers given
        ops.spmm_time_ms(B, short_rp, d.colIdx, d.val, warmup=1, iters=1)
    with pytest.raises(RuntimeError):
        ops.spmm_into(torch.empty(n, 32, device=dev), B, short_rp, d.colIdx, d.val, n_out_rows=n)
    with pytest.raises(RuntimeError):  # output with too few rows
        ops.spmm_into(torch.empty(n - 1, 32, device=dev), B, d.rowPtr, d.colIdx, d.val)
    with pytest.raises(RuntimeError):  # output of another width
        ops.spmm_into(torch.empty(n, 16, device=dev), B, d.rowPtr, d.colIdx, d.val)
    rps, tr = ops.split_csr(mats["powerlaw"].rowPtr, 32)
    with pytest.raises(RuntimeError):
        ops.spmm_time_ms(B, rps.to(dev), d.colIdx, d.val, tr.to(dev), out=torch.empty(n // 2, 32, device=dev),
                         warmup=1, iters=1)
    torch.cuda.synchronize()


def test_spmm_empty_inputs(dev):
    from paramspmm_ae_b200 import ops
    X = torch.randn(5, 16, device=dev)
    rp = torch.zeros(6, dtype=torch.int32, device=dev)
    e_i = torch.zeros(0, dtype=torch.int32, device=dev)
    e_f = torch.zeros(0, device=dev)
    out = ops.csr_spmm(X, rp, e_i, e_f, 1, 4)
    assert out.shape == (5, 16) and not out.any()
    out = ops.csr_split_spmm(X, torch.zeros(1, dtype=torch.int32, device=dev), e_i, e_f, e_i, 1, 4)
    assert out.shape == (5, 16) and not out.any()


@pytest.mark.parametrize("name", ["powerlaw", "rmat", "uniform16", "hub"])
def test_csr_sddmm_matches_oracle(dev, oracle, mats, name):
    from paramspmm_ae_b200 import ops
    m = mats[name]
    rp, ci, v = m.numpy()
    d = m.to(dev)
    rps, tr = ops.split_csr(m.rowPtr, 32)
    for dim in (4, 16, 47, 64, 100, 128, 200, 1100):
        A = dense(m.n_rows + 1, dim, 600 + dim)
        B = dense(m.n_cols, dim, 700 + dim)
        want = oracle.sddmm_csr(rp, ci, A.numpy(), B.numpy())
        got = ops.csr_sddmm(A.to(dev), B.to(dev), d.rowPtr, d.colIdx, d.val, min(4, (dim + 31) // 32), 4)
        assert got.shape == (m.nnz,)
        close(got, want)
        got = ops.csr_split_sddmm(A.to(dev), B.to(dev), rps.to(dev), d.colIdx, d.val, tr.to(dev),
                                  min(4, (dim + 31) // 32), 8)
        close(got, want)


@pytest.mark.parametrize("V", [2, 3])
def test_block_sddmm_matches_oracle(dev, oracle, mats, V):
    from paramspmm_ae_b200 import ops
    m = mats["powerlaw"]
    rp, ci, v = m.numpy()
    rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, m.n_cols, V)
    nbr = rpb.shape[0] - 1
    s_rpb, s_tr = ops.split_csr(rpb, 16)
    fn = ops.bcsr_sddmm if V == 2 else ops.vec_sddmm
    fn_split = ops.bcsr_split_sddmm if V == 2 else ops.vec_split_sddmm
    for dim in (16, 47, 64, 128):
        A = dense(nbr * V, dim, 800 + dim)
        B = dense(m.n_cols, dim, 900 + dim)
        want = oracle.sddmm_bcsr(rpb.numpy(), cb.numpy(), vb.numpy(), A.numpy(), B.numpy())
        got = fn(A.to(dev), B.to(dev), rpb.to(dev), cb.to(dev), vb.to(dev), min(4, (dim + 31) // 32), 4)
        assert got.shape == (cb.shape[0], V)
        close(got, want)
        got = fn_split(A.to(dev), B.to(dev), s_rpb.to(dev), cb.to(dev), vb.to(dev), s_tr.to(dev),
                       min(4, (dim + 31) // 32), 4)
        close(got, want)


@pytest.mark.parametrize("name", ["powerlaw", "rmat", "tiny", "hub"])
def test_genmask_bit_exact(dev, oracle, mats, name):
    from paramspmm_ae_b200 import ops
    m = mats[name]
    rp, ci, v = m.numpy()
    rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, m.n_cols, 2)
    want = oracle.genmask(rpb.numpy(), rp, vb.numpy(), m.nnz)
    got = ops.genmask(rpb.to(dev), m.rowPtr.to(dev), vb.to(dev), m.nnz)
    assert got.dtype == torch.int32 and got.shape == (m.nnz,)
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("gran", [1, 32, 96, 512])
def test_device_split_builder_bit_exact(dev, oracle, mats, gran):
    """The GPU partition builder against the host builder and the oracle."""
    from paramspmm_ae_b200 import ops, synth
    cases = [mats[k].rowPtr for k in ("powerlaw", "rmat", "hub", "tiny")]
    g = torch.Generator().manual_seed(gran)
    ln = torch.randint(0, 300, (5000,), generator=g)
    ln[torch.rand(5000, generator=g) < 0.3] = 0
    ln[::1024] = 40000                      # long rows right at tile starts
    cases.append(torch.cat([torch.zeros(1, dtype=torch.long), ln.cumsum(0)]).int())
    cases.append(torch.zeros(7, dtype=torch.int32))   # only empty rows
    cases.append(torch.zeros(1, dtype=torch.int32))   # no rows
    for rp in cases:
        want_rps, want_tr = oracle.split_csr(rp.numpy(), gran)
        h_rps, h_tr = ops.split_csr(rp, gran)
        rps, tr = ops.split_csr_device(rp.to(dev), gran)
        assert rps.dtype == torch.int32 and tr.dtype == torch.int32
        assert np.array_equal(rps.cpu().numpy(), want_rps) and np.array_equal(tr.cpu().numpy(), want_tr)
        assert torch.equal(rps.cpu(), h_rps) and torch.equal(tr.cpu(), h_tr)
    m = synth.rmat(20, 16_000_000, n=1_000_000, seed=23, device=dev)   # benchmark size
    rps, tr = ops.split_csr_device(m.rowPtr, 32)
    h_rps, h_tr = ops.split_csr(m.rowPtr.cpu(), 32)
    assert torch.equal(rps.cpu(), h_rps) and torch.equal(tr.cpu(), h_tr)


def test_device_split_builder_extreme_granularity_and_wrong_count(dev, mats):
    """A partition length near INT32_MAX (length + granularity overflows 32 bits) still gives the
    host builder's arrays, and a piece count that is not the partition's is flagged in
    rowPtr_split[0] (-1) without writing outside the arrays."""
    from paramspmm_ae_b200 import _lib, ops
    lib = _lib.lib()
    rp = mats["hub"].rowPtr
    big = 2**31 - 1
    h_rps, h_tr = ops.split_csr(rp, big)
    rps, tr = ops.split_csr_device(rp.to(dev), big)
    assert torch.equal(rps.cpu(), h_rps) and torch.equal(tr.cpu(), h_tr)
    assert int(rps[0]) == 0
    # wrong count: one piece fewer than the partition has
    n = rp.shape[0] - 1
    S = h_tr.shape[0] - 1
    need = ctypes.c_size_t(0)
    _lib.check(lib.pspmm_split_device_scratch_bytes(n, ctypes.byref(need)))
    scratch = torch.empty((need.value + 7) // 8, dtype=torch.int64, device=dev)
    out_rps = torch.full((S + 2,), -5, dtype=torch.int32, device=dev)
    out_tr = torch.full((S + 1,), -5, dtype=torch.int32, device=dev)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rp_d = rp.to(dev)
    _lib.check(lib.pspmm_split_csr_device(p(rp_d), n, big, p(out_rps), p(out_tr), S, p(scratch), need.value,
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    assert int(out_rps[0]) == -1                       # flagged
    assert int(out_rps[S + 1]) == -5 and int(out_tr[S]) == -5   # nothing past the caller's sizes


def test_profile_entry_points_return_gflops(dev, mats):
    """All twelve *_profile functions (SpMM/SpMM.cpp:482-889, SDDMM/sddmm.cpp:338-661): an integer
    GFLOP/s figure; the block forms take the CSR entry count before CF."""
    from paramspmm_ae_b200 import ops
    m = mats["powerlaw"]  # odd row count: the block forms pad
    d = m.to(dev)
    n, nnz = m.n_rows, m.nnz
    X = torch.ones(n, 64, device=dev)
    rps, tr = ops.split_csr(m.rowPtr, 32)
    rps, tr = rps.to(dev), tr.to(dev)
    got = [ops.csr_spmm_profile(X, d.rowPtr, d.colIdx, d.val, 2, 8),
           ops.csr_split_spmm_profile(X, rps, d.colIdx, d.val, tr, 2, 8),
           ops.csr_sddmm_profile(X, X, d.rowPtr, d.colIdx, d.val, 2, 8),
           ops.csr_split_sddmm_profile(X, X, rps, d.colIdx, d.val, tr, 2, 8)]
    for V, sp, sps, sd, sds in ((2, ops.bcsr_spmm_profile, ops.bcsr_split_spmm_profile, ops.bcsr_sddmm_profile,
                                 ops.bcsr_split_sddmm_profile),
                                (3, ops.vec_spmm_profile, ops.vec_split_spmm_profile, ops.vec_sddmm_profile,
                                 ops.vec_split_sddmm_profile)):
        rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, m.n_cols, V)
        b_rps, b_tr = ops.split_csr(rpb, 32)
        rpb, cb, vb, b_rps, b_tr = (t.to(dev) for t in (rpb, cb, vb, b_rps, b_tr))
        A = torch.ones((n + V - 1) // V * V, 64, device=dev)
        got += [sp(X, rpb, cb, vb, nnz, 2, 8), sps(X, b_rps, cb, vb, b_tr, nnz, 2, 8),
                sd(A, X, rpb, cb, vb, nnz, 2, 8), sds(A, X, b_rps, cb, vb, b_tr, nnz, 2, 8)]
    assert len(got) == 12 and all(isinstance(g, int) and g > 0 for g in got), got
    with pytest.raises(RuntimeError):
        ops.csr_spmm_profile(X, d.rowPtr, d.colIdx, d.val, 9, 8)      # CF outside 1..8
    with pytest.raises(RuntimeError):
        ops.csr_sddmm_profile(X, X, d.rowPtr, d.colIdx, d.val, 5, 8)  # CF outside 1..4


def test_spmm_output_rows_follow_the_dense_input(dev, oracle, mats):
    """The reference sizes the output from the dense input (zeros_like(input), padded to a multiple
    of the block height) and its own callers pass inputs with more rows than the matrix (features
    padded to an even row count): the extra output rows are zero, fewer rows than the matrix raise."""
    from paramspmm_ae_b200 import ops
    m = mats["powerlaw"]
    rp, ci, v = m.numpy()
    d = m.to(dev)
    n = m.n_rows
    X = dense(n + 1, 32, 5)
    want = oracle.spmm_csr(rp, ci, v, X[:n].numpy())
    Xd = X.to(dev)
    out = ops.csr_spmm(Xd, d.rowPtr, d.colIdx, d.val, 1, 8)
    assert out.shape == (n + 1, 32) and float(out[n].abs().max()) == 0.0
    close(out[:n], want)
    rps, tr = ops.split_csr(m.rowPtr, 32)
    out = ops.csr_split_spmm(Xd, rps.to(dev), d.colIdx, d.val, tr.to(dev), 1, 8)
    assert out.shape == (n + 1, 32) and float(out[n].abs().max()) == 0.0
    close(out[:n], want)
    rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, m.n_cols, 2)
    X3 = dense(n + 3, 32, 5)
    out = ops.bcsr_spmm(X3.to(dev), rpb.to(dev), cb.to(dev), vb.to(dev), 1, 8)
    assert out.shape == (n + 3, 32) and float(out[n:].abs().max()) == 0.0
    close(out[:n], oracle.spmm_csr(rp, ci, v, X3[:n].numpy()))
    with pytest.raises(RuntimeError):
        ops.csr_spmm(Xd[: n - 1].contiguous(), d.rowPtr, d.colIdx, d.val, 1, 8)


@pytest.mark.parametrize("fout", [24, 23, 1])
def test_spconv_forward_backward(dev, oracle, mats, fout):
    """GCN layer A(HW) and its gradients (SpCONV/SpCONV.h:43-72) against dense fp64 algebra; widths
    that are not a multiple of 4 travel padded through the products and come back cut."""
    from paramspmm_ae_b200 import ops
    m = mats["powerlaw"]  # symmetric: the backward pass multiplies by A, not A^T
    rp, ci, v = m.numpy()
    d = m.to(dev)
    n = m.n_rows
    H = dense(n, 40, 1)
    W = dense(40, fout, 2)
    G = dense(n, fout, 3)
    HW = (H.double() @ W.double()).float().numpy()
    want = oracle.spmm_csr(rp, ci, v, HW)
    got = ops.csr_spmm_forward(H.to(dev), W.to(dev), d.rowPtr, d.colIdx, d.val, 1, 4)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-4)
    AG = oracle.spmm_csr(rp, ci, v, G.numpy()).astype(np.float64)
    dH, dW = ops.csr_spmm_backward(G.to(dev), H.to(dev), W.to(dev), d.rowPtr, d.colIdx, d.val, 1, 4)
    assert dH.shape == (n, 40) and dW.shape == (40, fout) and dW.is_contiguous()
    np.testing.assert_allclose(dH.cpu().numpy(), AG @ W.double().numpy().T, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(dW.cpu().numpy(), H.double().numpy().T @ AG, rtol=1e-4, atol=2e-3)
    rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, n, 2)
    got = ops.bcsr_spmm_forward(H.to(dev), W.to(dev), rpb.to(dev), cb.to(dev), vb.to(dev), 1, 4)
    assert got.shape == (n, fout) and got.is_contiguous()  # sliced back from the padded row count
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-4)


def test_cusparse_comparators_agree(dev, oracle, mats):
    from paramspmm_ae_b200 import baselines
    m = mats["rmat"]
    rp, ci, v = m.numpy()
    d = m.to(dev)
    B = dense(m.n_cols, 64, 5)
    want = oracle.spmm_csr(rp, ci, v, B.numpy())
    close(baselines.cusparse_compute(B.to(dev), d.rowPtr, d.colIdx, d.val), want)
    close(baselines.cusparse_compute_csr_alg2(B.to(dev), d.rowPtr, d.colIdx, d.val), want)
    # COO (ALG4) and CSC forms, fed the way the reference's coo_spmm / csc_spmm objects feed them
    # (PCSR.py:45-124); the CSC arrays come from scipy, as there
    from scipy.sparse import csr_array
    rows = torch.repeat_interleave(torch.arange(m.n_rows, dtype=torch.int32), (m.rowPtr[1:] - m.rowPtr[:-1]).long())
    close(baselines.cusparse_compute_coo_alg4(B.to(dev), rows.to(dev), d.colIdx, d.val), want)
    csc = csr_array((v, ci, rp), shape=(m.n_rows, m.n_cols)).tocsc()
    t = lambda a, dt: torch.from_numpy(a.astype(dt)).to(dev)
    close(baselines.cusparse_compute_csc(B.to(dev), t(csc.indptr, "int32"), t(csc.indices, "int32"),
                                         t(csc.data, "float32")), want)
    assert baselines.cusparse_profile_coo_alg4(B.to(dev), rows.to(dev), d.colIdx, d.val) > 0
    assert baselines.cusparse_profile_csc(B.to(dev), t(csc.indptr, "int32"), t(csc.indices, "int32"),
                                          t(csc.data, "float32")) > 0
    close(baselines.gespmm_compute(B.to(dev), d.rowPtr, d.colIdx, d.val), want)
    for dim in (20, 100):  # the row-caching comparator on ragged widths
        B2 = dense(m.n_cols, dim, 8)
        close(baselines.gespmm_compute(B2.to(dev), d.rowPtr, d.colIdx, d.val), oracle.spmm_csr(rp, ci, v, B2.numpy()))
    A = dense(m.n_rows, 64, 6)
    vals = d.val.clone()
    baselines.cusparse_sddmm_compute(A.to(dev), B.to(dev), d.rowPtr, d.colIdx, vals)
    close(vals, oracle.sddmm_csr(rp, ci, A.numpy(), B.numpy()))


def test_full_size_properties(dev):
    """At benchmark size (10^6 rows, 1.6*10^7 entries) the oracle is too slow; check properties:
    A*ones equals the row sums of the values, the product is linear in B, split and plain
    layouts agree, and the result matches cuSPARSE through torch.sparse.mm on the device."""
    from paramspmm_ae_b200 import ops, synth
    n, dim = 1_000_000, 64
    m = synth.rmat(20, 16_000_000, n=n, seed=23, device=dev)
    assert m.nnz == 16_000_000
    ones = torch.ones(n, dim, device=dev)
    got = ops.csr_spmm(ones, m.rowPtr, m.colIdx, m.val, 2, 8)
    rows = torch.repeat_interleave(torch.arange(n, device=dev), (m.rowPtr[1:] - m.rowPtr[:-1]).long())
    rowsum = torch.zeros(n, device=dev, dtype=torch.float64).index_add_(0, rows, m.val.double())
    torch.testing.assert_close(got[:, 0].double(), rowsum, rtol=1e-5, atol=1e-4)
    torch.testing.assert_close(got[:, dim - 1], got[:, 0], rtol=0, atol=0)
    B1 = synth.dense_uniform(n, dim, 1, dev)
    B2 = synth.dense_uniform(n, dim, 2, dev)
    c1 = ops.csr_spmm(B1, m.rowPtr, m.colIdx, m.val, 2, 8)
    c2 = ops.csr_spmm(B2, m.rowPtr, m.colIdx, m.val, 2, 8)
    c12 = ops.csr_spmm(B1 + B2, m.rowPtr, m.colIdx, m.val, 2, 8)
    # hub rows sum tens of thousands of terms: scale the absolute floor by the row's magnitude
    scale = 1 + rowsum.max().item()
    torch.testing.assert_close(c12, c1 + c2, rtol=1e-5, atol=1e-6 * scale * 50)
    rps, tr = ops.split_csr(m.rowPtr.cpu(), 32)
    cs = ops.csr_split_spmm(B1, rps.to(dev), m.colIdx, m.val, tr.to(dev), 2, 8)
    torch.testing.assert_close(cs, c1, rtol=1e-5, atol=1e-6 * scale * 50)
    s = torch.sparse_csr_tensor(m.rowPtr, m.colIdx, m.val, size=(n, n))
    torch.testing.assert_close(torch.sparse.mm(s, B1), c1, rtol=1e-5, atol=1e-6 * scale * 50)


def test_spmm_column_tiles(dev, oracle, mats):
    """col_tile runs a wide product as several launches over column ranges: same result, plain and
    split layouts, widths that are and are not multiples of the tile, strided output."""
    from paramspmm_ae_b200 import _lib, ops
    m = mats["rmat"]
    rp, ci, v = m.numpy()
    d = m.to(dev)
    rps, tr = ops.split_csr(m.rowPtr, 32)
    rps, tr = rps.to(dev), tr.to(dev)
    for dim in (132, 144, 256, 260):
        B = dense(m.n_cols, dim, 600 + dim)
        want = oracle.spmm_csr(rp, ci, v, B.numpy())
        Bd = B.to(dev)
        for tile, lanes in ((128, 32), (64, 0), (4, 0)):
            cfg = _lib.make_cfg(lanes_per_row=lanes, col_tile=tile, rows_per_group=4, gather_batch=8)
            out = torch.full((m.n_rows, dim + 8), float("nan"), device=dev)[:, :dim]
            ops.spmm_into(out, Bd, d.rowPtr, d.colIdx, d.val, cfg=cfg)
            close(out, want)
            out = torch.full((m.n_rows, dim), float("nan"), device=dev)
            ops.spmm_into(out, Bd, rps, d.colIdx, d.val, target_row=tr, n_out_rows=m.n_rows, cfg=cfg)
            close(out, want)
    with pytest.raises(_lib.PspmmError):
        ops.spmm_into(torch.empty(m.n_rows, 132, device=dev), dense(m.n_cols, 132, 1).to(dev), d.rowPtr, d.colIdx,
                      d.val, cfg=_lib.make_cfg(col_tile=6))


# ----------------------------------------------------------------------------- fused AGNN aggregation
@pytest.mark.parametrize("dim", [4, 16, 32, 48, 64, 100, 128, 256])
@pytest.mark.parametrize("softmax", [True, False])
def test_agnn_fused_matches_the_oracle(dev, oracle, mats, dim, softmax):
    """SDDMM -> scale -> (edge softmax) -> SpMM in one kernel, plain CSR and split layouts, against
    the float64 row-by-row restatement."""
    from paramspmm_ae_b200 import ops
    for name in ("powerlaw", "rmat", "hub", "tiny"):
        m = mats[name]
        rp, ci, _ = m.numpy()
        X = torch.nn.functional.normalize(dense(m.n_rows, dim, 900 + dim), dim=1)
        beta = 1.7
        want = oracle.agnn_aggregate(rp, ci, X.numpy(), X.numpy(), beta, softmax)
        d, Xd = m.to(dev), X.to(dev)
        for vw in (0, 4, 8):
            for lanes, batch in ((0, 0), (4, 4), (8, 4), (8, 8), (16, 8), (16, 16), (32, 8), (32, 16)):
                got = ops.agnn_fused(Xd, Xd, d.rowPtr, d.colIdx, beta, softmax, batch=batch, lanes_per_row=lanes,
                                     vec_width=vw)
                close(got, want)
        for gran in (3, 32):
            rps, tr = ops.split_csr(m.rowPtr, gran)
            got = torch.full((m.n_rows, dim), float("nan"), device=dev)
            ops.agnn_fused(Xd, Xd, rps.to(dev), d.colIdx, beta, softmax, target_row=tr.to(dev),
                           n_out_rows=m.n_rows, out=got)
            close(got, want)


@pytest.mark.parametrize("dim", [4, 32, 64, 100, 128, 256])
@pytest.mark.parametrize("softmax", [False, True])
def test_agnn_fused_with_separate_aggregation_operand(dev, oracle, mats, dim, softmax):
    """out_i = sum_j a_ij V_j with the scores from A and B (pspmm_agnn_fused_apply_csr): a full
    matrix V, and one row shared by all columns (the row sums of the scores); plain and split."""
    from paramspmm_ae_b200 import ops
    for name in ("powerlaw", "rmat", "hub"):
        m = mats[name]
        rp, ci, _ = m.numpy()
        A = torch.nn.functional.normalize(dense(m.n_rows, dim, 910 + dim), dim=1)
        B = torch.nn.functional.normalize(dense(m.n_cols, dim, 920 + dim), dim=1)
        V = dense(m.n_cols, dim, 930 + dim)
        ones = torch.ones(1, dim)
        d = m.to(dev)
        for Vm in (V, ones):
            want = oracle.agnn_aggregate(rp, ci, A.numpy(), B.numpy(), 0.7, softmax, V=Vm.numpy())
            for lanes in (0, 8, 32):
                got = ops.agnn_fused(A.to(dev), B.to(dev), d.rowPtr, d.colIdx, 0.7, softmax, V=Vm.to(dev),
                                     lanes_per_row=lanes if lanes * 16 >= dim or lanes == 0 else 0)
                close(got, want)
            rps, tr = ops.split_csr(m.rowPtr, 32)
            got = ops.agnn_fused(A.to(dev), B.to(dev), rps.to(dev), d.colIdx, 0.7, softmax, target_row=tr.to(dev),
                                 n_out_rows=m.n_rows, V=Vm.to(dev))
            close(got, want)
    with pytest.raises(RuntimeError):
        ops.agnn_fused(A.to(dev), B.to(dev), d.rowPtr, d.colIdx, V=torch.ones(2, dim, device=dev))


def test_agnn_fused_equals_the_unfused_composition(dev, mats):
    """With softmax off and A == B the fused kernel is the reference's AGNN forward:
    csr_sddmm -> * beta -> csr_spmm."""
    from paramspmm_ae_b200 import ops
    m = mats["powerlaw"]
    d = m.to(dev)
    X = torch.nn.functional.normalize(dense(m.n_rows, 64, 77), dim=1).to(dev)
    beta = 0.8
    e = ops.csr_sddmm(X, X, d.rowPtr, d.colIdx, d.val, 2, 8) * beta
    want = ops.csr_spmm(X, d.rowPtr, d.colIdx, e, 2, 8)
    got = ops.agnn_fused(X, X, d.rowPtr, d.colIdx, beta, softmax=False)
    close(got, want.cpu().numpy())


def test_agnn_fused_rejects_what_it_cannot_run(dev):
    from paramspmm_ae_b200 import _lib, ops
    rp = torch.tensor([0, 1, 2], dtype=torch.int32, device=dev)
    ci = torch.tensor([0, 1], dtype=torch.int32, device=dev)
    X = torch.ones(2, 6, device=dev)  # dim not a multiple of 4
    with pytest.raises(_lib.PspmmError):
        ops.agnn_fused(X, X, rp, ci)
    with pytest.raises(RuntimeError):
        ops.agnn_fused(X.cpu(), X.cpu(), rp, ci)


# ----------------------------------------------------------------------------- row pull (exchange step)
@pytest.mark.parametrize("dim", [4, 64, 128, 132, 260])
def test_pull_rows_copies_the_listed_rows(dev, dim):
    """pspmm_pull_rows with several source blocks (all on this GPU here; on a node they are the
    peers' mapped blocks): every listed row lands at its list position, for every rotation and CTA
    budget, strided sources and destination included; bit-exact (a copy)."""
    from paramspmm_ae_b200 import _lib, ops
    g = torch.Generator().manual_seed(dim)
    sizes = [700, 1, 0, 1300, 64]
    wide = [torch.rand(s, dim + 4, generator=g).to(dev) for s in sizes]
    blocks = [w[:, :dim] for w in wide]           # row stride dim + 4
    counts = [333, 1, 0, 1300, 7]
    rows, first = [], [0]
    for s, c in zip(sizes, counts):
        rows.append(torch.sort(torch.randperm(s, generator=g)[:c]).values if c else torch.empty(0, dtype=torch.long))
        first.append(first[-1] + c)
    rows_d = torch.cat(rows).int().to(dev)
    want = torch.cat([b[r.to(dev)] for b, r in zip(blocks, rows)])
    n = first[-1]
    for bulk in (False, True):  # load/store kernel, and bulk asynchronous copies through shared memory
        for rotate, ctas in ((0, 0), (5, 1), (first[3], 3), (n - 1, 1000)):
            dst = torch.full((n, dim + 8), float("nan"), device=dev)[:, :dim]
            ops.pull_rows(dst, blocks, first, rows_d, rotate=rotate, ctas=ctas, bulk=bulk)
            assert torch.equal(dst, want)
    assert ops.pull_rows_status() == 0  # no bounded wait ran out
    # nothing to copy, and the argument checks
    ops.pull_rows(torch.empty(0, dim, device=dev), blocks[:1], [0, 0], torch.empty(0, dtype=torch.int32, device=dev))
    with pytest.raises(RuntimeError):
        ops.pull_rows(torch.empty(n, dim, device=dev), blocks, first[:-1], rows_d)
    with pytest.raises(_lib.PspmmError):
        ops.pull_rows(torch.empty(n, dim, device=dev), blocks, first, rows_d, rotate=n)


@pytest.mark.parametrize("exchange,row_chunks", [("needed", 1), ("needed_pipelined", 3), ("needed_rowgroups", 3),
                                                 ("needed_rowgroups", 7)])
@pytest.mark.parametrize("bulk", [0, 1, 2])
def test_pull_transport_single_rank(dev, oracle, mats, exchange, row_chunks, bulk):
    """The pull transport with one rank (the owner's block is this GPU's own buffer): same product
    as the plain kernel, twice in a row (buffers, streams and events are reused); with the
    load/store fetch kernel, and with the bulk-copy one for the later or for all fetches."""
    from paramspmm_ae_b200.shard import ShardedSpMM
    m = mats["rmat"]
    rp, ci, v = m.numpy()
    d = m.to(dev)
    B = dense(m.n_cols, 64, 31)
    want = oracle.spmm_csr(rp, ci, v, B.numpy())
    op = ShardedSpMM(d.rowPtr, d.colIdx, d.val, m.n_cols, 0, 1, device=dev, exchange=exchange, transport="pull",
                     row_chunks=row_chunks)
    op.pull_bulk = bulk
    Bd = B.to(dev)
    for _ in range(2):
        out = op.forward(Bd, torch.full((m.n_rows, 64), float("nan"), device=dev))
        torch.cuda.synchronize()
        close(out, want)
    src = op.symmetric_input(64)   # a producer writes the block in place: no staging copy
    src.copy_(Bd)
    close(op.forward(src), want)
    from paramspmm_ae_b200 import ops
    assert ops.pull_rows_status() == 0
    # a traced call: same result, and one [begin, end] pair per fetch and per product, in order
    op.trace = True
    close(op.forward(src), want)
    op.trace = False
    t = op.trace_result()
    assert len(t["fetch_ms"]) == len(op.chunk_plan) and len(t["product_ms"]) >= 1
    assert all(0.0 <= a <= b <= t["end_ms"] for a, b in t["fetch_ms"] + t["product_ms"])


# ----------------------------------------------------------------------------- length-bucketed plan
@pytest.mark.parametrize("name", ["powerlaw", "rmat", "hub", "uniform16", "tiny"])
@pytest.mark.parametrize("gran", [1, 7, 32, 512])
def test_bucketed_plan_spmm_matches_oracle(dev, oracle, mats, name, gran):
    """pspmm_cfg.bucketed: the pieces of split_csr ordered by length, entries permuted, flags in the
    high bits of target_row; every kernel shape, overwrite and accumulate, CSR and 2 x 1 blocks."""
    from paramspmm_ae_b200 import _lib, ops
    m = mats[name]
    rp, ci, v = m.numpy()
    d = m.to(dev)
    seg, ci_p, v_p, tg = ops.bucket_pcsr(d.rowPtr, d.colIdx, d.val, gran)
    assert seg.dtype == torch.int32 and tg.dtype == torch.int32 and int(seg[-1]) == m.nnz
    ln = (seg[1:] - seg[:-1])
    assert bool((ln[:-1] >= ln[1:]).all()) and int(ln.max()) <= gran
    rows = (tg.long() & ops.SEG_ROW_MASK)
    assert int(torch.bincount(rows, minlength=m.n_rows).min()) >= 1  # every row appears, empty ones too
    for dim in (4, 16, 47, 64, 128, 256):
        B = dense(m.n_cols, dim, 200 + dim)
        want = oracle.spmm_csr(rp, ci, v, B.numpy())
        for lanes, rpg, thr in ((0, 0, 0), (4, 2, 64), (32, 8, 128), (16, 1, 256)):
            cfg = _lib.make_cfg(bucketed=1, lanes_per_row=lanes, rows_per_group=rpg, cta_threads=thr)
            out = torch.full((m.n_rows, dim), float("nan"), device=dev)
            ops.spmm_into(out, B.to(dev), seg, ci_p, v_p, target_row=tg, n_out_rows=m.n_rows, cfg=cfg)
            close(out, want)
        if dim % 4 == 0:
            acc = torch.ones(m.n_rows, dim, device=dev)
            ops.spmm_into(acc, B.to(dev), seg, ci_p, v_p, target_row=tg, n_out_rows=m.n_rows,
                          cfg=_lib.make_cfg(bucketed=1, accumulate=1))
            close(acc, want + 1.0)
    # 2 x 1 blocks through the same plan builder
    rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, m.n_cols, 2)
    seg, cb_p, vb_p, tg = ops.bucket_pcsr(rpb.to(dev), cb.to(dev), vb.to(dev), gran)
    B = dense(m.n_cols, 64, 9)
    nbr = rpb.shape[0] - 1
    out = torch.full((nbr * 2, 64), float("nan"), device=dev)
    ops.spmm_into(out, B.to(dev), seg, cb_p, vb_p, target_row=tg, V=2, n_out_rows=nbr, cfg=_lib.make_cfg(bucketed=1))
    close(out[: m.n_rows], oracle.spmm_csr(rp, ci, v, B.numpy()))


def test_spmm_without_values_multiplies_by_the_pattern(dev, oracle, mats):
    """val = NULL: every stored entry counts as 1 (plain, split and bucketed layouts)."""
    from paramspmm_ae_b200 import _lib, ops
    m = mats["powerlaw"]
    rp, ci, v = m.numpy()
    d = m.to(dev)
    for dim in (16, 64, 100):
        B = dense(m.n_cols, dim, 60 + dim)
        want = oracle.spmm_csr(rp, ci, np.ones_like(v), B.numpy())
        out = torch.full((m.n_rows, dim), float("nan"), device=dev)
        close(ops.spmm_into(out, B.to(dev), d.rowPtr, d.colIdx, None), want)
        rps, tr = ops.split_csr_device(d.rowPtr, 32)
        out.fill_(float("nan"))
        close(ops.spmm_into(out, B.to(dev), rps, d.colIdx, None, target_row=tr, n_out_rows=m.n_rows), want)
    with pytest.raises(RuntimeError):
        rpb, cb, vb = ops.bcsr_from_csr(m.rowPtr, m.colIdx, m.val, m.n_cols, 2)
        ops._spmm_inputs(B.to(dev), rpb.to(dev), cb.to(dev), None, None, 2)


def test_planned_spmm_runs_every_layout(dev, oracle, mats):
    """decider.PlannedSpMM: plain, split and bucketed plans give the same product."""
    from paramspmm_ae_b200 import decider
    m = mats["powerlaw"]
    rp, ci, v = m.numpy()
    d = m.to(dev)
    B = dense(m.n_cols, 64, 12)
    want = oracle.spmm_csr(rp, ci, v, B.numpy())
    for kw in (dict(if_split=0), dict(if_split=1, granularity=32), dict(if_split=1, granularity=32, bucketed=1)):
        plan = decider.Plan(vec_size=1, lanes_per_row=0, vec_width=0, cta_threads=0, rows_per_group=0,
                            gather_batch=0, col_tile=0, bucketed=0, granularity=None)
        plan.update(kw)
        op = decider.PlannedSpMM(plan, d.rowPtr, d.colIdx, d.val)
        out = torch.full((m.n_rows, 64), float("nan"), device=dev)
        op(out, B.to(dev))
        close(out, want)
        op(out, B.to(dev), accumulate=True)
        close(out, 2 * want)


def test_relabel_symmetric_on_the_device_equals_the_host(dev, mats):
    """shard.relabel_symmetric runs where its arrays are: the device result equals the host result
    bit for bit (the sort keys are distinct), and the relabelled product is the original one with
    its rows permuted."""
    from paramspmm_ae_b200 import ops, shard
    m = mats["rmat"]
    new_of_old = shard.scattered_labels(m.n_rows, seed=11)
    host = shard.relabel_symmetric(m.rowPtr, m.colIdx, m.val, new_of_old)
    d = m.to(dev)
    got = shard.relabel_symmetric(d.rowPtr, d.colIdx, d.val, new_of_old)
    for a, b in zip(host, got):
        assert b.is_cuda and torch.equal(a, b.cpu())
    B = dense(m.n_cols, 32, 5).to(dev)
    old_of_new = torch.argsort(new_of_old).to(dev)
    want = ops.csr_spmm(B, d.rowPtr, d.colIdx, d.val, 1, 4)[old_of_new]
    out = ops.csr_spmm(B[old_of_new].contiguous(), got[0], got[1], got[2], 1, 4)
    torch.testing.assert_close(out, want, rtol=1e-5, atol=1e-4)
