"""CPU test: the reference's own graph_input.py, imported unmodified from the mounted reference
tree, runs on top of the drop-in extension modules (its host path calls ParamSpMM.split_csr_par),
and this package's builder produces the same arrays bit for bit.  Skipped when the reference
tree is not mounted."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import build_oracle

pytestmark = pytest.mark.skipif(not build_oracle.ref_available(), reason="reference tree not mounted")


@pytest.fixture(scope="module")
def ref_graph_input(pspmm_lib):
    import paramspmm_ae_b200
    paramspmm_ae_b200.install_dropin()
    sys.path.insert(0, build_oracle.REF_ROOT)
    try:
        import graph_input as ref_gi  # the reference's module
    finally:
        sys.path.remove(build_oracle.REF_ROOT)
    assert os.path.realpath(ref_gi.__file__).startswith(os.path.realpath(build_oracle.REF_ROOT))
    return ref_gi


@pytest.mark.parametrize("sub,name", [("", "pubmed"), ("rabbit/", "pubmed_rabbit")])
@pytest.mark.parametrize("normalize", [False, True])
def test_reference_loader_on_dropin_matches_native_builder(ref_graph_input, sub, name, normalize, capsys):
    from paramspmm_ae_b200 import graph_input as gi
    path = os.path.join(build_oracle.REF_ROOT, "toy_dataset", sub)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        g_ref = ref_graph_input.graph_input(mtx_name=name, path=path)
        g_ref.load(load_from_mtx=True, is_normalize=normalize)
        g = gi.graph_input(mtx_name=name, path=path)
        g.load(load_from_mtx=True, is_normalize=normalize)
    capsys.readouterr()
    for part in ("csr_data", "bcsr_data"):
        a, b = getattr(g_ref, part), getattr(g, part)
        for arr in ("rowPtr", "colIdx", "val", "rowPtr_split", "target_row"):
            x, y = getattr(a, arr), getattr(b, arr)
            assert x.dtype == y.dtype and x.shape == y.shape, (part, arr)
            assert torch.equal(x, y), (part, arr)
        assert a.split_granularity == b.split_granularity
        assert abs(float(a.split_ratio) - float(b.split_ratio)) < 1e-6
    assert g_ref.pack_rate == g.pack_rate
    np.testing.assert_allclose(g_ref.get_info(), g.get_info(), rtol=1e-6)
    if not normalize:
        assert g.mtx_nodes == 19717 and g.mtx_edges == 88651
        assert g.csr_data.target_row.shape[0] == 20005
