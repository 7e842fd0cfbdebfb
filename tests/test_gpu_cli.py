"""The decider's command line on a generated MatrixMarket file (needs a GPU: it runs and checks
the kernels it times)."""
import json

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_decider_command_line(tmp_path):
    assert torch.cuda.is_available()
    sp = pytest.importorskip("scipy.sparse")
    from scipy.io import mmwrite

    from paramspmm_ae_b200 import decider

    rng = np.random.default_rng(4)
    n = 4000
    deg = np.minimum(n - 1, (rng.pareto(1.2, n) * 3 + 1).astype(np.int64))  # skewed row lengths, a few hubs
    rows = np.repeat(np.arange(n), deg)
    cols = rng.integers(0, n, rows.size)
    A = sp.coo_matrix((np.ones(rows.size), (rows, cols)), shape=(n, n))
    A.sum_duplicates()
    mmwrite(str(tmp_path / "skewed.mtx"), A)
    mmwrite(str(tmp_path / "even.mtx"), sp.random(n, n, density=8 / n, random_state=1, format="coo"))
    out = tmp_path / "out.jsonl"
    recs = decider.main(["--path", str(tmp_path), "--dim_list", "16", "64", "100", "--json", str(out),
                         "--cache_dir", str(tmp_path / "cache")])
    assert [r["mtx"] for r in recs] == ["even"] * 3 + ["skewed"] * 3  # every product passed the comparison
    assert all(r["gflops"] > 0 and r["cusparse_gflops"] > 0 and r["gespmm_gflops"] > 0 for r in recs)
    assert all(r["regime"].endswith("skewed") for r in recs if r["mtx"] == "skewed")
    assert all(r["regime"].endswith("even") for r in recs if r["mtx"] == "even")
    lines = [json.loads(x) for x in out.read_text().splitlines()]
    assert lines == json.loads(json.dumps(recs))
    assert len(list((tmp_path / "cache").iterdir())) == 2
    # second run reads the containers and takes one named matrix
    again = decider.main(["--path", str(tmp_path) + "/", "--mtx_name", "even", "--dim_list", "32", "--no_baselines",
                          "--cache_dir", str(tmp_path / "cache")])
    assert len(again) == 1 and "cusparse_gflops" not in again[0]
