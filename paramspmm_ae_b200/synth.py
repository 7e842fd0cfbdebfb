"""Seeded synthetic sparse matrices and dense operands.

The reference evaluates on public graph collections that are not available
offline; these generators produce matrices with the same shapes, densities and
degree distributions from a seed.  Everything is built with torch ops, so the
same code runs on the CPU (small test cases) and on a CUDA device (full-size
benchmark inputs).  A given (seed, device type) pair always yields the same
matrix; CPU and CUDA streams of random numbers differ, so the two device types
give different (equally distributed) matrices.

Index arrays are int32, values fp32, columns sorted and distinct within a row
(the layout ``graph_input.py:21-23`` of the reference hands to its kernels).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class CSR:
    rowPtr: torch.Tensor  # int32 [n_rows + 1]
    colIdx: torch.Tensor  # int32 [nnz]
    val: torch.Tensor  # float32 [nnz]
    n_rows: int
    n_cols: int

    @property
    def nnz(self) -> int:
        return int(self.colIdx.shape[0])

    def to(self, device):
        return CSR(self.rowPtr.to(device), self.colIdx.to(device), self.val.to(device),
                   self.n_rows, self.n_cols)

    def numpy(self):
        return (self.rowPtr.cpu().numpy(), self.colIdx.cpu().numpy(), self.val.cpu().numpy())


def _gen(seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def _csr_from_sorted_keys(keys, n_rows, n_cols, val):
    rows = torch.div(keys, n_cols, rounding_mode="floor")
    cols = keys - rows * n_cols
    counts = torch.bincount(rows, minlength=n_rows)
    rowPtr = torch.zeros(n_rows + 1, dtype=torch.int64, device=keys.device)
    rowPtr[1:] = torch.cumsum(counts, 0)
    return CSR(rowPtr.to(torch.int32), cols.to(torch.int32), val, n_rows, n_cols)


def dense_uniform(n, dim, seed, device="cpu"):
    """Dense operand 2*U[0,1) - 1, fp32."""
    return torch.rand(n, dim, generator=_gen(seed, device), device=device, dtype=torch.float32) * 2 - 1


def dense_normal(n, dim, seed, device="cpu"):
    return torch.randn(n, dim, generator=_gen(seed, device), device=device, dtype=torch.float32)


def uniform_rows(n, k=16, seed=21, device="cpu", n_cols=None):
    """Exactly k distinct uniformly random columns in every row; values U[0,1)."""
    n_cols = n if n_cols is None else n_cols
    if k > n_cols:
        raise ValueError("k exceeds the number of columns")
    g = _gen(seed, device)
    cols = torch.randint(0, n_cols, (n, k), generator=g, device=device, dtype=torch.int64)
    cols, _ = torch.sort(cols, dim=1)
    for _ in range(1000):
        bad = (cols[:, 1:] == cols[:, :-1]).any(dim=1)
        nb = int(bad.sum())
        if nb == 0:
            break
        fresh = torch.randint(0, n_cols, (nb, k), generator=g, device=device, dtype=torch.int64)
        cols[bad], _ = torch.sort(fresh, dim=1)
    else:
        raise RuntimeError("could not draw distinct columns")
    val = torch.rand(n * k, generator=g, device=device, dtype=torch.float32)
    rowPtr = torch.arange(0, n * k + 1, k, device=device, dtype=torch.int64).to(torch.int32)
    return CSR(rowPtr, cols.reshape(-1).to(torch.int32), val, n, n_cols)


def banded_rows(n, k=16, half_bw=32, seed=22, device="cpu", chunk=1 << 18):
    """Exactly k distinct columns per row, uniform in [i-half_bw, i+half_bw] clipped to the matrix."""
    if n < half_bw + 1 or k > half_bw + 1:
        raise ValueError("matrix too small for the requested band")
    g = _gen(seed, device)
    width = 2 * half_bw + 1
    offs = torch.arange(-half_bw, half_bw + 1, device=device, dtype=torch.int64)
    out = torch.empty((n, k), dtype=torch.int64, device=device)
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        rows = torch.arange(lo, hi, device=device, dtype=torch.int64)
        cand = rows[:, None] + offs[None, :]
        keys = torch.rand(hi - lo, width, generator=g, device=device)
        keys[(cand < 0) | (cand >= n)] = 2.0
        pick = torch.argsort(keys, dim=1)[:, :k]
        out[lo:hi], _ = torch.sort(torch.gather(cand, 1, pick), dim=1)
    val = torch.rand(n * k, generator=g, device=device, dtype=torch.float32)
    rowPtr = torch.arange(0, n * k + 1, k, device=device, dtype=torch.int64).to(torch.int32)
    return CSR(rowPtr, out.reshape(-1).to(torch.int32), val, n, n)


def _trim_to(keys, target, g):
    """Keep exactly `target` of the sorted distinct keys, dropping a seeded random subset."""
    extra = keys.shape[0] - target
    if extra <= 0:
        return keys
    score = torch.rand(keys.shape[0], generator=g, device=keys.device)
    drop = torch.topk(score, extra).indices
    keep = torch.ones(keys.shape[0], dtype=torch.bool, device=keys.device)
    keep[drop] = False
    return keys[keep]


def rmat(scale, nnz, n=None, a=0.57, b=0.19, c=0.19, seed=23, device="cpu", batch=1 << 26):
    """R-MAT matrix with exactly `nnz` distinct entries; values U[0,1).

    Endpoints at or beyond `n` (when n < 2**scale) are discarded, duplicates are merged,
    and edges are generated until `nnz` distinct ones exist.
    """
    n = (1 << scale) if n is None else n
    g = _gen(seed, device)
    keys = torch.empty(0, dtype=torch.int64, device=device)
    ab, abc = a + b, a + b + c
    for _ in range(200):
        need = nnz - keys.shape[0]
        if need <= 0:
            break
        m = min(batch, int(need * 1.15) + 4096)
        r = torch.zeros(m, dtype=torch.int64, device=device)
        col = torch.zeros(m, dtype=torch.int64, device=device)
        for _bit in range(scale):
            u = torch.rand(m, generator=g, device=device)
            r = (r << 1) | (u >= ab).to(torch.int64)
            col = (col << 1) | (((u >= a) & (u < ab)) | (u >= abc)).to(torch.int64)
        ok = (r < n) & (col < n)
        keys = torch.unique(torch.cat([keys, r[ok] * n + col[ok]]))
    else:
        raise RuntimeError("R-MAT generation did not reach the requested nnz")
    keys = _trim_to(keys, nnz, g)
    val = torch.rand(keys.shape[0], generator=g, device=device, dtype=torch.float32)
    return _csr_from_sorted_keys(keys, n, n, val)


def powerlaw_graph(n, n_pairs, gamma=2.1, seed=1, device="cpu", self_loops=True, normalize=True,
                   batch=1 << 26):
    """Symmetric Chung-Lu style graph: `n_pairs` distinct undirected pairs, power-law degrees.

    Endpoint i is drawn with probability proportional to (i+10)**(-1/(gamma-1)).  The
    adjacency is symmetrised, optionally given self-loops, and optionally carries the GCN
    weights D^-1/2 (A+I) D^-1/2 computed in fp64 and cast to fp32 (what
    ``graph_input.py:366-379`` of the reference computes); otherwise all values are 1.
    """
    g = _gen(seed, device)
    w = (torch.arange(n, device=device, dtype=torch.float64) + 10.0) ** (-1.0 / (gamma - 1.0))
    cdf = torch.cumsum(w, 0)
    cdf = cdf / cdf[-1]
    pairs = torch.empty(0, dtype=torch.int64, device=device)
    for _ in range(400):
        need = n_pairs - pairs.shape[0]
        if need <= 0:
            break
        m = min(batch, int(need * 1.2) + 4096)
        u = torch.rand(2, m, generator=g, device=device, dtype=torch.float64)
        e = torch.searchsorted(cdf, u).clamp_(max=n - 1)
        lo, hi = torch.minimum(e[0], e[1]), torch.maximum(e[0], e[1])
        ok = lo != hi
        pairs = torch.unique(torch.cat([pairs, lo[ok] * n + hi[ok]]))
    else:
        raise RuntimeError("graph generation did not reach the requested number of pairs")
    pairs = _trim_to(pairs, n_pairs, g)
    lo = torch.div(pairs, n, rounding_mode="floor")
    hi = pairs - lo * n
    parts = [lo * n + hi, hi * n + lo]
    if self_loops:
        d = torch.arange(n, device=device, dtype=torch.int64)
        parts.append(d * n + d)
    keys, _ = torch.sort(torch.cat(parts))
    out = _csr_from_sorted_keys(keys, n, n, None)
    if normalize:
        deg = (out.rowPtr[1:] - out.rowPtr[:-1]).to(torch.float64)
        dis = deg.pow(-0.5)
        dis[torch.isinf(dis)] = 0.0
        rows = torch.div(keys, n, rounding_mode="floor")
        out.val = (dis[rows] * dis[out.colIdx.long()]).to(torch.float32)
    else:
        out.val = torch.ones(keys.shape[0], dtype=torch.float32, device=device)
    return out


def with_empty_rows(m: CSR, every=7):
    """Copy of `m` where every `every`-th row has been emptied (edge-case input for tests)."""
    rp = m.rowPtr.long()
    ln = rp[1:] - rp[:-1]
    rows = torch.repeat_interleave(torch.arange(m.n_rows, device=rp.device), ln)
    keep = (rows % every) != 0
    ln2 = ln.clone()
    ln2[::every] = 0
    rp2 = torch.zeros_like(rp)
    rp2[1:] = torch.cumsum(ln2, 0)
    return CSR(rp2.to(torch.int32), m.colIdx[keep], m.val[keep], m.n_rows, m.n_cols)
