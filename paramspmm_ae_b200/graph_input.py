"""PCSR builder: host-side mirror of the reference's ``graph_input.py``.

Keeps the class and attribute names (``csr_data``, ``graph_input``, ``.rowPtr/.colIdx/.val``,
``.rowPtr_split/.target_row``, ``.split_granularity/.split_ratio``, ``.bcsr_data``, ``.mask``,
``.pack_rate``, ``get_info()``) so code written against the reference keeps working, but the
work is done by libpspmm's native builders:

* the row split is ``pspmm_split_csr`` with 64-bit integer piece offsets (the reference
  derives them from an fp32 cumulative sum, graph_input.py:49,135, exact only below 2**24
  pieces);
* the 2 x 1 block layout is ``pspmm_bcsr_count/fill`` (parallel over block rows) instead of
  scipy's single-threaded ``tobsr`` (graph_input.py:245-266); the arrays are bit-identical;
* ``mask`` is ``pspmm_genmask`` on the device (graph_input.py:277-286).

* a MatrixMarket file is parsed by ``pspmm_mtx_read_csr`` (parallel, memory-mapped) instead of
  scipy's ``mmread`` + ``tocsr`` (graph_input.py:226-232) and can be kept as a binary CSR container
  (``cache_dir``) so that later runs skip the parse.

A matrix can come from a MatrixMarket file (``load``, as in the reference) or from CSR arrays
already in memory (``load_csr``).
"""
from __future__ import annotations

import math
import os

import numpy as np
import torch

from . import ops


class csr_data(object):
    """CSR or block-CSR arrays as CPU torch tensors plus the statistics the decider reads
    (graph_input.py:17-177 of the reference)."""

    def __init__(self, rowPtr, colIdx, val, num_nodes, num_edges, csr_flag=True):
        self.csr_flag = csr_flag
        self.rowPtr = torch.as_tensor(rowPtr).to(torch.int32).contiguous()
        self.colIdx = torch.as_tensor(colIdx).to(torch.int32).contiguous()
        self.val = torch.as_tensor(val).to(torch.float32).contiguous()
        self.num_nodes = num_nodes
        self.num_edges = num_edges
        self.row_nnz = None
        self.max_row_nnz = self.real_nrow = self.nonempty_rate = None
        self.avg_degree = self.COV = self.real_avg_degree = self.real_COV = None
        self.max_bw = self.avg_bw = None
        self.split_granularity = self.split_ratio = self.row_split_nnz = None
        self.rowPtr_split = self.target_row = None

    # -- statistics ---------------------------------------------------------------------
    def split_ratio_comp(self, split_granularity):
        """Pieces per row for a partition length and pieces / non-empty rows
        (graph_input.py:48-51); integer arithmetic."""
        pieces = torch.div(self.row_nnz.long() + (split_granularity - 1), split_granularity,
                           rounding_mode="floor")
        return int(pieces.sum()) / self.real_nrow, pieces

    def _pick_granularity(self, manual_granularity, is_avg_granularity):
        if is_avg_granularity:
            return int(self.real_avg_degree)
        if manual_granularity is not None:
            return int(manual_granularity)
        return int(math.ceil(self.real_avg_degree / 32) * 32)  # graph_input.py:101

    def init_info(self, manual_granularity=None, is_avg_granularity=False):
        if not self.csr_flag:
            return self.get_split_info(manual_granularity, is_avg_granularity)
        rp = self.rowPtr.long()
        ln = rp[1:] - rp[:-1]
        self.row_nnz = ln
        self.max_row_nnz = ln.max()
        nz = ln != 0
        self.real_nrow = nz.sum()
        self.nonempty_rate = self.real_nrow / self.num_nodes
        self.avg_degree = self.num_edges / self.num_nodes
        self.COV = ln.float().std() / self.avg_degree
        if self.nonempty_rate < 0.98:  # graph_input.py:72-77
            self.real_avg_degree = (self.num_edges / self.real_nrow).item()
            self.real_COV = ln[nz].float().std() / self.real_avg_degree
        else:
            self.real_avg_degree, self.real_COV = self.avg_degree, self.COV
        first = self.colIdx[rp[:-1][nz]]
        last = self.colIdx[(rp[1:] - 1)[nz]]
        bw = last - first
        self.max_bw = bw.max()
        self.avg_bw = bw.sum() / self.real_nrow
        self.split_granularity = self._pick_granularity(manual_granularity, is_avg_granularity)
        self.split_ratio, self.row_split_nnz = self.split_ratio_comp(self.split_granularity)

    def get_split_info(self, manual_granularity=None, is_avg_granularity=False):
        rp = self.rowPtr.long()
        self.row_nnz = rp[1:] - rp[:-1]
        self.real_nrow = (self.row_nnz != 0).sum()
        self.real_avg_degree = (self.num_edges / self.real_nrow).item()
        self.split_granularity = self._pick_granularity(manual_granularity, is_avg_granularity)
        self.split_ratio, self.row_split_nnz = self.split_ratio_comp(self.split_granularity)

    def get_split(self):
        if self.split_granularity is None:
            raise ValueError("split_granularity is None, must be init first")
        self.rowPtr_split, self.target_row = ops.split_csr(self.rowPtr, self.split_granularity)


class graph_input(object):
    """One matrix in every representation the kernels accept (graph_input.py:180-430)."""

    def __init__(self, mtx_name=None, path=None, cache_dir=None):
        """``cache_dir`` (default: the environment variable PSPMM_CACHE_DIR, else none): where the
        parsed CSR arrays of a MatrixMarket file are kept as a binary container, so that later
        loads skip the text parse."""
        self.path, self.mtx_name = path, mtx_name
        self.cache_dir = cache_dir if cache_dir is not None else os.environ.get("PSPMM_CACHE_DIR")
        self.loaded_flag = self.reordered_flag = False
        self.csr_split_flag = self.bcsr_split_flag = self.bcsr_flag = False
        self.mtx_nodes = self.mtx_edges = self.density = None
        self.csr_data = self.bcsr_data = None
        self.pack_rate = None
        self.mask = None

    # -- loading ------------------------------------------------------------------------
    def load(self, load_from_mtx=True, manual_granularity=None, is_avg_granularity=False,
             is_normalize=False, GIN_epsilon=None, blk_size=2, if_mask=False):
        if self.path is None:
            raise ValueError("Graph path must be assigned first")
        if not load_from_mtx:
            raise ValueError("only MatrixMarket input is supported; use load_csr for in-memory arrays")
        # The library's parallel reader (or its binary container) replaces scipy's mmread + tocsr
        # (graph_input.py:226-232 of the reference); stored values become 1 as there (:227).
        rowPtr, colIdx, val, n_rows, n_cols = ops.load_matrix(self.path + self.mtx_name + ".mtx",
                                                              self.cache_dir, force_ones=True)
        if is_normalize or GIN_epsilon is not None:
            from scipy.sparse import csr_matrix

            mtx = csr_matrix((val.numpy().astype(np.float64), colIdx.numpy(), rowPtr.numpy()),
                             shape=(n_rows, n_cols))
            mtx = self.normalize_adj(mtx) if is_normalize else self.normalize_adj_GIN(mtx, GIN_epsilon)
            csr = mtx.tocsr()
            csr.sort_indices()
            rowPtr, colIdx, val = csr.indptr, csr.indices, csr.data
        return self.load_csr(rowPtr, colIdx, val, n_rows, manual_granularity, is_avg_granularity,
                             blk_size, if_mask)

    def load_csr(self, rowPtr, colIdx, val, n_nodes=None, manual_granularity=None,
                 is_avg_granularity=False, blk_size=2, if_mask=False):
        """Build CSR, block CSR, both row splits and (optionally) the mask from CSR arrays."""
        rowPtr = torch.as_tensor(rowPtr)
        n = int(rowPtr.shape[0] - 1) if n_nodes is None else int(n_nodes)
        self.mtx_nodes = n
        self.mtx_edges = int(rowPtr[-1])
        self.density = self.mtx_edges / (n * n)
        self.csr_data = csr_data(rowPtr, colIdx, val, n, self.mtx_edges, True)
        self.csr_data.init_info(manual_granularity, is_avg_granularity)
        c = self.csr_data
        rpb, cb, vb = ops.bcsr_from_csr(c.rowPtr, c.colIdx, c.val, n, blk_size)
        nnzblk = int(cb.shape[0])
        self.bcsr_data = csr_data(rpb, cb, vb, int(rpb.shape[0] - 1), nnzblk, False)
        self.bcsr_data.init_info(manual_granularity, is_avg_granularity)
        self.pack_rate = self.mtx_edges / (nnzblk * blk_size) if nnzblk else 0.0
        self.mask = None
        if if_mask:
            if blk_size != 2:
                raise ValueError("the mask is defined for 2 x 1 blocks only")
            dev = torch.device("cuda")
            self.mask = ops.genmask(rpb.to(dev), c.rowPtr.to(dev), vb.to(dev), self.mtx_edges).to(torch.int64)
        self.loaded_flag = self.reordered_flag = self.bcsr_flag = True
        self.get_split_csr()
        self.get_split_bcsr()
        return self

    def get_split_csr(self):
        self.csr_split_flag = True
        self.csr_data.get_split()

    def get_split_bcsr(self):
        self.bcsr_split_flag = True
        self.bcsr_data.get_split()

    # -- normalisation (scipy, as in the reference) ---------------------------------------
    def normalize_adj(self, mtx):
        """D^-1/2 (A + I) D^-1/2 in fp64 (graph_input.py:366-379)."""
        from scipy.sparse import diags

        mtx.data = np.ones_like(mtx.data)
        mtx.setdiag(1)
        deg = np.asarray(mtx.sum(1)).flatten()
        with np.errstate(divide="ignore"):
            dis = np.power(deg, -0.5)
        dis[np.isinf(dis)] = 0.0
        d = diags(dis)
        return mtx.dot(d).transpose().dot(d)

    def normalize_adj_GIN(self, mtx, epsilon):
        """(A + A^T) / 2 with (1 + epsilon) on the diagonal (graph_input.py:381-390)."""
        mtx.data = np.ones_like(mtx.data)
        mtx.setdiag(1 + epsilon)
        return (mtx + mtx.T) / 2

    # -- decider features -----------------------------------------------------------------
    def get_info(self):
        """The 1 x 15 feature vector of the reference's decider (graph_input.py:392-410)."""
        c = self.csr_data
        f = lambda x: x.item() if hasattr(x, "item") else x
        data = [self.mtx_nodes, self.mtx_edges, self.density, f(c.max_row_nnz), f(c.real_nrow),
                f(c.nonempty_rate), c.avg_degree, f(c.COV), c.real_avg_degree, f(c.real_COV),
                f(c.max_bw), f(c.avg_bw), f(c.split_ratio), f(self.bcsr_data.split_ratio), self.pack_rate]
        return np.array(data, dtype=np.float64).reshape(1, -1)

    def init_feat_embedding(self, num_features, vec_size=None):
        if num_features is None:
            raise ValueError("num_features must be assigned first")
        self.num_features = num_features
        rows = self.mtx_nodes if vec_size is None else (self.mtx_nodes + vec_size - 1) // vec_size * vec_size
        self.x = torch.randn(rows, num_features).cuda()

    def init_labels(self, num_classes, vec_size=None):
        if num_classes is None:
            raise ValueError("num_classes must be assigned first")
        self.num_classes = num_classes
        rows = self.mtx_nodes if vec_size is None else (self.mtx_nodes + vec_size - 1) // vec_size * vec_size
        self.y = torch.ones(rows).long().cuda()
