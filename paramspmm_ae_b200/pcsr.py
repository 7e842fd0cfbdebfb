"""Operator objects: host-side mirror of the reference's ``pcsr_spmm`` (PCSR.py:127-657) and
``pcsr_sddmm`` (SDDMM.py:46-254).

A ``pcsr_spmm`` holds the device copies of one representation of a matrix (CSR or V x 1
block CSR, plain or row-split) together with the legacy ``(vec_size, if_split, CF,
blkWarpNum)`` tuple and routes every method to the matching operator.  Method names,
arguments and return values follow the reference; the routing is a table instead of the
reference's nested conditionals.
"""
from __future__ import annotations

import torch

from . import baselines, ops

# (vec_size class, if_split) -> operator.  vec_size class: 1 -> "csr", 2 -> "bcsr", else "vec".
_SPMM = {("csr", False): ops.csr_spmm, ("csr", True): ops.csr_split_spmm,
         ("bcsr", False): ops.bcsr_spmm, ("bcsr", True): ops.bcsr_split_spmm,
         ("vec", False): ops.vec_spmm, ("vec", True): ops.vec_split_spmm}
_SDDMM = {("csr", False): ops.csr_sddmm, ("csr", True): ops.csr_split_sddmm,
          ("bcsr", False): ops.bcsr_sddmm, ("bcsr", True): ops.bcsr_split_sddmm,
          ("vec", False): ops.vec_sddmm, ("vec", True): ops.vec_split_sddmm}
_SPMM_PROFILE = {("csr", False): ops.csr_spmm_profile, ("csr", True): ops.csr_split_spmm_profile,
                 ("bcsr", False): ops.bcsr_spmm_profile, ("bcsr", True): ops.bcsr_split_spmm_profile,
                 ("vec", False): ops.vec_spmm_profile, ("vec", True): ops.vec_split_spmm_profile}
_SDDMM_PROFILE = {("csr", False): ops.csr_sddmm_profile, ("csr", True): ops.csr_split_sddmm_profile,
                  ("bcsr", False): ops.bcsr_sddmm_profile, ("bcsr", True): ops.bcsr_split_sddmm_profile,
                  ("vec", False): ops.vec_sddmm_profile, ("vec", True): ops.vec_split_sddmm_profile}
_CONV_FWD = {("csr", False): ops.csr_spmm_forward, ("csr", True): ops.csr_split_spmm_forward,
             ("bcsr", False): ops.bcsr_spmm_forward, ("bcsr", True): ops.bcsr_split_spmm_forward}


class _format_spmm(object):
    """Shared body of the COO and CSC comparator objects (PCSR.py:45-124): device copies of one
    storage format of the graph's matrix, a result and a timing method over cuSPARSE."""

    label = ""

    def _arrays(self):
        raise NotImplementedError

    def _input(self, dim, x):
        if x is None and dim is None:
            raise ValueError("at least one of x and dim should be given")
        return torch.ones(self.mtx_nodes, dim, device="cuda") if dim is not None else x.to("cuda")

    def get_spmm_result(self, dim=None, x=None):
        return self._compute(self._input(dim, x), *self._arrays()).to("cpu")

    def profiling(self, dim=None, x=None):
        tp = self._profile(self._input(dim, x), *self._arrays())
        print("{}-> dim: {} gflops: {:.0f}".format(self.label, dim, tp))
        return tp


class coo_spmm(_format_spmm):
    """cuSPARSE COO (ALG4) comparator built from a ``graph_input`` (PCSR.py:45-84)."""

    label = "coo"
    _compute = staticmethod(baselines.cusparse_compute_coo_alg4)
    _profile = staticmethod(baselines.cusparse_profile_coo_alg4)

    def __init__(self, graph, device="cuda"):
        c = graph.csr_data
        lens = (c.rowPtr[1:] - c.rowPtr[:-1]).long()
        self.row = torch.repeat_interleave(torch.arange(graph.mtx_nodes, dtype=torch.int32), lens).to(device)
        self.col, self.val = c.colIdx.to(device), c.val.to(device)
        self.mtx_nodes = graph.mtx_nodes

    def _arrays(self):
        return self.row, self.col, self.val


class csc_spmm(_format_spmm):
    """cuSPARSE CSC comparator built from a ``graph_input`` (PCSR.py:87-124)."""

    label = "csc"
    _compute = staticmethod(baselines.cusparse_compute_csc)
    _profile = staticmethod(baselines.cusparse_profile_csc)

    def __init__(self, graph, device="cuda"):
        from scipy.sparse import csr_array
        c = graph.csr_data
        csc = csr_array((c.val.numpy(), c.colIdx.numpy(), c.rowPtr.numpy()),
                        shape=(graph.mtx_nodes, graph.mtx_nodes)).tocsc()
        self.colPtr = torch.from_numpy(csc.indptr.astype("int32")).to(device)
        self.rowIdx = torch.from_numpy(csc.indices.astype("int32")).to(device)
        self.val = torch.from_numpy(csc.data).to(device)
        self.mtx_nodes = graph.mtx_nodes

    def _arrays(self):
        return self.colPtr, self.rowIdx, self.val


def _kind(vec_size):
    return "csr" if vec_size == 1 else ("bcsr" if vec_size == 2 else "vec")


class pcsr_spmm(object):
    def __init__(self, graph, vec_size, if_split, mtx_nodes=None, mtx_edges=None, rowPtr=None,
                 colIdx=None, val=None, target_row=None, CF=1, blkWarpNum=4, device="cuda"):
        """From a ``graph_input`` (graph is not None) or from raw tensors (PCSR.py:128-204)."""
        if_split = bool(if_split)
        self.mask = None
        if graph is None:
            if any(x is None for x in (mtx_edges, mtx_nodes, rowPtr, colIdx, val)):
                raise ValueError("when graph is None, mtx_nodes, mtx_edges, rowPtr, colIdx, val should be given")
            if if_split and target_row is None:
                raise ValueError("target_row should be given when if_split is True")
            if not if_split and target_row is not None:
                raise ValueError("target_row should not be given when if_split is False")
            if (vec_size == 1) != (val.dim() == 1):
                raise ValueError("val must be 1-D for vec_size 1 and [nblk, vec_size] otherwise")
            self.mtx_nodes, self.mtx_edges = mtx_nodes, mtx_edges
            self.rowPtr, self.colIdx, self.val = rowPtr.to(device), colIdx.to(device), val.to(device)
            self.target_row = target_row.to(device) if target_row is not None else None
        else:
            self.mtx_nodes, self.mtx_edges = graph.mtx_nodes, graph.mtx_edges
            src = graph.csr_data if vec_size == 1 else graph.bcsr_data
            self.rowPtr = (src.rowPtr_split if if_split else src.rowPtr).to(device)
            self.colIdx, self.val = src.colIdx.to(device), src.val.to(device)
            self.target_row = src.target_row.to(device) if if_split else None
            if vec_size != 1 and graph.mask is not None:
                self.mask = graph.mask.to(device)
        self.vec_size, self.if_split, self.CF, self.blkWarpNum = vec_size, if_split, CF, blkWarpNum
        self.result = None
        self._planned = None

    @classmethod
    def from_plan(cls, plan, rowPtr, colIdx, val, mtx_nodes=None, device="cuda"):
        """Operator bound to a decider plan (``decider.choose`` / ``SpMMDecider.plan``) instead of
        the legacy tuple: the products with the stored values (``GIN_spmm``, ``forward``,
        ``backward``, ``get_spmm_result``) run the layout and kernel parameters the plan names,
        the length-bucketed internal plan included, which the legacy signatures cannot express.
        The CSR arrays stay attached for everything else (SDDMM, ``AGNN_spmm`` with caller-supplied
        edge values, the comparators).  The reference has no counterpart: its operators carry
        ``(vec_size, if_split, CF, blkWarpNum)`` only (PCSR.py:128-204)."""
        from . import decider
        n = rowPtr.shape[0] - 1 if mtx_nodes is None else mtx_nodes
        self = cls(None, 1, False, n, colIdx.shape[0], rowPtr, colIdx, val, None, CF=1, blkWarpNum=8, device=device)
        self._planned = decider.PlannedSpMM(plan, self.rowPtr, self.colIdx, self.val, n_cols=n)
        return self

    def _planned_product(self, X):
        """One output row per input row, as the legacy operators give (rows beyond the matrix zero);
        a width that is not a multiple of 4 is padded for the launch and cut back."""
        n, dim = X.shape
        Xp = ops._pad_cols(X, -dim % 4).contiguous()
        rows = self._planned.n_rows
        if n < rows:
            raise RuntimeError("the matrix has %d rows, the input only %d" % (rows, n))
        out = torch.empty((n, Xp.shape[1]), dtype=torch.float32, device=X.device)
        if n > rows:
            out[rows:].zero_()
        self._planned(out[:rows], Xp)
        return out[:, :dim].contiguous() if Xp.shape[1] != dim else out

    # -- helpers ------------------------------------------------------------------------
    def _key(self):
        return _kind(self.vec_size), self.if_split

    def _layout(self, val=None):
        v = self.val if val is None else val
        if self.if_split:
            return (self.rowPtr, self.colIdx, v, self.target_row)
        return (self.rowPtr, self.colIdx, v)

    def _dense_input(self, dim, x):
        if x is None and dim is None:
            raise ValueError("at least one of x and dim should be given")
        if dim is not None:
            return torch.ones(self.mtx_nodes, dim, device="cuda")
        return x.to("cuda")

    # -- SpMM ---------------------------------------------------------------------------
    def get_spmm_result(self, dim=None, x=None, CF=None, blkWarpNum=None):
        X = self._dense_input(dim, x)
        CF = self.CF if CF is None else CF
        W = self.blkWarpNum if blkWarpNum is None else blkWarpNum
        out = self._planned_product(X) if self._planned else _SPMM[self._key()](X, *self._layout(), CF, W)
        self.result = out[: self.mtx_nodes].to("cpu")  # block layouts pad the row count

    def AGNN_spmm(self, spVal, X):
        """SpMM with caller-supplied edge values in place of the stored ones (PCSR.py:244-265)."""
        return _SPMM[self._key()](X, *self._layout(spVal), self.CF, self.blkWarpNum)

    def GIN_spmm(self, X):
        if self._planned:
            return self._planned_product(X)
        return _SPMM[self._key()](X, *self._layout(), self.CF, self.blkWarpNum)

    # -- SDDMM --------------------------------------------------------------------------
    def AGNN_sddmm(self, A):
        """Edge scores <A[i], A[j]> on the pattern (PCSR.py:290-320); CF = ceil(dim/32)."""
        if self.vec_size == 2 and self.mask is None:
            raise ValueError("mask should be given when vec_size=2")
        CF = (A.size(1) + 31) // 32
        return _SDDMM[self._key()](A, A, *self._layout(), CF, self.blkWarpNum)

    def get_sddmm_result(self, dim, blkWarpNum):
        A = torch.ones((self.mtx_nodes + 1) // 2 * 2, dim, device="cuda")
        B = torch.ones(self.mtx_nodes, dim, device="cuda")
        self.result = _SDDMM[self._key()](A, B, *self._layout(), (dim + 31) // 32, blkWarpNum).to("cpu")
        return self.result

    # -- GCN layer ----------------------------------------------------------------------
    def _conv_key(self):
        return ("csr" if self.vec_size == 1 else "bcsr"), self.if_split

    def forward(self, H, w):
        if H is None or w is None:
            raise ValueError("H and w should be given")
        if self._planned:
            return ops._conv_forward(1, H, w, None, None, None, None, self.CF, self.blkWarpNum, product=self._planned_product)
        return _CONV_FWD[self._conv_key()](H, w, *self._layout(), self.CF, self.blkWarpNum)

    def backward(self, d_output, H, w, input_grad=True):
        """(dH, dW) of the layer (PCSR.py:381-432); ``input_grad=False`` skips the dH product and
        returns None in its place (no reference counterpart: it always forms both)."""
        if d_output is None or H is None:
            raise ValueError("d_output and H should be given")
        V = 1 if self.vec_size == 1 else 2
        layout = (None, None, None, None) if self._planned else self._layout() + ((None,) if not self.if_split else ())
        return tuple(ops._conv_backward(V, d_output, H, w, *layout, self.CF, self.blkWarpNum,
                                        product=self._planned_product if self._planned else None,
                                        input_grad=input_grad))

    # -- timing -------------------------------------------------------------------------
    def cf_warpnum_profiling(self, CF, blkWarpNum, dim=None, x=None):
        X = self._dense_input(dim, x)
        extra = () if self.vec_size == 1 else (self.mtx_edges,)
        tp = _SPMM_PROFILE[self._key()](X, *self._layout(), *extra, CF, blkWarpNum)
        print("dim: {} gflops: {:.0f}".format(X.shape[1], tp))
        return tp

    def profiling(self, dim=None, x=None):
        return self.cf_warpnum_profiling(self.CF, self.blkWarpNum, dim, x)

    def _baseline(self, compute, profile, label, dim, x, is_profiling):
        if self.if_split or self.vec_size != 1:
            raise ValueError("cusparse only support vec_size=1 and if_split=False")
        X = self._dense_input(dim, x)
        if is_profiling:
            tp = profile(X, self.rowPtr, self.colIdx, self.val)
            print("{}-> dim: {} gflops: {:.0f}".format(label, dim, tp))
            return tp
        return compute(X, self.rowPtr, self.colIdx, self.val).to("cpu")

    def cusparse_ref(self, dim=None, x=None, is_profiling=False):
        return self._baseline(baselines.cusparse_compute, baselines.cusparse_profile, "cusparse", dim, x, is_profiling)

    def cusparse_csr_alg2_ref(self, dim=None, x=None, is_profiling=False):
        return self._baseline(baselines.cusparse_compute_csr_alg2, baselines.cusparse_profile_csr_alg2,
                              "cusparse_csr_alg2", dim, x, is_profiling)

    def gespmm_ref(self, dim=None, x=None, is_profiling=False):
        return self._baseline(baselines.gespmm_compute, baselines.gespmm_profile, "gespmm", dim, x, is_profiling)


class pcsr_sddmm(pcsr_spmm):
    """SDDMM-side operator object (SDDMM.py:46-254): same storage, SDDMM timing and reference."""

    def profiling(self, blkWarpNum, dim):
        A = torch.ones((self.mtx_nodes + 1) // 2 * 2, dim, device="cuda")
        B = torch.ones(self.mtx_nodes, dim, device="cuda")
        extra = () if self.vec_size == 1 else (self.mtx_edges,)
        tp = _SDDMM_PROFILE[self._key()](A, B, *self._layout(), *extra, (dim + 31) // 32, blkWarpNum)
        print("dim: {} gflops: {:.0f}".format(dim, tp))
        return tp

    def cusparse_ref(self, dim=None, is_profiling=False):
        if self.if_split or self.vec_size != 1:
            raise ValueError("cusparse only support vec_size=1 and if_split=False")
        A = torch.ones(self.mtx_nodes, dim, device="cuda")
        vals = self.val.clone()
        if is_profiling:
            return baselines.cusparse_sddmm_profile(A, A, self.rowPtr, self.colIdx, vals)
        return baselines.cusparse_sddmm_compute(A, A, self.rowPtr, self.colIdx, vals).to("cpu")


def compare(result, result_ref, rel=1e-4):
    """The reference's SDDMM acceptance rule (SDDMM.py:19-36): relative error at most 1e-4."""
    err = (result_ref - result).abs()
    return not bool((err > rel * result_ref.abs()).any())


def compare_2d(result, result_ref, mask, rel=1e-4):
    """Block results are compared in CSR order through the mask (SDDMM.py:39-43)."""
    return compare(result.reshape(-1)[mask], result_ref, rel)
