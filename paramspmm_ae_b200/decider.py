"""SpMM-decider: picks the PCSR representation and kernel parameters for a matrix and a dim.

Stands in for the reference's ``SpMMDecider`` (decider.py:18-93), which feeds 15 matrix
statistics to a pickled random forest per dim and decodes the predicted class into
``<if_split, vec_size, CF, blkWarpNum>``.  Here the choice comes from a measured table
(``config_table.json`` next to this file) keyed on a bucket of the nnz-per-row distribution
and on dim; the table's values are the parameters of the sm_100a kernels: vector width,
lanes per row (= 32 / rows per warp), rows per lane group and PCSR partition length.  The
legacy 4-tuple is still returned to callers that expect it; its CF / blkWarpNum members are
valid values of the reference's domain and act only as hints.
"""
from __future__ import annotations

import json
import math
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
TABLE_PATH = os.path.join(_HERE, "config_table.json")


def gap_calculator(dim, CF, warp_size=32):
    """Idle lanes in the last column tile (same rule as PCSR.py:19-26 of the reference)."""
    t_res = dim % (warp_size * CF)
    return 0 if t_res == 0 else min(dim, CF * warp_size) - t_res


def dynamic_CF_prompter(dim, CF_set=None, warp_size=32):
    """Coarsening factors the reference considers valid for a dim (PCSR.py:30-42)."""
    if CF_set is None:
        CF_set = [1, 2, 3, 4, 5, 6, 7, 8]
    CF_set = CF_set[: math.ceil(dim / 32)]
    return [cf for cf in CF_set if gap_calculator(dim, cf, warp_size) < 32]


NEAR_DIAGONAL = 256  # |column - row| up to which an entry counts as local


def near_diagonal_share(rowPtr, colIdx, reach=NEAR_DIAGONAL):
    """Share of the entries whose column lies within `reach` of their row: close to 1 for banded and
    locality-ordered matrices, whose rows of the dense operand are re-read out of L1 by neighbouring
    rows, close to 0 for scattered columns, whose gathers go to L2 and DRAM.  (The reference's
    statistics carry the same information as max_bw / avg_bw, graph_input.py:392-410.)"""
    rp = torch.as_tensor(rowPtr).long()
    ci = torch.as_tensor(colIdx).long()
    n = rp.numel() - 1
    if n <= 0 or ci.numel() == 0:
        return 0.0
    rows = torch.repeat_interleave(torch.arange(n, device=rp.device), rp[1:] - rp[:-1])
    return float(((ci - rows).abs() <= reach).double().mean())


def row_stats(rowPtr, colIdx=None):
    """nnz-per-row summary of a CSR row pointer (torch tensor or numpy array, any device); with the
    column indices also `near_diag`, the share of entries close to the diagonal."""
    rp = torch.as_tensor(rowPtr).long()
    ln = (rp[1:] - rp[:-1]).double()
    n = ln.numel()
    if n == 0:
        return {"n_rows": 0, "nnz": 0, "avg": 0.0, "cov": 0.0, "max": 0, "real_avg": 0.0, "near_diag": 0.0}
    nnz = int(rp[-1] - rp[0])
    avg = nnz / n
    nonempty = int((ln > 0).sum())
    std = float(ln.std(unbiased=True)) if n > 1 else 0.0
    real_avg = nnz / nonempty if nonempty and nonempty / n < 0.98 else avg
    return {"n_rows": n, "nnz": nnz, "avg": avg, "cov": std / avg if avg else 0.0,
            "max": int(ln.max()), "real_avg": real_avg,
            "near_diag": near_diagonal_share(rp, colIdx) if colIdx is not None else 0.0}


SIZES = ("tiny", "short", "medium", "long")
KINDS = ("even", "local", "skewed")


def regime(stats):
    """Bucket of the matrix: mean row length class x {skewed, local, even}.  Skewed = row lengths
    vary strongly (hub rows: they need the row split); local = even lengths with nearly all columns
    next to the diagonal (L1-bound gathers); even = the rest (scattered columns, L2 / DRAM bound)."""
    avg = stats["avg"]
    size = "tiny" if avg < 6 else ("short" if avg < 24 else ("medium" if avg < 128 else "long"))
    if stats["cov"] > 0.75 or stats["max"] > 16 * max(avg, 1.0):
        kind = "skewed"
    elif stats.get("near_diag", 0.0) >= 0.9:
        kind = "local"
    else:
        kind = "even"
    return size + "_" + kind


def auto_granularity(real_avg_degree):
    """The reference's partition length: ceil(avg / 32) * 32 (graph_input.py:101)."""
    return max(32, int(math.ceil(real_avg_degree / 32) * 32))


_DEFAULT_TABLE = {"version": 1, "source": "built-in defaults (no measurements)", "entries": {}}
_table = None


def load_table(path=None):
    global _table
    p = path or TABLE_PATH
    if os.path.exists(p):
        with open(p) as f:
            _table = json.load(f)
    else:
        _table = dict(_DEFAULT_TABLE)
    return _table


def table():
    return _table if _table is not None else load_table()


def _dim_key(dim):
    return str(int(math.ceil(dim / 16) * 16)) if dim <= 256 else "256"


class Plan(dict):
    """Chosen representation and kernel parameters.

    Keys: if_split (0/1), vec_size (1/2), granularity (partition length or None = the
    reference's rule), and kernel fields lanes_per_row / vec_width / cta_threads /
    rows_per_group (0 = library default).
    """

    def kernel_cfg(self):
        return {k: int(self.get(k, 0) or 0)
                for k in ("lanes_per_row", "vec_width", "cta_threads", "rows_per_group", "gather_batch", "col_tile",
                          "bucketed")}


def choose(stats, dim, op="spmm"):
    """Table lookup (regime x dim); falls back to a rule when the table has no entry."""
    reg = regime(stats)
    per_regime = table().get("entries", {}).get(op, {})
    ent = per_regime.get(reg, {})
    if not ent:
        # A regime the sweep has not measured borrows from the nearest measured size of the same kind
        # (the kernel shape depends on the dim first, the row-length class second); a local matrix
        # without any local measurement is treated as an even one.
        size, kind = reg.split("_")
        i = SIZES.index(size)
        near = sorted((s for s in SIZES if s != size), key=lambda s: abs(SIZES.index(s) - i))
        for k in ([kind] if kind != "local" else ["local", "even"]):
            for other in ([size] if k != kind else []) + near:
                ent = per_regime.get(other + "_" + k, {})
                if ent:
                    break
            if ent:
                break
    e = ent.get(_dim_key(dim)) or ent.get("*")
    if e is not None and ent is not per_regime.get(reg) and e.get("if_split"):
        e = dict(e, granularity=None)  # a borrowed partition length does not transfer: use the rule
    if e is None:
        e = {"if_split": 1 if reg.endswith("skewed") else 0, "vec_size": 1}
    plan = Plan(if_split=0, vec_size=1, granularity=None, lanes_per_row=0, vec_width=0, cta_threads=0,
                rows_per_group=0, gather_batch=0, col_tile=0, bucketed=0)
    plan.update(e)
    plan["regime"] = reg
    if plan["if_split"] and not plan.get("granularity"):
        plan["granularity"] = auto_granularity(stats["real_avg"])
    return plan


class PlannedSpMM:
    """A plan bound to one matrix: builds the arrays the plan's layout needs once (the PCSR split on
    the device, or the length-bucketed plan with its permuted entries) and launches the SpMM with
    the plan's kernel parameters.  ``rowPtr`` / ``colIdx`` / ``val`` are CUDA tensors of a CSR matrix."""

    def __init__(self, plan, rowPtr, colIdx, val, n_cols=None):
        from . import ops
        self.plan, self.n_rows = plan, rowPtr.shape[0] - 1
        self.V = int(plan.get("vec_size", 1) or 1)
        self.n_seg_rows = self.n_rows  # (block-)rows of the output
        if self.V > 1:  # V x 1 blocks: built by the host builder (scipy's tobsr layout), then moved back
            dev = rowPtr.device
            if n_cols is None:
                n_cols = int(colIdx.max()) + 1 if colIdx.numel() else 1
            rowPtr, colIdx, val = (t.to(dev) for t in ops.bcsr_from_csr(rowPtr.cpu(), colIdx.cpu(), val.cpu(), n_cols, self.V))
            self.n_seg_rows = rowPtr.shape[0] - 1
        self.colIdx, self.val, self.target = colIdx, val, None
        self.segPtr = rowPtr
        if plan.get("bucketed") and plan["if_split"]:
            self.segPtr, self.colIdx, self.val, self.target = ops.bucket_pcsr(rowPtr, colIdx, val, int(plan["granularity"]))
        elif plan["if_split"]:
            self.segPtr, self.target = ops.split_csr_device(rowPtr, int(plan["granularity"]))
        self.n_seg = self.segPtr.shape[0] - 1

    def __call__(self, out, B, accumulate=False):
        from . import _lib, ops
        kw = self.plan.kernel_cfg()
        if accumulate:  # built for 128-bit loads at one gather-batch depth
            kw.update(vec_width=0, gather_batch=0, accumulate=1)
        dst = out
        if out.shape[0] < self.n_seg_rows * self.V:  # block layouts write whole blocks: an odd row count needs a pad row
            dst = torch.empty(self.n_seg_rows * self.V, out.shape[1], dtype=out.dtype, device=out.device)
        ops.spmm_into(dst, B, self.segPtr, self.colIdx, self.val, target_row=self.target, V=self.V,
                      n_out_rows=self.n_seg_rows, cfg=_lib.make_cfg(**kw))
        if dst is not out:
            out.copy_(dst[: out.shape[0]])
        return out

    @property
    def launches(self):
        """Kernels per product: the SpMM, plus the zeroing pre-pass of a split layout."""
        return 2 if self.target is not None else 1


def legacy_tuple(plan, dim):
    """<if_split, vec_size, CF, blkWarpNum> in the reference's domain (decider.py:63-80)."""
    cfs = dynamic_CF_prompter(int(math.ceil(dim / 16) * 16))
    return int(plan["if_split"]), int(plan["vec_size"]), cfs[-1], 8


class SpMMDecider(object):
    """Same surface as the reference's class (decider.py:18-93).  ``pickle_path`` is accepted
    for compatibility; a path to a JSON table may be given instead and is loaded."""

    def __init__(self, pickle_path=None):
        self.pickle_path = pickle_path
        self.model_dict = {}
        if pickle_path and str(pickle_path).endswith(".json"):
            load_table(pickle_path)

    def gen_model_dict(self, dim_list):
        if dim_list is None or len(dim_list) == 0:
            raise ValueError("dim_list must be assigned and non-empty")
        self.model_dict = {d: table() for d in dim_list}

    def decode_tree(self, code, dim, vec_size_list=(1, 2), warpNum_list=(4, 8)):
        if_split = code % 2
        cf_list = dynamic_CF_prompter(dim)
        nv = len(vec_size_list)
        vec_size = vec_size_list[code // 2 % nv]
        CF = cf_list[code // (nv * 2) % len(cf_list)]
        W = warpNum_list[code // (len(cf_list) * nv * 2)]
        return if_split, vec_size, CF, W

    def plan(self, graph, dim):
        key = id(graph)
        if getattr(self, "_stats_of", None) != key:  # the statistics of a graph are computed once, not per dim
            self._stats, self._stats_of = row_stats(graph.csr_data.rowPtr, graph.csr_data.colIdx), key
        return choose(self._stats, dim)

    def config_PCSR(self, graph, dim):
        if dim not in self.model_dict:
            raise ValueError("dim-" + str(dim) + " not found in model_dict")
        return legacy_tuple(self.plan(graph, dim), dim)


def install_tuner():
    """Route the table's kernel parameters into the torch-level operators: every call made
    through the legacy signatures then picks lanes per row / rows per group from the table,
    keyed on dim and on the mean entries per (split-)row, which the call's tensor shapes give
    without touching the device."""
    from . import ops

    def tuner(op, dim, mean_len, V, split):
        size = "tiny" if mean_len < 6 else ("short" if mean_len < 24 else ("medium" if mean_len < 128 else "long"))
        ent = table().get("entries", {}).get(op, {})
        e = (ent.get(size + "_even", {}) or {}).get(_dim_key(dim)) or {}
        return {k: int(e.get(k, 0) or 0) for k in ("lanes_per_row", "vec_width", "cta_threads", "rows_per_group",
                                                   "gather_batch", "col_tile")}

    ops.tuner = tuner
    return tuner


def main(argv=None):
    """Command line of the reference's decider.py (:96-173): for every MatrixMarket file under
    ``--path`` (or the one named by ``--mtx_name``) and every dim, choose the configuration, check
    the product against ``torch.sparse.mm`` with the reference's rule, time it (200 back-to-back
    launches) and time cuSPARSE and the GE-SpMM restatement on the same arrays.  Prints the
    reference's separator lines plus one summary line per dim; ``--json`` also writes one JSON
    object per (matrix, dim)."""
    import argparse
    import glob

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--path", type=str, default="./dataset/all-mtx/", help="path to the mtx files")
    ap.add_argument("--dim_list", nargs="*", type=int, default=[16, 32, 48, 64, 80, 96, 112, 128])
    ap.add_argument("--mtx_name", type=str, default="", help="mtx file name (without .mtx)")
    ap.add_argument("--json", type=str, default="", help="write one JSON line per (matrix, dim) to this file")
    ap.add_argument("--cache_dir", type=str, default=None, help="keep parsed matrices here as binary CSR")
    ap.add_argument("--no_baselines", action="store_true", help="skip the cuSPARSE and GE-SpMM timings")
    args = ap.parse_args(argv)
    print(args)

    import torch

    from . import _lib, baselines, ops
    from .graph_input import graph_input
    from .verification import SpMM_verification

    path = args.path if args.path.endswith(os.sep) else args.path + os.sep
    if args.mtx_name:
        names = [args.mtx_name]
    else:
        names = sorted(os.path.basename(f)[:-4] for f in glob.glob(os.path.join(path, "*.mtx")))
    decider = SpMMDecider()
    decider.gen_model_dict(args.dim_list)
    dev = torch.device("cuda")
    records = []
    for name in names:
        graph = graph_input(mtx_name=name, path=path, cache_dir=args.cache_dir)
        print("-------------mtx: {}-------------".format(name))
        graph.load(load_from_mtx=True)
        c = graph.csr_data
        n, nnz = graph.mtx_nodes, graph.mtx_edges
        veri = SpMM_verification(1, c.rowPtr, c.colIdx, c.val)
        rp, ci, v = c.rowPtr.to(dev), c.colIdx.to(dev), c.val.to(dev)
        layouts = {}
        for dim in args.dim_list:
            plan = decider.plan(graph, dim)
            legacy = decider.config_PCSR(graph, dim)
            X = torch.ones(n, dim, device=dev)
            out = torch.empty(n, dim, device=dev)
            key = (int(plan["if_split"]), plan.get("granularity"), int(plan.get("bucketed", 0)))
            if key not in layouts:
                layouts[key] = PlannedSpMM(plan, rp, ci, v)
            op = layouts[key]
            op.plan = plan
            op(out, X)
            veri.reference(dim)
            veri.compare(out.cpu(), name)
            ms = ops.spmm_time_ms(X, op.segPtr, op.colIdx, op.val, op.target, cfg=_lib.make_cfg(**plan.kernel_cfg()),
                                  n_out_rows=n)
            rec = {"mtx": name, "nodes": n, "edges": nnz, "dim": dim, "regime": plan["regime"],
                   "if_split": int(plan["if_split"]), "vec_size": int(plan["vec_size"]),
                   "granularity": plan["granularity"], "kernel": plan.kernel_cfg(), "legacy_tuple": list(legacy),
                   "ms": round(ms, 5), "gflops": int(nnz / 1e6 * dim * 2 / ms)}
            if not args.no_baselines:
                rec["cusparse_gflops"] = baselines.cusparse_profile(X, rp, ci, v)
                rec["gespmm_gflops"] = baselines.gespmm_profile(X, rp, ci, v)
            print("=======================================")
            line = "dim: {dim} regime: {regime} if_split: {if_split} vec_size: {vec_size} gflops: {gflops}".format(**rec)
            if not args.no_baselines:
                line += " cusparse: {} ({:.2f}x) gespmm: {} ({:.2f}x)".format(
                    rec["cusparse_gflops"], rec["gflops"] / max(1, rec["cusparse_gflops"]),
                    rec["gespmm_gflops"], rec["gflops"] / max(1, rec["gespmm_gflops"]))
            print(line)
            records.append(rec)
    if args.json:
        with open(args.json, "w") as f:
            for rec in records:
                f.write(json.dumps(rec) + "\n")
    return records


if __name__ == "__main__":
    main()
