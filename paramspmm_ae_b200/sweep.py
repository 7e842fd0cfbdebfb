#!/usr/bin/env python3
"""Measured configuration sweep: the stand-in for the reference's ``profile_engine`` /
``training_data_gen`` (PCSR.py:672-823), which time every <representation, CF, blkWarpNum>
on a matrix collection and label each (matrix, dim) with the fastest, and for the hold-out
evaluation of its decider (models/rnd_tree.ipynb: accuracy and "normalised performance" of the
predicted configuration against the best one on matrices the forests were not trained on).

The swept space is that of the sm_100a kernels: PCSR split on/off and partition length, block
height (vec_size 1 or 2), lanes per row (rows per warp), rows per lane group, gather depth, CTA
size, column tiles.

    python -m paramspmm_ae_b200.sweep fit     --table paramspmm_ae_b200/config_table.json
    python -m paramspmm_ae_b200.sweep holdout --out paramspmm_ae_b200/decider_holdout.json

``fit`` times every candidate on the fitting matrices of each row-length regime and writes, per
(regime, dim), the configuration with the smallest summed time.
``holdout`` takes matrices that ``fit`` never sees (other generators' parameters, sizes and seeds),
times for each (matrix, dim) the whole candidate space and the configuration the table gives, and
records table-choice time / best time.  Each candidate is verified against the plain-CSR result of
the default configuration before it is timed (the reference verifies each candidate against
torch.sparse.mm, PCSR.py:759-770).
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
import time

import torch

from . import _lib, decider, ops, synth

ALL_REGIMES = ["tiny_even", "tiny_skewed", "short_even", "short_local", "short_skewed", "medium_even", "medium_local",
               "medium_skewed", "long_even", "long_skewed"]


def fitting_matrices(n, device, which):
    """Matrices the table is fitted on, per regime.  Seeds and sizes differ from the benchmark's
    matrices (bench.py: seeds 21-23 at 10^6 rows) and from the hold-out set below."""
    scale = max(1, (n - 1).bit_length())
    makers = {
        "tiny_even": lambda: [("uniform4", synth.uniform_rows(n, 4, seed=127, device=device))],
        "tiny_skewed": lambda: [("rmat4", synth.rmat(scale, 4 * n, n=n, seed=128, device=device))],
        "short_even": lambda: [("uniform16", synth.uniform_rows(n, 16, seed=121, device=device))],
        "short_local": lambda: [("banded16", synth.banded_rows(n, 16, 32, seed=122, device=device)),
                                ("banded12_bw100", synth.banded_rows(n, 12, 100, seed=130, device=device))],
        "short_skewed": lambda: [("rmat16", synth.rmat(scale, 16 * n, n=n, seed=123, device=device)),
                                 ("powerlaw12", synth.powerlaw_graph(n // 2, (n // 2) * 6, seed=124, device=device))],
        "medium_even": lambda: [("uniform64", synth.uniform_rows(n // 4, 64, seed=125, device=device))],
        "medium_local": lambda: [("banded64_bw96", synth.banded_rows(n // 4, 64, 96, seed=129, device=device))],
        "medium_skewed": lambda: [("powerlaw50", synth.powerlaw_graph(n // 4, (n // 4) * 25, seed=131, device=device)),
                                  ("rmat40", synth.rmat(max(1, scale - 2), 10 * n, seed=132, device=device))],
        "long_even": lambda: [("uniform256", synth.uniform_rows(n // 16, 256, seed=126, device=device))],
        "long_skewed": lambda: [("powerlaw490", synth.powerlaw_graph(232965 if n >= 1_000_000 else n // 8,
                                                                     (232965 if n >= 1_000_000 else n // 8) * 245,
                                                                     seed=141, device=device))],
    }
    out = {}
    for r in which:
        for name, m in makers[r]():  # a matrix is fitted for the regime the decider puts it in
            got = decider.regime(decider.row_stats(m.rowPtr, m.colIdx))
            if got != r:
                print("note: fitting matrix %s falls into %s, not %s" % (name, got, r), flush=True)
            out.setdefault(got, []).append((name, m))
    return out


def holdout_matrices(device, scale=1.0):
    """Eighteen matrices no fit ever sees: other sizes, mean degrees 4..600, R-MAT and Chung-Lu
    exponents, narrow and wide bands, all six regimes."""
    s = lambda x: max(2048, int(x * scale))
    return [
        ("uniform_k8", synth.uniform_rows(s(500_000), 8, seed=201, device=device)),
        ("uniform_k4", synth.uniform_rows(s(1_200_000), 4, seed=202, device=device)),
        ("uniform_k40", synth.uniform_rows(s(300_000), 40, seed=203, device=device)),
        ("uniform_k200", synth.uniform_rows(s(60_000), 200, seed=204, device=device)),
        ("banded_k12_bw48", synth.banded_rows(s(700_000), 12, 48, seed=205, device=device)),
        ("banded_k48_bw64", synth.banded_rows(s(200_000), 48, 64, seed=206, device=device)),
        ("banded_k16_bw200", synth.banded_rows(s(800_000), 16, 200, seed=207, device=device)),
        ("rmat_deg8", synth.rmat(19, s(4_000_000), seed=208, device=device)),
        ("rmat_deg46", synth.rmat(18, s(12_000_000), seed=209, device=device)),
        ("rmat_flat_deg23", synth.rmat(20, s(24_000_000), a=0.45, b=0.22, c=0.22, seed=210, device=device)),
        ("chunglu_g2.1_deg11", synth.powerlaw_graph(s(400_000), s(2_000_000), gamma=2.1, seed=211, device=device)),
        ("chunglu_g3.0_deg11", synth.powerlaw_graph(s(600_000), s(3_000_000), gamma=3.0, seed=212, device=device)),
        ("chunglu_g2.5_deg61", synth.powerlaw_graph(s(150_000), s(4_500_000), gamma=2.5, seed=213, device=device)),
        ("chunglu_g2.1_deg600", synth.powerlaw_graph(s(50_000), s(15_000_000), gamma=2.1, seed=214, device=device)),
        ("uniform_k24", synth.uniform_rows(s(400_000), 24, seed=215, device=device)),
        ("banded_k6_bw20", synth.banded_rows(s(900_000), 6, 20, seed=216, device=device)),
        ("rmat_deg5", synth.rmat(20, s(5_000_000), seed=217, device=device)),
        ("rmat_skew_deg30", synth.rmat(19, s(15_000_000), a=0.65, b=0.15, c=0.15, seed=218, device=device)),
    ]


def candidates(dim, regime, quick=False, vecs=(1, 2), cta_threads=(64, 128, 256)):
    vw = 4 if dim % 4 == 0 else (2 if dim % 2 == 0 else 1)
    nvec = dim // vw
    top = 1
    while top < nvec and top < 32:
        top <<= 1
    lprs = sorted({l for l in (top, top // 2, top // 4) if 4 <= l <= 32 and (nvec + l - 1) // l <= 8} or {max(4, top)})
    rpgs = (4, 8) if quick else (2, 4, 8)
    mlps = (4, 8) if quick else (4, 8, 16)
    skew = regime.endswith("skewed")
    long_rows = regime.startswith("long") or regime.startswith("medium")
    if regime.startswith("tiny"):
        rpgs = (4, 8) if quick else (2, 4, 8, 16)  # very short rows: more of them per lane group
    if skew or long_rows:
        grans = [0, 32, 64, 128] if not long_rows else [0, 64, 128, 256, 512]
    else:
        grans = [0]
    if quick:
        vecs, cta_threads = (1,), (256,)
    tiles = [0] + [t for t in (32, 64, 128) if t < dim and dim % 4 == 0]
    if dim >= 96 and dim % 4 == 0 and not skew:
        # equal parts: a width that is not a multiple of 64 would otherwise end in a narrow remainder launch
        tiles += [t for t in sorted({(-(-dim // parts) + 3) // 4 * 4 for parts in (2, 3, 4)}) if t not in tiles and 32 <= t < dim]
    for vec, gran, lpr, rpg, mlp, thr, tile in itertools.product(vecs, grans, lprs, rpgs, mlps, cta_threads, tiles):
        if vec != 1 and (mlp != 8 or thr != 256 or tile):
            continue  # block kernels are built with one gather depth; measured at one CTA size, untiled
        if thr == 64 and lpr == 32 and rpg == 2:
            continue
        if tile and (lpr * vw > tile or thr != 256 or rpg != 4):
            continue  # column ranges narrower than a lane group make no sense; tiles measured at one shape
        if tile and tile < 128 and skew:
            continue  # narrow column ranges re-read A for every range: only the even regimes try them
        base = {"vec_size": vec, "if_split": int(gran > 0), "granularity": gran or None,
                "lanes_per_row": lpr, "vec_width": vw, "rows_per_group": rpg, "cta_threads": thr,
                "gather_batch": mlp, "col_tile": tile, "bucketed": 0}
        yield base
        if skew and gran and vec == 1 and not tile:
            yield dict(base, bucketed=1)  # the same pieces ordered by length


class Layouts:
    """Builds (and caches) the PCSR arrays a candidate needs for one matrix."""

    def __init__(self, m, device):
        self.m, self.dev, self.cache = m, device, {}

    def get(self, vec, gran, bucketed=False):
        key = (vec, gran, bool(bucketed))
        if key in self.cache:
            return self.cache[key]
        m = self.m
        if vec == 1:
            rp, ci, v = m.rowPtr, m.colIdx, m.val
        else:
            if ("b", vec) not in self.cache:
                c = m.to("cpu")
                self.cache["b", vec] = tuple(t.to(self.dev) for t in
                                             ops.bcsr_from_csr(c.rowPtr, c.colIdx, c.val, m.n_cols, vec))
            rp, ci, v = self.cache["b", vec]
        tr = None
        if gran and bucketed:
            rp, ci, v, tr = ops.bucket_pcsr(rp, ci, v, gran)
        elif gran:
            rp, tr = ops.split_csr_device(rp, gran)
        self.cache[key] = (rp, ci, v, tr)
        return self.cache[key]


class Timer:
    """Times candidates on one (matrix, dim): verification against the default plain-CSR product
    first, then back-to-back launches between CUDA events."""

    def __init__(self, m, dim, dev, warmup, iters, layouts=None):
        # matrices far larger than the benchmark's 1.6e7 entries get proportionally fewer timed launches
        iters = max(5, int(iters * min(1.0, 2.0e7 / max(1, m.nnz))))
        self.m, self.dim, self.dev, self.warmup, self.iters = m, dim, dev, warmup, iters
        self.lay = layouts if layouts is not None else Layouts(m, dev)  # PCSR arrays are per matrix, not per dim
        self.B = synth.dense_uniform(m.n_cols, dim, 1000 + dim, dev)
        self.ref = ops.csr_spmm(self.B, m.rowPtr, m.colIdx, m.val, 1, 8)
        # hub rows sum thousands of terms in a different order: the floor grows with the row's length
        ln = (m.rowPtr[1:] - m.rowPtr[:-1]).double()
        self.tol = (1e-5 * self.ref.abs() + 1e-4 * torch.clamp(ln / 256.0, min=1.0)[:, None]).float()
        self.max_row = int(ln.max())

    def ms(self, cand):
        """Milliseconds per launch, or None for a candidate that is not run (hub rows without a
        split) or that the library rejects for this width / layout."""
        try:
            return self._ms(cand)
        except _lib.PspmmError as e:
            if e.code in (_lib.PSPMM_E_UNSUPPORTED, _lib.PSPMM_E_CONFIG):
                return None
            raise

    def _ms(self, cand):
        m, dim = self.m, self.dim
        if not cand.get("if_split") and self.max_row > 4096:
            return None  # one lane group per hub row would take milliseconds
        V = cand.get("vec_size", 1)
        rp, ci, v, tr = self.lay.get(V, cand.get("granularity") if cand.get("if_split") else None,
                                     cand.get("bucketed"))
        nbr = (m.n_rows + V - 1) // V
        out = torch.full((nbr * V, dim), float("nan"), device=self.dev)
        cfg = _lib.make_cfg(**{k: int(cand.get(k, 0) or 0) for k in
                               ("lanes_per_row", "vec_width", "cta_threads", "rows_per_group", "gather_batch",
                                "col_tile", "bucketed")})
        ops.spmm_into(out, self.B, rp, ci, v, target_row=tr, V=V, n_out_rows=nbr, cfg=cfg)
        bad = int(((out[: m.n_rows] - self.ref).abs() > self.tol).sum())
        if bad or bool(torch.isnan(out[: m.n_rows]).any()):
            raise RuntimeError("candidate %s disagrees with the default on dim %d (%d elements)" % (cand, dim, bad))
        return ops.spmm_time_ms(self.B, rp, ci, v, tr, V, cfg=cfg, warmup=self.warmup, iters=self.iters, out=out)


def _load_table(path):
    if path and os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return {"version": 2, "entries": {"spmm": {}}}


def _save_table(path, table, note):
    table["version"] = 2
    table.setdefault("sources", {}).update(note)
    with open(path, "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)


def fit(args):
    dev = torch.device("cuda:0")
    _lib.lib()
    mats = fitting_matrices(args.rows, dev, args.regimes)
    raw, best = [], {}
    t0 = time.time()
    for regime, lst in mats.items():
        lays = {mname: Layouts(m, dev) for mname, m in lst}
        for dim in args.dims:
            agg = {}
            for mname, m in lst:
                tm = Timer(m, dim, dev, args.warmup, args.iters, lays[mname])
                for cand in candidates(dim, regime, args.quick):
                    ms = tm.ms(cand)
                    if ms is None:
                        continue
                    raw.append(dict(cand, regime=regime, matrix=mname, dim=dim, ms=ms))
                    agg.setdefault(json.dumps(cand, sort_keys=True), []).append(ms)
                del tm
            full = {k: v for k, v in agg.items() if len(v) == len(lst)}  # timed on every matrix of the regime
            k = min(full, key=lambda kk: sum(full[kk]))
            e = json.loads(k)
            e["ms_sum"] = sum(full[k])
            best.setdefault(regime, {})[str(dim)] = e
            print("%-14s dim %3d best %s  (%.0f s)" % (regime, dim, e, time.time() - t0), flush=True)
    if args.raw:
        with open(args.raw, "w") as f:
            json.dump({"rows": args.rows, "iters": args.iters, "results": raw}, f)
    if args.table:
        table = _load_table(args.table)
        table.setdefault("entries", {}).setdefault("spmm", {}).update(best)
        _save_table(args.table, table, {"fit:" + ",".join(sorted(best)): "python -m paramspmm_ae_b200.sweep fit, rows=%d "
                                        "iters=%d, back-to-back launches, B200; fitting matrices: %s"
                                        % (args.rows, args.iters, {r: [n for n, _ in l] for r, l in mats.items()})})
    return best


def holdout(args):
    dev = torch.device("cuda:0")
    _lib.lib()
    decider.load_table(args.table)
    rows_out = []
    t0 = time.time()
    for name, m in holdout_matrices(dev, args.scale):
        st = decider.row_stats(m.rowPtr, m.colIdx)
        reg = decider.regime(st)
        lay = Layouts(m, dev)
        for dim in args.dims:
            tm = Timer(m, dim, dev, args.warmup, args.iters, lay)
            plan = decider.choose(st, dim)
            t_ms = tm.ms(dict(plan))
            best = (t_ms, "table")
            n_c = 0
            for cand in candidates(dim, reg):
                ms = tm.ms(cand)
                if ms is None:
                    continue
                n_c += 1
                if ms < best[0]:
                    best = (ms, cand)
            rec = {"matrix": name, "n_rows": m.n_rows, "nnz": m.nnz, "regime": reg,
                   "dim": dim, "table_ms": round(t_ms, 5), "best_ms": round(best[0], 5),
                   "normalised_performance": round(best[0] / t_ms, 4), "candidates": n_c,
                   "table_choice": {k: plan[k] for k in ("if_split", "vec_size", "granularity") if k in plan},
                   "table_kernel": plan.kernel_cfg(),
                   "best": best[1]}
            rows_out.append(rec)
            print("%-20s %-14s dim %3d table %.4f best %.4f  ratio %.3f  (%.0f s)"
                  % (name, reg, dim, t_ms, best[0], best[0] / t_ms, time.time() - t0), flush=True)
            del tm
    ratios = torch.tensor([r["normalised_performance"] for r in rows_out], dtype=torch.float64)
    by_regime = {}
    for r in rows_out:
        by_regime.setdefault(r["regime"], []).append(r["normalised_performance"])
    summary = {"pairs": len(rows_out), "mean_normalised_performance": round(float(ratios.mean()), 4),
               "geomean_normalised_performance": round(float(ratios.log().mean().exp()), 4),
               "worst": round(float(ratios.min()), 4),
               "share_within_5_percent": round(float((ratios >= 0.95).double().mean()), 4),
               "per_regime_mean": {k: round(sum(v) / len(v), 4) for k, v in sorted(by_regime.items())},
               "vec_size_2_best_in": sum(1 for r in rows_out if isinstance(r["best"], dict) and r["best"].get("vec_size") == 2)}
    out = {"what": "table-choice time vs the fastest of the whole candidate space, per (hold-out matrix, dim); "
                   "normalised_performance = best_ms / table_ms (1 = the table picked the fastest); matrices, sizes "
                   "and seeds are disjoint from the fitting set; back-to-back launches, %d iterations, B200" % args.iters,
           "dims": list(args.dims), "summary": summary, "rows": rows_out}
    with open(args.out, "w") as f:
        json.dump(out, f, indent=1)
    print(json.dumps(summary))
    return out


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    here = os.path.dirname(os.path.abspath(__file__))
    table = os.path.join(here, "config_table.json")
    p = sub.add_parser("fit")
    p.add_argument("--rows", type=int, default=1_000_000)
    p.add_argument("--dims", type=int, nargs="*", default=list(range(16, 257, 16)))
    p.add_argument("--regimes", nargs="*", default=ALL_REGIMES)
    p.add_argument("--quick", action="store_true")
    p.add_argument("--raw", default=None, help="write every timing to this file")
    p.add_argument("--table", default=table)
    p = sub.add_parser("holdout")
    p.add_argument("--dims", type=int, nargs="*", default=[16, 32, 64, 128, 256])
    p.add_argument("--scale", type=float, default=1.0, help="shrink the hold-out matrices (quick checks)")
    p.add_argument("--table", default=table)
    p.add_argument("--out", default=os.path.join(here, "decider_holdout.json"))
    for q in sub.choices.values():
        q.add_argument("--iters", type=int, default=20)
        q.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    {"fit": fit, "holdout": holdout}[args.cmd](args)


if __name__ == "__main__":
    main()
