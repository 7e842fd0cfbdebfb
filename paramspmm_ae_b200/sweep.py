#!/usr/bin/env python3
"""Measured configuration sweep: the stand-in for the reference's ``profile_engine`` /
``training_data_gen`` (PCSR.py:672-823), which time every <representation, CF, blkWarpNum>
on a matrix collection and label each (matrix, dim) with the fastest.

Here the swept space is that of the sm_100a kernels: PCSR split on/off and partition length,
block height (vec_size 1 or 2), lanes per row (rows per warp), rows per lane group, CTA size.
For every (row-length regime, dim) the fastest configuration is written to a JSON table that
``paramspmm_ae_b200.decider`` loads; all raw timings are kept next to it.

    python -m paramspmm_ae_b200.sweep --out sweep_raw.json --table paramspmm_ae_b200/config_table.json

Each candidate is verified against the plain-CSR result of the default configuration before
it is timed (the reference verifies each candidate against torch.sparse.mm, PCSR.py:759-770).
"""
from __future__ import annotations

import argparse
import itertools
import json
import time

import torch

from . import _lib, decider, ops, synth


def regime_matrices(n, device, which):
    out = {}
    if "short_even" in which:
        out["short_even"] = [("uniform", synth.uniform_rows(n, 16, seed=21, device=device)),
                             ("banded", synth.banded_rows(n, 16, 32, seed=22, device=device))]
    if "short_skewed" in which:
        out["short_skewed"] = [("rmat", synth.rmat(max(1, (n - 1).bit_length()), 16 * n, n=n, seed=23, device=device))]
    if "medium_skewed" in which:
        out["medium_skewed"] = [("powerlaw50", synth.powerlaw_graph(n // 4, (n // 4) * 25, seed=31, device=device))]
    if "long_skewed" in which:
        out["long_skewed"] = [("powerlaw490", synth.powerlaw_graph(232965 if n >= 1_000_000 else n // 8,
                                                                   (232965 if n >= 1_000_000 else n // 8) * 245,
                                                                   seed=41, device=device))]
    return out


VEC1_ONLY = False
CTA_THREADS = (256,)


def candidates(dim, regime, quick):
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
    if skew or long_rows:
        grans = [0, 32, 64, 128] if not long_rows else [0, 64, 128, 256, 512]
    else:
        grans = [0]
    vecs = (1,) if (quick or VEC1_ONLY) else (1, 2)
    tiles = (0, 128) if dim > 128 else (0,)
    for vec, gran, lpr, rpg, mlp, thr, tile in itertools.product(vecs, grans, lprs, rpgs, mlps, CTA_THREADS, tiles):
        if vec != 1 and mlp != 8:
            continue  # block kernels are built with one gather depth
        if tile and (vec != 1 or lpr != 32):
            continue  # column ranges of 128: one 16-byte slice per lane of a full warp
        yield {"vec_size": vec, "if_split": int(gran > 0), "granularity": gran or None,
               "lanes_per_row": lpr, "vec_width": vw, "rows_per_group": rpg, "cta_threads": thr,
               "gather_batch": mlp, "col_tile": tile}


class Layouts:
    """Builds (and caches) the PCSR arrays a candidate needs for one matrix."""

    def __init__(self, m, device):
        self.m, self.dev, self.cache = m, device, {}

    def get(self, vec, gran):
        key = (vec, gran)
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
        if gran:
            rps, tr = ops.split_csr(rp.cpu(), gran)
            rp, tr = rps.to(self.dev), tr.to(self.dev)
        self.cache[key] = (rp, ci, v, tr)
        return self.cache[key]


def run(args):
    global VEC1_ONLY, CTA_THREADS
    VEC1_ONLY = bool(getattr(args, "vec1_only", False))
    CTA_THREADS = tuple(getattr(args, "cta_threads", None) or (256,))
    dev = torch.device("cuda:0")
    _lib.lib()
    which = args.regimes
    mats = regime_matrices(args.rows, dev, which)
    results = []
    best = {}
    t_start = time.time()
    for regime, lst in mats.items():
        for dim in args.dims:
            agg = {}
            for mname, m in lst:
                lay = Layouts(m, dev)
                B = synth.dense_uniform(m.n_cols, dim, 1000 + dim, dev)
                ref = ops.csr_spmm(B, m.rowPtr, m.colIdx, m.val, 1, 8)
                tol = 1e-4 + 1e-5 * ref.abs()
                max_row = int((m.rowPtr[1:] - m.rowPtr[:-1]).max())
                for cand in candidates(dim, regime, args.quick):
                    if not cand["if_split"] and max_row > 4096:
                        continue  # one lane group per hub row would take milliseconds
                    rp, ci, v, tr = lay.get(cand["vec_size"], cand["granularity"])
                    V = cand["vec_size"]
                    nbr = (m.n_rows + V - 1) // V
                    out = torch.empty(nbr * V, dim, device=dev)
                    cfg = _lib.make_cfg(lanes_per_row=cand["lanes_per_row"], vec_width=cand["vec_width"],
                                        cta_threads=cand["cta_threads"], rows_per_group=cand["rows_per_group"],
                                        gather_batch=cand["gather_batch"], col_tile=cand.get("col_tile", 0))
                    ops.spmm_into(out, B, rp, ci, v, target_row=tr, V=V, n_out_rows=nbr, cfg=cfg)
                    # hub rows sum thousands of terms in a different order: scale the floor
                    bad = ((out[: m.n_rows] - ref).abs() > tol * 50).sum().item()
                    if bad:
                        raise RuntimeError("candidate %s disagrees with the default on %s dim %d (%d elements)"
                                           % (cand, mname, dim, bad))
                    ms = ops.spmm_time_ms(B, rp, ci, v, tr, V, cfg=cfg, warmup=args.warmup, iters=args.iters,
                                          out=out)
                    rec = dict(cand, regime=regime, matrix=mname, dim=dim, ms=ms,
                               gflops=2.0 * m.nnz * dim / ms / 1e6)
                    results.append(rec)
                    key = json.dumps(cand, sort_keys=True)
                    agg.setdefault(key, []).append(ms)
                del B, ref
            # fastest candidate by summed time over the regime's matrices
            k = min(agg, key=lambda kk: sum(agg[kk]))
            e = json.loads(k)
            e["ms_sum"] = sum(agg[k])
            best.setdefault(regime, {})[str(dim)] = e
            print("%-14s dim %3d best %s  (%.1f s elapsed)" % (regime, dim, e, time.time() - t_start), flush=True)
    with open(args.out, "w") as f:
        json.dump({"rows": args.rows, "iters": args.iters, "results": results}, f)
    if args.table:
        table = {"version": 1,
                 "source": "python -m paramspmm_ae_b200.sweep, rows=%d iters=%d, back-to-back launches, B200" % (args.rows, args.iters),
                 "entries": {"spmm": best}}
        # regimes that were not measured inherit from the nearest measured one
        with open(args.table, "w") as f:
            json.dump(table, f, indent=1, sort_keys=True)
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=1_000_000)
    ap.add_argument("--dims", type=int, nargs="*", default=list(range(16, 257, 16)))
    ap.add_argument("--regimes", nargs="*", default=["short_even", "short_skewed"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--vec1-only", action="store_true", help="skip the 2 x 1 block layout")
    ap.add_argument("--cta-threads", type=int, nargs="*", default=[256], help="CTA sizes to try (128, 256)")
    ap.add_argument("--out", default="sweep_raw.json")
    ap.add_argument("--table", default=None)
    run(ap.parse_args())


if __name__ == "__main__":
    main()
