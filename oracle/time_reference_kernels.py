"""Measurement aid (test infrastructure, not part of the product): times the reference's own CUDA
SpMM kernels, compiled unmodified into oracle/_ref by oracle/build_oracle.py, on the three benchmark
matrices next to this library's kernels.  For every case the reference gets its best of
{csr, csr_split with partition length 32} x CF x blkWarpNum; both sides run 20 back-to-back launches
after 3 warm-ups, no L2 flush (the reference's own protocol, SpMM/SpMM_kernel.cu:564-657).

    python oracle/time_reference_kernels.py          # needs a B200 and oracle/_ref/ParamSpMM_cuda_ref.so
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import build_oracle
from paramspmm_ae_b200 import ops, synth, decider, _lib
ref = build_oracle.load_ref_spmm_cuda()
if ref is None:
    sys.exit("oracle/_ref/ParamSpMM_cuda_ref.so not found: run python oracle/build_oracle.py where the reference tree is mounted")
dev = torch.device('cuda:0')
n = 1_000_000
mats = {"uniform": synth.uniform_rows(n, 16, seed=21, device=dev), "banded": synth.banded_rows(n, 16, 32, seed=22, device=dev),
        "rmat": synth.rmat(20, 16 * n, n=n, seed=23, device=dev)}
def t(fn, it=20):
    for _ in range(3): fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(it): fn()
    b.record(); b.synchronize()
    return a.elapsed_time(b) / it
for dim in (16, 64, 128, 256):
    X = synth.dense_uniform(n, dim, 1000 + dim, dev)
    for name, m in mats.items():
        best = None
        rps, tr = ops.split_csr(m.rowPtr.cpu(), 32); rps, tr = rps.to(dev), tr.to(dev)
        for CF in sorted({1, 2, min(8, (dim + 31) // 32)}):
            if CF * 32 > max(32, dim): continue
            for W in (4, 8):
                ms = t(lambda: ref.csr_spmm(X, m.rowPtr, m.colIdx, m.val, CF, W))
                if best is None or ms < best[0]: best = (ms, 'csr', CF, W)
                ms = t(lambda: ref.csr_split_spmm(X, rps, m.colIdx, m.val, tr, CF, W))
                if ms < best[0]: best = (ms, 'csr_split32', CF, W)
        st = decider.row_stats(m.rowPtr); p = decider.choose(st, dim); cfg = _lib.make_cfg(**p.kernel_cfg())
        C = torch.empty(n, dim, device=dev)
        if p["if_split"]:
            r2, t2 = ops.split_csr(m.rowPtr.cpu(), p["granularity"]); r2, t2 = r2.to(dev), t2.to(dev)
            ours = t(lambda: ops.spmm_into(C, X, r2, m.colIdx, m.val, target_row=t2, n_out_rows=n, cfg=cfg))
        else:
            ours = t(lambda: ops.spmm_into(C, X, m.rowPtr, m.colIdx, m.val, cfg=cfg))
        print(dim, name, 'reference best %.4f ms %s' % (best[0], best[1:]), 'ours %.4f ms' % ours, 'ratio %.2f' % (best[0] / ours), flush=True)
