#!/usr/bin/env python3
"""Benchmark of the SpMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload ("c2_dim_sweep"): three seeded synthetic 1,000,000 x 1,000,000 CSR matrices with
16 entries per row on average (uniform-random columns, banded with half-bandwidth 32, R-MAT
power-law a=.57 b=c=.19), values U[0,1), dense operand 2U-1, dims 16..256 step 16, fp32.
One step = one pass over all 48 (matrix, dim) SpMMs.  Metric: GFLOP/s = 2*nnz*dim / t summed
over the pass.  Every launch is timed on the device with its own pair of CUDA events and the
L2 cache is flushed (a 256 MiB device memset) before each launch, outside the events; the
step time is the sum of the launch times.  With N > 1 (torchrun, one rank per GPU) every rank
runs the same pass on its own row block of an N-times taller matrix with the dense operand
replicated (no data-path collective); the step time is the maximum over ranks.

Beside `value` the line carries `scaleout`: the strong-scaling times of the row-sharded SpMM of
ONE global R-MAT matrix (2^24 nodes, 5.12e8 entries, dim 128) at this GPU count, with the dense
operand replicated, all-gathered, and exchanged row by row through the pull kernel; the speed-up at
N GPUs is the N = 1 run's figure divided by this one.  `scaleout.scattered_labels` holds the same three
times for the same matrix after a seeded random relabelling of its nodes (P A P^T), which gives every
rank the same share of rows, entries and exchange traffic.

`--impl reference` times the reference's CPU path for the same products, torch.sparse.mm on CSR
tensors on the host (verification.py:44-77 of the reference): one step is the same pass over all
48 (matrix, dim) SpMMs, with all the host threads the process may use.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_ROWS = 1_000_000
NNZ_PER_ROW = 16
DIMS = list(range(16, 257, 16))
MATRICES = ("uniform", "banded", "rmat")
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes of one SpMM (dram__bytes_read.sum + dram__bytes_write.sum of an `ncu` capture at
# 1,000,000 rows, summed over the launches of its column tiles) and the source revision the captured
# library was built from.
NCU_DRAM_BYTES = {
    ("uniform", 64): (3.171e9, "ea49569"), ("banded", 64): (0.605e9, "ea49569"), ("rmat", 64): (0.712e9, "ea49569"),
    ("uniform", 128): (6.272e9, "ea49569"), ("banded", 128): (1.131e9, "ea49569"), ("rmat", 128): (1.908e9, "ea49569"),
    ("uniform", 256): (12.452e9, "ea49569"), ("banded", 256): (2.195e9, "ea49569"), ("rmat", 256): (5.784e9, "ea49569"),
    ("uniform", 240): (15.854e9, "16831dc"), ("banded", 240): (2.056e9, "16831dc"), ("rmat", 240): (5.389e9, "16831dc"),
}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="c2_dim_sweep", choices=["c2_dim_sweep", "c4_agnn_layer", "c3_gcn", "c5_scaleout"],
                    help="c2_dim_sweep is the benchmark proper; the others are one-GPU side measurements")
    ap.add_argument("--rows", type=int, default=N_ROWS, help="rows per matrix (smaller for quick checks)")
    ap.add_argument("--c5-scale", type=int, default=24, help="c5_scaleout: log2 of the node count")
    ap.add_argument("--c5-nnz", type=int, default=512_000_000, help="c5_scaleout: entries of the global matrix")
    ap.add_argument("--dims", type=int, nargs="*", default=DIMS)
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-comparators", action="store_true", help="skip the cuSPARSE timing rows")
    ap.add_argument("--no-scaleout", action="store_true", help="skip the strong-scaling leg (the `scaleout` key)")
    ap.add_argument("--scaleout-iters", type=int, default=5)
    return ap.parse_args()


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def bench_config(n, dims):
    """The workload description both arms print."""
    return {"workload": "c2_dim_sweep", "rows_per_gpu": n, "nnz_per_row": NNZ_PER_ROW,
            "matrices": list(MATRICES), "dims": list(dims), "launches_per_step": 3 * len(dims),
            "l2": "flushed before every launch (256 MiB memset outside the timed events)",
            "sharding": "`value`: every rank runs the pass on its own row block with the dense operand replicated, "
                        "no collective (weak scaling); `scaleout`: one global matrix row-sharded over the ranks "
                        "(strong scaling), dense operand replicated / all-gathered / exchanged"}


def spmm_bytes(n_rows, n_cols, nnz, dim, n_seg=None):
    """Compulsory traffic of one SpMM: every array touched exactly once."""
    b = 4 * (n_rows + 1) + 8 * nnz + 4 * dim * n_cols + 4 * dim * n_rows
    if n_seg is not None:
        b += 4 * (n_seg + 1) + 4 * n_seg - 4 * (n_rows + 1)
    return b


def build_matrices(n, device, seed_shift=0):
    from paramspmm_ae_b200 import synth
    scale = max(1, (n - 1).bit_length())
    nnz = n * NNZ_PER_ROW
    return {
        "uniform": synth.uniform_rows(n, NNZ_PER_ROW, seed=21 + seed_shift, device=device),
        "banded": synth.banded_rows(n, NNZ_PER_ROW, 32, seed=22 + seed_shift, device=device),
        "rmat": synth.rmat(scale, nnz, n=n, seed=23 + seed_shift, device=device),
    }


# ----------------------------------------------------------------------------- clocks
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU every 200 ms through NVML (read only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            }
            get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self._stop_evt.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = get(h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
                self._stop_evt.wait(0.2)
        except Exception as e:  # NVML missing: report that instead of inventing clocks
            self.reasons.add("nvml_unavailable:%s" % type(e).__name__)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


# ----------------------------------------------------------------------------- CPU arms
def use_all_host_threads():
    """torch's intra-op thread count = the cores this process may run on.  Under
    torch.distributed.run the environment carries OMP_NUM_THREADS=1; the CPU arms are timed on one
    rank only, so they take every core of the affinity mask back."""
    import torch
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_spmm_gflops(mats_cpu, dim, seconds, max_iters=50):
    """torch.sparse.mm on CSR tensors on the host, all threads: GFLOP/s over one SpMM per matrix."""
    import torch
    from paramspmm_ae_b200 import synth
    B = synth.dense_uniform(next(iter(mats_cpu.values())).n_cols, dim, 11)
    sps = [torch.sparse_csr_tensor(m.rowPtr, m.colIdx, m.val, size=(m.n_rows, m.n_cols)) for m in mats_cpu.values()]
    flops = sum(2.0 * m.nnz * dim for m in mats_cpu.values())
    for s in sps:
        torch.sparse.mm(s, B)  # warm-up
    t_all, it = 0.0, 0
    while t_all < seconds and it < max_iters:
        t0 = time.perf_counter()
        for s in sps:
            torch.sparse.mm(s, B)
        t_all += time.perf_counter() - t0
        it += 1
    return flops * it / t_all / 1e9, it


def run_reference(args):
    """The reference's CPU implementation of the product on the same workload: one step = the same
    48 SpMMs as the native arm (3 matrices x 16 dims), torch.sparse.mm on CSR tensors."""
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = use_all_host_threads()
    from paramspmm_ae_b200 import synth
    mats = build_matrices(args.rows, "cpu")
    sps = {k: torch.sparse_csr_tensor(m.rowPtr, m.colIdx, m.val, size=(m.n_rows, m.n_cols)) for k, m in mats.items()}
    Bs = {dim: synth.dense_uniform(args.rows, dim, 1000 + dim) for dim in args.dims}
    flops = sum(2.0 * m.nnz * dim for m in mats.values() for dim in args.dims)

    def one_pass():
        for dim in args.dims:
            for name in MATRICES:
                torch.sparse.mm(sps[name], Bs[dim])

    # One full pass takes seconds on the host: one untimed pass warms caches and thread pools, however
    # many warm-up steps the native arm is asked for.
    warm = 1 if args.warmup > 0 else 0
    for _ in range(warm):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one_pass()
    dt = time.perf_counter() - t0
    val = flops * args.steps / dt / 1e9
    sample = ("%d passes over all %d SpMMs of the workload (3 matrices x dims %s, %d rows, 16 nnz/row), "
              "%d untimed pass before them" % (args.steps, 3 * len(args.dims), list(args.dims), args.rows, warm))
    print(json.dumps({
        "impl": "reference", "metric": "SpMM GFLOP/s (2*nnz*dim/t)", "value": val, "unit": "GFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "warmup_passes_run": warm,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(args.rows, args.dims),
        "cpu_baseline": {"value": val, "unit": "GFLOP/s", "cores": cores, "kind": "reference",
                         "sample": sample + "; torch.sparse.mm(CSR) on the host, the reference's CPU path"},
        "e2e": {"value": val, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------- native arm
def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    import torch
    import torch.distributed as dist
    from paramspmm_ae_b200 import _lib, decider, ops, synth

    _lib.lib()  # no CUDA library, no benchmark
    if args.workload == "c5_scaleout":
        from paramspmm_ae_b200 import workloads
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        if world > 1:
            dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local))
        r = workloads.scaleout_spmm(scale=args.c5_scale, nnz=args.c5_nnz, iters=max(3, args.steps), rank=rank,
                                    world=world, device="cuda:%d" % local)
        if rank == 0:
            print(json.dumps({"metric": "row-sharded SpMM GFLOP/s (2*nnz*dim/t), exchange of B included",
                              "value": max(r["allgather_overlapped_gflops"], r["allgather_spmm_gflops"],
                                           r["needed_rows_exchange_spmm_gflops"], r["allgather_pipelined_gflops"],
                                           r["needed_rows_pipelined_gflops"], r["copy_engine_pipelined_gflops"]),
                              "unit": "GFLOP/s", "n_gpus": world,
                              "higher_is_better": True, "scaling": "strong", "dtype": "f32", "data": "synthetic",
                              "config": {"workload": "c5_scaleout", "scale": args.c5_scale, "nnz": r["nnz"],
                                         "dim": r["dim"]}, "detail": r}))
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload != "c2_dim_sweep":
        from paramspmm_ae_b200 import workloads
        if args.workload == "c4_agnn_layer":
            r = workloads.agnn_layer(iters=max(3, args.steps))
            # two products (scores and aggregation) of 2*nnz*dim flop each, on the fused kernel with
            # the edge softmax; the separate-kernel composition is in detail.layer_sddmm_scale_spmm_ms
            line = {"metric": "AGNN layer (SDDMM, scale, edge softmax, SpMM) GFLOP/s (2 x 2*nnz*dim / t)",
                    "value": 2 * 2.0 * r["nnz"] * r["dim"] / r["fused_softmax_best_ms"] / 1e6, "unit": "GFLOP/s"}
        else:
            r = workloads.gcn_forward_backward(iters=max(2, min(args.steps, 5)))
            line = {"metric": "GCN 3-layer forward+backward ms/step", "value": r["ms_per_step"], "unit": "ms",
                    "higher_is_better": False}
        line.update({"n_gpus": 1, "dtype": "f32", "data": "synthetic", "config": {"workload": args.workload}, "detail": r})
        print(json.dumps(line))
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group(backend="nccl", device_id=dev)
    n = args.rows
    dims = args.dims

    # ---- inputs, resident in HBM before any timing starts
    mats = build_matrices(n, dev, seed_shift=100 * rank)
    plans, runners, shared = {}, {}, {}
    for name, m in mats.items():
        st = decider.row_stats(m.rowPtr, m.colIdx)
        for dim in dims:
            p = plans[name, dim] = decider.choose(st, dim)
            # one set of layout arrays per (matrix, layout), shared by the dims that use it
            key = (name, int(p["if_split"]), p.get("granularity"), int(p.get("bucketed", 0)))
            if key not in shared:
                shared[key] = decider.PlannedSpMM(p, m.rowPtr, m.colIdx, m.val)
            base = shared[key]
            r = runners[name, dim] = decider.PlannedSpMM.__new__(decider.PlannedSpMM)
            r.__dict__.update(base.__dict__)
            r.plan = p
    Bs = {dim: synth.dense_uniform(n, dim, 1000 + dim, dev) for dim in dims}
    Cs = {dim: torch.empty(n, dim, device=dev) for dim in dims}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    cases = [(name, dim) for dim in dims for name in MATRICES]

    def launch(name, dim):
        r = runners[name, dim]
        r(Cs[dim], Bs[dim])
        return r.launches

    def one_pass(events=None):
        launches = 0
        for i, (name, dim) in enumerate(cases):
            flush.zero_()  # evict L2 (outside the timed events)
            if events is not None:
                events[i][0].record()
            launches += launch(name, dim)
            if events is not None:
                events[i][1].record()
        return launches

    for _ in range(max(3, args.warmup)):
        one_pass()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local)
    sampler.start()
    evs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in cases]
           for _ in range(args.steps)]
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    launches = 0
    for s in range(args.steps):
        launches += one_pass(evs[s])
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    per_case = [[evs[s][i][0].elapsed_time(evs[s][i][1]) for s in range(args.steps)] for i in range(len(cases))]
    mean_ms = [sum(x) / len(x) for x in per_case]
    step_ms = sum(mean_ms)
    t = torch.tensor([step_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.barrier()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms_max = float(t.item())
    flops_step = sum(2.0 * mats[name].nnz * dim for name, dim in cases)
    value = world * flops_step / (step_ms_max * 1e-3) / 1e9

    # ---- roofline of the launch that takes the largest share of the pass
    peak, peak_kind = measured_peak()
    sweep = []
    for (name, dim), ms in zip(cases, mean_ms):
        p = plans[name, dim]
        n_seg = runners[name, dim].n_seg if p["if_split"] else None
        by = spmm_bytes(n, n, mats[name].nnz, dim, n_seg)
        sweep.append({"matrix": name, "dim": dim, "ms": round(ms, 5),
                      "gflops": round(2.0 * mats[name].nnz * dim / ms / 1e6, 1),
                      "gbs": round(by / ms / 1e6, 1), "frac": round(by / ms / 1e6 / peak, 4),
                      "split": int(p["if_split"]), "bucketed": int(p.get("bucketed", 0))})

    def roofline_of(i):
        r = {"bound": "hbm", "achieved": sweep[i]["gbs"], "peak": peak, "unit": "GB/s", "frac": sweep[i]["frac"],
             "traffic": None, "peak_source": peak_kind,
             "kernel": "spmm_seg_kernel %s dim=%d" % (sweep[i]["matrix"], sweep[i]["dim"]),
             "ms": sweep[i]["ms"],
             "bytes_model": "4(n+1)+8nnz+4*dim*n_cols+4*dim*n_rows (+8S for a split layout)"}
        key = (sweep[i]["matrix"], sweep[i]["dim"])
        if n == N_ROWS and key in NCU_DRAM_BYTES:
            tb, rev = NCU_DRAM_BYTES[key]
            algo = sweep[i]["gbs"] * sweep[i]["ms"] * 1e6
            r["traffic"] = tb
            r["traffic_source"] = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this case, "
                                   "library built from revision %s" % rev)
            r["traffic_over_algorithmic"] = round(tb / algo, 2)
            # the same launch measured on the bytes it actually moves
            r["traffic_gbs"] = round(tb / mean_ms[i] / 1e6, 1)
            r["traffic_frac"] = round(tb / mean_ms[i] / 1e6 / peak, 4)
        return r

    top = max(range(len(cases)), key=lambda i: mean_ms[i])
    roofline = roofline_of(top)
    roofline["best_frac"] = max(s["frac"] for s in sweep)
    roofline["rmat_dim_ge_64_frac"] = [s["frac"] for s in sweep if s["matrix"] == "rmat" and s["dim"] >= 64]
    # the power-law case at dim 128, and how close the two gather-bound launches come to the rate at
    # which this GPU can fetch their rows at all (the bare gather of the same column stream, timed here)
    roofline_rmat, gather = None, None
    if ("rmat", 128) in cases:
        roofline_rmat = roofline_of(cases.index(("rmat", 128)))
    if rank == 0 and not args.no_comparators:
        try:
            from paramspmm_ae_b200 import baselines
            gather = []
            for key in sorted({("rmat", 128), (sweep[top]["matrix"], sweep[top]["dim"])}):
                if key not in cases or key[1] % 4 != 0:
                    continue
                m, ms = mats[key[0]], mean_ms[cases.index(key)]
                flush.zero_()
                floor_ms = baselines.gather_ceiling_ms(m.colIdx, Bs[key[1]], warmup=2, iters=5)
                gb = 4.0 * key[1] * m.nnz
                gather.append({"matrix": key[0], "dim": key[1], "gathered_bytes": gb,
                               "spmm_gather_gbs": round(gb / ms / 1e6, 1),
                               "bare_gather_gbs": round(gb / floor_ms / 1e6, 1), "bare_gather_ms": round(floor_ms, 5),
                               "frac_of_bare_gather": round(floor_ms / ms, 4)})
        except Exception as e:
            gather = {"unavailable": "%s: %s" % (type(e).__name__, e)}

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region
    e2e = None
    if not args.no_e2e and args.e2e_steps > 0:
        hostA = {name: [t.cpu().pin_memory() for t in (m.rowPtr, m.colIdx, m.val)] for name, m in mats.items()}
        maxd = max(dims)
        hostB = torch.empty(n * maxd, dtype=torch.float32).pin_memory()
        hostB.copy_(synth.dense_uniform(n, maxd, 7).reshape(-1))
        hostC = torch.empty(n * maxd, dtype=torch.float32).pin_memory()
        h2d = d2h = 0

        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        s_comp = torch.cuda.current_stream()
        Bdev = [torch.empty(n * maxd, dtype=torch.float32, device=dev) for _ in range(2)]

        def e2e_pass():
            """Host buffers in, host buffer out, copies and kernels pipelined over three streams:
            the sparse arrays of a matrix cross the bus once per pass, the dense operand of a width
            once per width, every result goes back; copy-in of the next width and copy-out of the
            previous result overlap the running product."""
            nonlocal h2d, d2h
            h2d = d2h = 0
            s_in.wait_stream(s_comp)
            s_out.wait_stream(s_comp)
            devA, evA = {}, {}
            with torch.cuda.stream(s_in):
                for name in MATRICES:
                    devA[name] = [t.to(dev, non_blocking=True) for t in hostA[name]]
                    evA[name] = torch.cuda.Event()
                    evA[name].record(s_in)
                    h2d += sum(t.numel() * t.element_size() for t in hostA[name])
            b_free = [None, None]  # last product that read Bdev[slot]
            outs = []
            for di, dim in enumerate(dims):
                slot = di % 2
                with torch.cuda.stream(s_in):
                    if b_free[slot] is not None:
                        s_in.wait_event(b_free[slot])
                    X = Bdev[slot][: n * dim].view(n, dim)
                    X.copy_(hostB[: n * dim].view(n, dim), non_blocking=True)
                    evB = torch.cuda.Event()
                    evB.record(s_in)
                    h2d += n * dim * 4
                s_comp.wait_event(evB)
                for name in MATRICES:
                    s_comp.wait_event(evA[name])
                    rp, ci, v = devA[name]
                    out = ops.csr_spmm(X, rp, ci, v, 1, 8)
                    done = torch.cuda.Event()
                    done.record(s_comp)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(done)
                        hostC[: n * dim].view(n, dim).copy_(out, non_blocking=True)
                    out.record_stream(s_out)
                    outs.append(out)
                    d2h += n * dim * 4
                b_free[slot] = torch.cuda.Event()
                b_free[slot].record(s_comp)
            for name in MATRICES:
                for t in devA[name]:
                    t.record_stream(s_comp)
            s_comp.wait_stream(s_out)
            s_comp.wait_stream(s_in)
            torch.cuda.synchronize()

        e2e_pass()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.e2e_steps):
            e2e_pass()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / args.e2e_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e = {"value": world * flops_step / (float(t.item()) * 1e-3) / 1e9, "unit": "GFLOP/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": args.e2e_steps,
               "call": "ParamSpMM.csr_spmm on device copies of pinned host CSR arrays (once per matrix and pass) "
                       "and B (once per width and pass); every result copied back to pinned host memory; "
                       "copies and kernels pipelined over three streams"}

    # ---- cuSPARSE on the same GPU, same inputs (reported next to the kernels; rank 0, N = 1 only)
    comparators = None
    if rank == 0 and world == 1 and not args.no_comparators:
        try:
            from paramspmm_ae_b200 import baselines
            rows = []
            for dim in [d for d in (16, 64, 128, 256) if d in dims]:
                for name in MATRICES:
                    m = mats[name]
                    ours = mean_ms[cases.index((name, dim))]
                    mine = per_case[cases.index((name, dim))]
                    rec = {"matrix": name, "dim": dim, "ours_ms": round(ours, 5),
                           "ours_ms_min_max": [round(min(mine), 5), round(max(mine), 5)]}
                    for label, fmt in (("cusparse_csr_default", 0), ("cusparse_csr_alg2", 1)):
                        plan = baselines.spmm_plan(fmt, m.rowPtr, m.colIdx, m.val, Bs[dim], Cs[dim])
                        runs = [baselines.time_plan_ms(plan, warmup=3 if i == 0 else 0, iters=20) for i in range(3)]
                        plan.close()
                        rec[label + "_ms"] = round(min(runs), 5)  # the fastest of three blocks of 20 launches
                        rec[label + "_ms_max"] = round(max(runs), 5)
                    rec["gespmm_ms"] = round(baselines.gespmm_time_ms(Bs[dim], m.rowPtr, m.colIdx, m.val, warmup=3, iters=20), 5)
                    rec["speedup_vs_best_cusparse"] = round(min(rec["cusparse_csr_default_ms"], rec["cusparse_csr_alg2_ms"]) / ours, 3)
                    rows.append(rec)
            sp = [r["speedup_vs_best_cusparse"] for r in rows]
            comparators = {"note": "cusparseSpMM fp32 CSR, row-major B/C, plan and workspace created outside the loop, "
                                   "fastest of three blocks of 20 back-to-back launches without L2 flush (our column is the mean over "
                                   "the timed steps, L2 flushed before every launch): favours cuSPARSE; "
                                   "gespmm = this library's restatement of the published GE-SpMM algorithm, same protocol",
                           "geomean_speedup_vs_best_cusparse": round(float(torch.tensor(sp).log().mean().exp()), 3),
                           "rows": rows}
        except Exception as e:
            comparators = {"unavailable": "%s: %s" % (type(e).__name__, e)}

    # ---- CPU baseline on the host cores (rank 0, N = 1 only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cores = use_all_host_threads()
        mats_cpu = {k: m.to("cpu") for k, m in mats.items()}
        g, it = cpu_spmm_gflops(mats_cpu, 64, args.cpu_seconds)
        cpu = {"value": g, "unit": "GFLOP/s", "cores": cores, "kind": "reference",
               "sample": "%d passes of one SpMM per matrix (3 matrices, %d rows, 16 nnz/row) at dim 64 with "
                         "torch.sparse.mm(CSR) on the host, the reference's CPU path (verification.py:44-77)" % (it, n)}

    # ---- strong scaling of one global matrix over the ranks (BASELINE's scale-out configuration)
    scaleout = None
    if not args.no_scaleout:
        from paramspmm_ae_b200 import workloads
        del Bs, Cs, mats, runners, shared, flush
        torch.cuda.empty_cache()
        try:
            r = workloads.scaleout_brief(scale=args.c5_scale, nnz=args.c5_nnz, iters=args.scaleout_iters, rank=rank,
                                         world=world, device="cuda:%d" % local)
            flop = 2.0 * r["nnz"] * r["dim"]
            gf = lambda ms: round(flop / ms / 1e6, 1)
            scaleout = {"workload": "c5_scaleout: R-MAT 2^%d nodes, %d entries, dim %d, rows of A in contiguous blocks "
                                    "balanced by nnz, one block per GPU" % (args.c5_scale, r["nnz"], r["dim"]),
                        "scaling": "strong", "n_gpus": world,
                        "replicated_ms": r["replicated_ms"], "allgather_ms": r["allgather_ms"],
                        "exchange_ms": r["exchange_ms"],
                        "replicated_gflops": gf(r["replicated_ms"]), "allgather_gflops": gf(r["allgather_ms"]),
                        "exchange_gflops": gf(r["exchange_ms"]),
                        "exchange_form": "rows referenced by the shard only, fetched from the owners' peer-mapped blocks "
                                         "by the pull kernel: %s (transport %s)" % (r["exchange_form"], r["transport"]),
                        "detail": r}
            # the same matrix with its nodes relabelled by a seeded random permutation (P A P^T): equal rows,
            # entries and exchange traffic per rank instead of the nnz-balanced blocks of the natural order
            # (at one GPU it is the baseline of that curve)
            torch.cuda.empty_cache()
            try:
                ri = workloads.scaleout_brief(scale=args.c5_scale, nnz=args.c5_nnz, iters=args.scaleout_iters,
                                              rank=rank, world=world, device="cuda:%d" % local,
                                              labels="scattered", legs=False)
                scaleout["scattered_labels"] = {
                    "what": "same global matrix, nodes relabelled by a seeded random permutation before sharding "
                            "(shard.scattered_labels); same product up to the order of rows",
                    "replicated_ms": ri["replicated_ms"], "allgather_ms": ri["allgather_ms"],
                    "exchange_ms": ri["exchange_ms"], "exchange_gflops": gf(ri["exchange_ms"]),
                    "exchange_form": ri["exchange_form"], "detail": ri}
            except Exception as e:
                scaleout["scattered_labels"] = {"unavailable": "%s: %s" % (type(e).__name__, e)}
        except Exception as e:  # the headline number must not depend on this leg
            scaleout = {"unavailable": "%s: %s" % (type(e).__name__, e)}

    if rank == 0:
        print(json.dumps({
            "metric": "SpMM GFLOP/s (2*nnz*dim/t)", "value": value, "unit": "GFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": step_ms_max,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": bench_config(n, dims),
            "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
            "roofline_rmat": roofline_rmat, "gather": gather, "scaleout": scaleout,
            "cpu_baseline": cpu, "comparators": comparators, "wall_ms_per_step_incl_flush": wall / args.steps * 1e3, "sweep": sweep,
        }))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
