#!/usr/bin/env python3
"""In-tree build of libpspmm.so (sm_100a only) with nvcc; no torch headers involved.

    python -m paramspmm_ae_b200.build [--force] [--verbose]

Translation units are compiled in parallel; objects land in ``paramspmm_ae_b200/csrc/build``
and the shared library next to the package (``paramspmm_ae_b200/libpspmm.so``).
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(PKG, "libpspmm.so")
BASELINES_LIB = os.path.join(PKG, "libpspmm_baselines.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fopenmp,-fvisibility=hidden",
              "-cudart", "shared", "-I", os.path.join(ROOT, "include"), "-I", CSRC]

CORE_SOURCES = ["pspmm_api.cu", "spmm_vw4.cu", "spmm_vw4_acc.cu", "spmm_vw2.cu", "spmm_vw1.cu", "sddmm_vw4.cu",
                "sddmm_vw2.cu", "sddmm_vw1.cu", "host_builders.cpp", "mtx_io.cpp", "device_builders.cu", "agnn_fused.cu", "exchange.cu"]
BASELINE_SOURCES = ["baselines.cu"]


def _deps(src):
    deps = [os.path.join(CSRC, src), os.path.join(ROOT, "include", "pspmm.h")]
    deps += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    return deps


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src, force, verbose):
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    if not force and not _stale(obj, _deps(src)):
        return obj, ""
    cmd = [NVCC] + ARCH + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else [])
    if src.endswith(".cpp"):
        cmd += ["-x", "cu"]
    cmd += ["-c", os.path.join(CSRC, src), "-o", obj]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise RuntimeError("nvcc failed on %s:\n%s" % (src, p.stdout))
    return obj, p.stdout


def _link(objs, out, extra):
    cmd = [NVCC] + ARCH + ["-shared", "-cudart", "shared", "-Xcompiler", "-fopenmp",
                            "-Xlinker", "-rpath,/usr/local/cuda/lib64"] + objs + extra + ["-o", out]
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise RuntimeError("link failed for %s:\n%s" % (out, p.stdout))


def build(force=False, verbose=False, baselines=True):
    """Compile whatever is stale and return the path of libpspmm.so."""
    os.makedirs(OBJ, exist_ok=True)
    core = [s for s in CORE_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    base = [s for s in BASELINE_SOURCES if baselines and os.path.exists(os.path.join(CSRC, s))]
    logs = []
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        results = list(ex.map(lambda s: _compile(s, force, verbose), core + base))
    objs = [r[0] for r in results]
    logs = [r[1] for r in results if r[1]]
    core_objs, base_objs = objs[: len(core)], objs[len(core):]
    if force or _stale(LIB, core_objs):
        _link(core_objs, LIB, [])
    if base_objs and (force or _stale(BASELINES_LIB, base_objs)):
        _link(base_objs, BASELINES_LIB, ["-lcusparse"])
    if verbose:
        print("\n".join(logs))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
