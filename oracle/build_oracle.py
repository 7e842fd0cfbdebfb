#!/usr/bin/env python3
"""Build recipe for the CPU oracle (test infrastructure, never part of the product).

Two targets:

* ``build_oracle()``  -> ``oracle/liboracle.so`` from ``oracle/pspmm_oracle.c``
  (gcc, OpenMP).  Always possible.

* ``build_ref()``     -> ``oracle/_ref/ParamSpMM_ref.so``: the HOST side of the
  reference's own ``SpMM/SpMM.cpp`` (its ``split_csr`` / ``split_csr_par``
  PCSR partition builders, SpMM.cpp:15-75), compiled with g++ from the source
  where it lies in the mounted reference tree.  Nothing is copied: only the
  shared object lands in ``oracle/_ref/`` (git-ignored).  The CUDA launchers
  that file refers to (``*_cuda<CF,W>``, cuSPARSE and GE-SpMM wrappers) live
  in the reference's ``.cu`` files, which are not compiled here; each such
  undefined symbol is satisfied by a generated stub that aborts if ever
  called, so the module loads and its two CPU functions can be used to pin
  the oracle's restatement.  Skipped silently when the reference tree is not
  mounted (e.g. on a GPU box).

* ``build_ref_sddmm()`` -> ``oracle/_ref/ParamSDDMM_ref.so``: the reference's
  complete SDDMM extension (``SDDMM/sddmm.cpp``, ``sddmm_kernel.cu``,
  ``sddmm_baseline_kernel.cu``), compiled unmodified with nvcc for sm_100a from
  the sources where they lie and linked against the installed libtorch and
  cuSPARSE.  It needs a GPU to run: the GPU tests import it (when the file
  travelled with the tree) to pin the oracle's SDDMM and ``genmask``
  restatements against the reference's own CUDA kernels.  About three minutes.

* ``build_ref_spmm_cuda()`` -> ``oracle/_ref/ParamSpMM_cuda_ref.so``: the
  reference's complete SpMM extension (``SpMM/SpMM.cpp``, ``SpMM_kernel.cu``,
  ``Baseline_kernel.cu``), sources unmodified.  They dispatch on the deprecated
  ``Tensor::type()``, whose ATen overload newer torch releases removed;
  ``oracle/torch_compat_shim.h`` (force-included) restores that one overload.
  About seven minutes.  (The SpCONV extension is the same kernels behind a
  GEMM and is not built.)
"""
from __future__ import annotations

import os
import re
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
# The reference checkout: PSPMM_REFERENCE_ROOT, else a directory named "reference" beside this
# repository's own directory.  Where neither exists everything built from it is skipped.
REF_ROOT = os.environ.get("PSPMM_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
REF_OUT = os.path.join(HERE, "_ref")


def _run(cmd):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(cmd), proc.stdout))
    return proc.stdout


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "pspmm_oracle.c")
    out = os.path.join(HERE, "liboracle.so")
    if not force and _newer(out, [src]):
        return out
    _run(["gcc", "-O2", "-fopenmp", "-fvisibility=hidden", "-shared", "-fPIC", "-std=c11",
          src, "-o", out])
    return out


def ref_available():
    return os.path.isfile(os.path.join(REF_ROOT, "SpMM", "SpMM.cpp"))


def build_ref(force=False):
    """Compile the reference's SpMM.cpp host code into oracle/_ref (see module docstring)."""
    if not ref_available():
        return None
    src = os.path.join(REF_ROOT, "SpMM", "SpMM.cpp")
    out = os.path.join(REF_OUT, "ParamSpMM_ref.so")
    if not force and os.path.exists(out):
        return out
    import torch  # noqa: F401  (only to locate headers / libs)
    from torch.utils import cpp_extension as ce

    os.makedirs(REF_OUT, exist_ok=True)
    obj = os.path.join(REF_OUT, "SpMM_host.o")
    incs = []
    for p in ce.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include",
                                   os.path.join(REF_ROOT, "SpMM")]:
        incs += ["-I", p]
    _run(["g++", "-O2", "-fopenmp", "-fPIC", "-std=c++17", "-c",
          "-DTORCH_EXTENSION_NAME=ParamSpMM_ref", "-DTORCH_API_INCLUDE_EXTENSION_H"]
         + incs + [src, "-o", obj])
    # Symbols that only the reference's .cu files define.
    undefined = [ln.split()[-1] for ln in _run(["nm", "-u", obj]).splitlines() if ln.strip()]
    gpu_only = [s for s in undefined if re.search(r"_cuda|cusparse_|gespmm_", s)]
    stub_s = os.path.join(REF_OUT, "gpu_stubs.s")
    with open(stub_s, "w") as f:
        f.write("\t.text\n")
        for s in gpu_only:
            f.write("\t.globl %s\n\t.type %s,@function\n%s:\n\tcall abort@PLT\n" % (s, s, s))
        f.write('\t.section .note.GNU-stack,"",@progbits\n')
    libdir = ce.library_paths()[0]
    _run(["g++", "-shared", "-fopenmp", obj, stub_s, "-o", out, "-L", libdir,
          "-Wl,-rpath," + libdir, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python"])
    os.remove(obj)
    return out


_REF_EXTENSIONS = {
    # module name -> (directory in the reference tree, sources, needs the ATen compatibility shim)
    "ParamSDDMM_ref": ("SDDMM", ("sddmm_kernel.cu", "sddmm_baseline_kernel.cu", "sddmm.cpp"), False),
    "ParamSpMM_cuda_ref": ("SpMM", ("SpMM_kernel.cu", "Baseline_kernel.cu", "SpMM.cpp"), True),
}


def build_ref_extension(module, force=False):
    """Compile one of the reference's torch extensions (host + CUDA, unmodified, from where the
    sources lie) for sm_100a into oracle/_ref/<module>.so.  The SpMM sources dispatch on the
    deprecated ``Tensor::type()``; ``oracle/torch_compat_shim.h`` is force-included to restore the
    ATen overload they rely on."""
    sub, names, shim = _REF_EXTENSIONS[module]
    src_dir = os.path.join(REF_ROOT, sub)
    sources = [os.path.join(src_dir, f) for f in names]
    if not all(os.path.isfile(f) for f in sources):
        return None
    out = os.path.join(REF_OUT, module + ".so")
    if not force and os.path.exists(out):
        return out
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(REF_OUT, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    incs = []
    for p in ce.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include", src_dir]:
        incs += ["-I", p]
    defs = ["-DTORCH_EXTENSION_NAME=" + module, "-DTORCH_API_INCLUDE_EXTENSION_H",
            "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    if shim:
        defs += ["-include", os.path.join(HERE, "torch_compat_shim.h")]
    objs = []
    for f in sources:
        obj = os.path.join(REF_OUT, module + "." + os.path.basename(f) + ".o")
        if f.endswith(".cu"):
            _run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O1", "-std=c++17", "-Xcompiler",
                  "-fPIC,-fopenmp", "--expt-relaxed-constexpr", "-c"] + defs + incs + [f, "-o", obj])
        else:
            _run(["g++", "-O2", "-fopenmp", "-fPIC", "-std=c++17", "-c"] + defs + incs + [f, "-o", obj])
        objs.append(obj)
    libdir = ce.library_paths()[0]
    _run(["g++", "-shared", "-fopenmp"] + objs + ["-o", out, "-L", libdir, "-Wl,-rpath," + libdir,
          "-L/usr/local/cuda/lib64", "-Wl,-rpath,/usr/local/cuda/lib64", "-ltorch", "-ltorch_cpu", "-ltorch_cuda",
          "-lc10", "-lc10_cuda", "-ltorch_python", "-lcudart", "-lcusparse"])
    for o in objs:
        os.remove(o)
    return out


def build_ref_sddmm(force=False):
    return build_ref_extension("ParamSDDMM_ref", force)


def build_ref_spmm_cuda(force=False):
    return build_ref_extension("ParamSpMM_cuda_ref", force)


def load_ref_extension(module):
    """Import a compiled reference extension, or return None when it is not there."""
    path = os.path.join(REF_OUT, module + ".so")
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded first)

    spec = importlib.util.spec_from_file_location(module, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_ref_sddmm():
    return load_ref_extension("ParamSDDMM_ref")


def load_ref_spmm_cuda():
    return load_ref_extension("ParamSpMM_cuda_ref")


def load_ref():
    """Import the compiled reference host module, or return None when it is not there."""
    path = os.path.join(REF_OUT, "ParamSpMM_ref.so")
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded first)

    spec = importlib.util.spec_from_file_location("ParamSpMM_ref", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


# The reference's Python layers, run unmodified on top of the drop-in extension modules by
# tests/test_gpu_reference_python.py.  They cannot be imported from the reference checkout on a
# machine that does not have it, so they are staged (copied as they are, never edited, never
# committed: the directory is git-ignored like oracle/_ref) next to the other reference-derived
# artefacts; the staging directory travels with the tree.
PY_STAGE = os.path.join(os.path.dirname(HERE), "baseline", "_ref")
# (GNN.py parses the command line when imported, so it cannot be used as a module and is not staged)
_PY_FILES = ("PCSR.py", "SDDMM.py", "gnn_conv.py", "graph_input.py", "verification.py", "decider.py")
_PY_DATA = (os.path.join("toy_dataset", "pubmed.mtx"),)


def stage_reference_python(force=False):
    """Copy the reference's Python layers and its toy matrix into baseline/_ref (returns the
    directory, or None when the reference checkout is absent)."""
    if not ref_available():
        return None
    import shutil

    for rel in _PY_FILES + _PY_DATA:
        src, dst = os.path.join(REF_ROOT, rel), os.path.join(PY_STAGE, rel)
        if not os.path.isfile(src):
            continue
        if force or not os.path.exists(dst) or os.path.getmtime(dst) < os.path.getmtime(src):
            os.makedirs(os.path.dirname(dst), exist_ok=True)
            shutil.copyfile(src, dst)
    return PY_STAGE


def staged_reference_python():
    """The staging directory when it holds the reference's layers, else None."""
    return PY_STAGE if os.path.isfile(os.path.join(PY_STAGE, "PCSR.py")) else None


if __name__ == "__main__":
    print(stage_reference_python(force="--force" in sys.argv))
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
    print(build_ref_sddmm(force="--force" in sys.argv))
    print(build_ref_spmm_cuda(force="--force" in sys.argv))
