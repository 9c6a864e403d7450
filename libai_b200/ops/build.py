"""In-tree build of the native extensions: ``libai_b200/_C.so`` (GEMM, attention, norms, optimizer, collectives) and
``libai_b200/_C_seq.so`` (ragged-batch sequence mixers with per-sequence state), ``libai_b200/_C_kv.so`` (ring and paged key/value
caches, masked grouped-query attention, attention with mixed heads, Dynamic-Tanh and post-norm residuals, mixture of experts) and ``libai_b200/_C_lin.so`` (bigram embedding,
hyper-connection streams, decayed linear-attention recurrences).

    python -m libai_b200.ops.build [--force] [--verbose] [--only _C|_C_seq|_C_kv|_C_lin]

CUDA sources are compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a -lineinfo``);
nvcc cross-compiles without a GPU.  Objects are cached under ``libai_b200/csrc/build`` keyed by
source mtime.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "csrc")
BUILD = os.path.join(CSRC, "build")
SO_PATH = os.path.join(ROOT, "_C.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

CU_SOURCES = ["gemm_sm100.cu", "norm.cu", "elementwise.cu", "attention_sm100.cu", "comm_kernels.cu"]
CPP_SOURCES = ["bindings.cpp", "symm_mem.cpp"]
SEQ_SO_PATH = os.path.join(ROOT, "_C_seq.so")
SEQ_CU_SOURCES = ["seq_mixers.cu"]
SEQ_CPP_SOURCES = ["seq_bindings.cpp"]
KV_SO_PATH = os.path.join(ROOT, "_C_kv.so")
KV_CU_SOURCES = ["kv_mixers.cu", "paged_mixers.cu"]
KV_CPP_SOURCES = ["kv_bindings.cpp"]
LIN_SO_PATH = os.path.join(ROOT, "_C_lin.so")
LIN_CU_SOURCES = ["lin_mixers.cu"]
LIN_CPP_SOURCES = ["lin_bindings.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "--use_fast_math", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
# the sequence mixers promise fp32 results exact to rounding: IEEE division / sqrt / exp, no fast-math
SEQ_NVCC_FLAGS = [f for f in NVCC_FLAGS if f != "--use_fast_math"]


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"command failed ({res.returncode}): {' '.join(cmd)}\n{res.stdout}")
    return res.stdout


def _stale(src, obj, deps=()):
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return any(os.path.getmtime(p) > t for p in (src,) + tuple(deps) if os.path.exists(p))


def build(force: bool = False, verbose: bool = False, only=None) -> str:
    """Build the libraries named in ``only`` (default: all), side by side; returns the path of ``_C.so``."""
    libs = [(KV_SO_PATH, KV_CU_SOURCES, KV_CPP_SOURCES, SEQ_NVCC_FLAGS, "_C_kv"),
            (LIN_SO_PATH, LIN_CU_SOURCES, LIN_CPP_SOURCES, SEQ_NVCC_FLAGS, "_C_lin"),
            (SEQ_SO_PATH, SEQ_CU_SOURCES, SEQ_CPP_SOURCES, SEQ_NVCC_FLAGS, "_C_seq"),
            (SO_PATH, CU_SOURCES, CPP_SOURCES, NVCC_FLAGS, "_C")]
    libs = [lib for lib in libs if only is None or lib[4] in only]
    import torch  # noqa: F401  (imported before the threads start: the first import is not thread-safe)
    from torch.utils import cpp_extension  # noqa: F401

    with ThreadPoolExecutor(max_workers=max(1, len(libs))) as ex:
        list(ex.map(lambda lib: _build_lib(*lib, force, verbose), libs))
    return SO_PATH


def _build_lib(SO_PATH, CU_SOURCES, CPP_SOURCES, NVCC_FLAGS, ext_name, force, verbose):
    import torch
    from torch.utils import cpp_extension

    os.makedirs(BUILD, exist_ok=True)
    headers = tuple(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))
    cu = [s for s in CU_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    cpp = [s for s in CPP_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    jobs, objs, logs = [], [], {}
    for s in cu:
        src, obj = os.path.join(CSRC, s), os.path.join(BUILD, s + ".o")
        objs.append(obj)
        if force or _stale(src, obj, headers):
            jobs.append((s, [NVCC, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj]))
    inc = []
    for p in cpp_extension.include_paths(device_type="cuda"):
        inc += ["-isystem", p]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    for s in cpp:
        src, obj = os.path.join(CSRC, s), os.path.join(BUILD, s + ".o")
        objs.append(obj)
        if force or _stale(src, obj, headers):
            jobs.append((s, ["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                             f"-DTORCH_EXTENSION_NAME={ext_name}", *inc, "-I", os.path.join(CUDA_HOME, "include"),
                             "-I", CSRC, "-c", src, "-o", obj]))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for (name, _), out in zip(jobs, ex.map(lambda j: _run(j[1], verbose), jobs)):
                logs[name] = out
        os.makedirs(os.path.join(os.path.dirname(ROOT), "profiles"), exist_ok=True)
        with open(os.path.join(BUILD, f"ptxas{ext_name}.log"), "w") as f:
            for name, out in logs.items():
                f.write(f"==== {name}\n{out}\n")
    if jobs or force or not os.path.exists(SO_PATH):
        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        tmp_so = f"{SO_PATH}.{os.getpid()}.tmp"         # link beside the target, then rename: a reader never sees half a file
        _run(["g++", "-shared", "-o", tmp_so, *objs, f"-L{tlib}", "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda",
              "-ltorch_cuda", f"-L{os.path.join(CUDA_HOME, 'lib64')}", "-lcudart",
              f"-Wl,-rpath,{tlib}", f"-Wl,-rpath,{os.path.join(CUDA_HOME, 'lib64')}"], verbose)
        os.replace(tmp_so, SO_PATH)
    return SO_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--only", action="append", choices=["_C", "_C_seq", "_C_kv", "_C_lin"])
    a = ap.parse_args()
    print(build(a.force, a.verbose, a.only))
