"""In-tree build of the native libraries.

Two shared objects and one executable are produced next to this file:

* ``libipex_quant_core.so``  — C++ host library (quantizers, layout transforms, CPU matmul oracle)
* ``libipex_llm_cuda.so``    — every sm_100a CUDA kernel of the package, plain C ABI launchers
* ``bin/ipex-quantize``      — GGUF -> k-quant GGUF rewriter on the host library (``tools/quantize_main.cpp``)

Both are loaded through ctypes (``ipex_llm_b200.native.lib``).  A content hash of the sources is kept
beside each library so that an unchanged tree is never recompiled (the libraries travel with the
source snapshot to GPU machines, where nothing has to be rebuilt).

Run ``python -m ipex_llm_b200.native.build`` to (re)build; ``--verbose`` prints ptxas resource usage.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
HOST_DIR = os.path.join(HERE, "host")
CUDA_DIR = os.path.join(HERE, "cuda")
OBJ_DIR = os.path.join(HERE, "build")

TOOLS_DIR = os.path.join(HERE, "tools")
BIN_DIR = os.path.join(HERE, "bin")
QUANTIZE_BIN = os.path.join(BIN_DIR, "ipex-quantize")

HOST_LIB = os.path.join(HERE, "libipex_quant_core.so")
CUDA_LIB = os.path.join(HERE, "libipex_llm_cuda.so")

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str | None:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def _hash_files(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _sources(d, exts):
    out = []
    for root, _, files in os.walk(d):
        for f in files:
            if f.endswith(exts):
                out.append(os.path.join(root, f))
    return sorted(out)


def _stamp_ok(lib, digest):
    stamp = lib + ".hash"
    if not (os.path.exists(lib) and os.path.exists(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == digest


def _write_stamp(lib, digest):
    with open(lib + ".hash", "w") as f:
        f.write(digest)


def build_host(force=False, verbose=False):
    srcs = _sources(HOST_DIR, (".cpp",))
    deps = _sources(HOST_DIR, (".cpp", ".h"))
    flags = ["-O3", "-fopenmp", "-fPIC", "-shared", "-std=c++17", "-Wall"]
    digest = _hash_files(deps, " ".join(flags))
    if not force and _stamp_ok(HOST_LIB, digest):
        return HOST_LIB
    cmd = ["g++", *flags, "-o", HOST_LIB, *srcs]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    _write_stamp(HOST_LIB, digest)
    return HOST_LIB


def build_tools(force=False, verbose=False):
    """Stand-alone executables: ``bin/ipex-quantize`` (GGUF -> k-quant GGUF), statically carrying the quant core."""
    srcs = _sources(TOOLS_DIR, (".cpp",)) + _sources(HOST_DIR, (".cpp",))
    deps = srcs + _sources(HOST_DIR, (".h",))
    flags = ["-O3", "-fopenmp", "-std=c++17", "-Wall"]
    digest = _hash_files(deps, " ".join(flags))
    if not force and _stamp_ok(QUANTIZE_BIN, digest):
        return QUANTIZE_BIN
    os.makedirs(BIN_DIR, exist_ok=True)
    cmd = ["g++", *flags, "-o", QUANTIZE_BIN, *srcs]
    if verbose:
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    _write_stamp(QUANTIZE_BIN, digest)
    return QUANTIZE_BIN


def cuda_flags(verbose=False):
    flags = [*NVCC_ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
             "--expt-relaxed-constexpr", "-I", CUDA_DIR]
    if verbose:
        flags += ["-Xptxas", "-v"]
    return flags


def build_cuda(force=False, verbose=False):
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernels")
    srcs = _sources(CUDA_DIR, (".cu",))
    deps = _sources(CUDA_DIR, (".cu", ".cuh", ".h"))
    flags = cuda_flags(verbose)
    digest = _hash_files(deps, " ".join(f for f in flags if f != CUDA_DIR and f != "-v" and f != "-Xptxas"))
    if not force and _stamp_ok(CUDA_LIB, digest):
        return CUDA_LIB
    os.makedirs(OBJ_DIR, exist_ok=True)

    def compile_one(src):
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        # per-file incremental rebuild: hash of this file + every header
        fdig = _hash_files([src] + [d for d in deps if not d.endswith(".cu")], " ".join(flags))
        if not force and os.path.exists(obj) and _stamp_ok(obj, fdig):
            return obj, ""
        cmd = [nvcc, *flags, "-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        _write_stamp(obj, fdig)
        return obj, res.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        results = list(ex.map(compile_one, srcs))
    objs = [o for o, _ in results]
    if verbose:
        for (_, log), s in zip(results, srcs):
            if log:
                print(f"== {os.path.basename(s)}\n{log}")
    cmd = [nvcc, *NVCC_ARCH, "-shared", "-o", CUDA_LIB, *objs, "-lcuda"]
    subprocess.check_call(cmd)
    _write_stamp(CUDA_LIB, digest)
    return CUDA_LIB


def build_all(force=False, verbose=False):
    return build_host(force, verbose), build_tools(force, verbose), build_cuda(force, verbose)


if __name__ == "__main__":
    force = "--force" in sys.argv
    verbose = "--verbose" in sys.argv
    print(build_all(force, verbose))
