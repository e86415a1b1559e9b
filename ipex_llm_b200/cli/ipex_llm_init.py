"""``ipex-llm-init``: print the environment a run should start with, for ``source <(ipex-llm-init --gpu)``.

Reference: python/llm/scripts/ipex-llm-init (a bash script that LD_PRELOADs tcmalloc / jemalloc and Intel OpenMP,
sets ``OMP_NUM_THREADS`` to the physical core count and exports the SYCL / oneCCL variables of its GPUs).  Here the
accelerator side is CUDA / NCCL: one connection per device so that graph replays and copies do not interleave,
NVLS on for the library collectives, a rendezvous address that always resolves, and the host-side allocator /
thread settings of the original.
"""
from __future__ import annotations

import argparse
import glob
import os
import sys


def _find(patterns):
    for pat in patterns:
        hits = sorted(glob.glob(pat))
        if hits:
            return hits[0]
    return None


def settings(gpu: bool, tcmalloc: bool, jemalloc: bool, threads: int = None) -> dict:
    env = {}
    cores = threads or max(1, (os.cpu_count() or 2) // 2)
    env["OMP_NUM_THREADS"] = str(cores)
    env["TOKENIZERS_PARALLELISM"] = "false"
    if gpu:
        env["CUDA_DEVICE_MAX_CONNECTIONS"] = "1"
        env["NCCL_NVLS_ENABLE"] = "1"
        env["TORCH_NCCL_ASYNC_ERROR_HANDLING"] = "1"
        env["MASTER_ADDR"] = "127.0.0.1"
        env["IPEX_LLM_QUANTIZE_KV_CACHE"] = os.environ.get("IPEX_LLM_QUANTIZE_KV_CACHE", "1")
    lib = None
    if jemalloc:
        lib = _find(["/usr/lib/*/libjemalloc.so*", "/usr/local/lib/libjemalloc.so*"])
        if lib:
            env["MALLOC_CONF"] = "oversize_threshold:1,background_thread:true,metadata_thp:auto"
    elif tcmalloc:
        lib = _find(["/usr/lib/*/libtcmalloc.so*", "/usr/lib/*/libtcmalloc_minimal.so*", "/usr/local/lib/libtcmalloc.so*"])
    if lib:
        prev = os.environ.get("LD_PRELOAD", "")
        env["LD_PRELOAD"] = f"{lib}:{prev}" if prev else lib
    return env


def main(argv=None):
    ap = argparse.ArgumentParser(prog="ipex-llm-init", description=__doc__.split("\n")[0])
    ap.add_argument("-g", "--gpu", action="store_true", help="settings for CUDA / NCCL runs")
    ap.add_argument("-c", "--cpu", action="store_true", help="host-only settings (default when --gpu is absent)")
    ap.add_argument("-t", "--tcmalloc", action="store_true", help="preload tcmalloc when it is installed")
    ap.add_argument("-j", "--jemalloc", action="store_true", help="preload jemalloc when it is installed")
    ap.add_argument("--threads", type=int, default=None)
    a = ap.parse_args(argv)
    for k, v in settings(a.gpu, a.tcmalloc, a.jemalloc, a.threads).items():
        print(f"export {k}={v}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
