"""Kernel micro-benchmarks: ``python -m ipex_llm_b200.utils.kernel_bench --op gemv --qtype sym_int4 --n 12288 --k 4096``.

Times one op in isolation with CUDA events after warm-up.  The weights are rotated through enough copies to exceed
the 126 MB L2 (``--copies`` overrides), so every timed launch reads its weights from HBM.  Prints one JSON line with
the device time per launch and the achieved weight-streaming bandwidth (or TFLOP/s for GEMM-shaped ops), next to the
measured peaks of the machine when a ``MEASURED_PEAKS.json`` sits in the working directory.

Ops: ``gemv`` (low-bit GEMV, decode), ``gemm`` (low-bit or fp16 GEMM, prefill), ``attn`` (split-KV decode
attention), ``rmsnorm``.  The same command line is what the profiler captures are taken from (``--iters 3
--warmup 1`` keeps those short).
"""
from __future__ import annotations

import argparse
import json

import torch


_GRAPH = False


def _time(fn, iters, warmup):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if _GRAPH:
        # replay `iters` launches from one CUDA graph: removes the host's per-launch cost from the measurement
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e3
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3     # us


def _peaks():
    try:
        with open("MEASURED_PEAKS.json") as f:
            return json.load(f)
    except OSError:
        return {}


def bench_gemv(a):
    from ..ops import cuda_ops
    from ..ops.cuda_quant import quantize_to_device_layout
    from ..quant import qtypes as qt
    q = qt.qtype_from_name(a.qtype)
    dt = torch.float16 if a.dtype == "fp16" else torch.bfloat16
    if a.impl:
        cuda_ops._GEMV_IMPL = a.impl
    ws = []
    for _ in range(2):
        ws.append(quantize_to_device_layout(torch.randn(a.n, a.k, device="cuda", dtype=dt) * 0.02, q))
    wbytes = ws[0].numel() * ws[0].element_size()
    copies = a.copies or max(2, int(300e6 // wbytes) + 1)
    while len(ws) < copies:
        ws.append(ws[len(ws) % 2].clone())
    x = torch.randn(a.m, a.k, device="cuda", dtype=dt)
    out = torch.empty(a.m, a.n, device="cuda", dtype=dt)
    us = _time(lambda i: cuda_ops.gemv_lowbit(x, ws[i % copies], q, a.n, a.k, out=out), a.iters, a.warmup)
    cuda_ops.check_error_flag(x.device)
    return {"op": "gemv", "qtype": a.qtype, "n": a.n, "k": a.k, "m": a.m, "us": us, "weight_bytes": wbytes,
            "gbs": wbytes / us / 1e3, "copies": copies}


def bench_gemm(a):
    from ..ops import cuda_ops
    from ..ops.cuda_quant import quantize_to_device_layout
    from ..quant import qtypes as qt
    dt = torch.float16 if a.dtype == "fp16" else torch.bfloat16
    x = torch.randn(a.m, a.k, device="cuda", dtype=dt)
    flops = 2.0 * a.m * a.n * a.k
    if a.qtype in ("fp16", "bf16"):
        w = torch.randn(a.n, a.k, device="cuda", dtype=dt) * 0.02
        from ..ops import tcgen05_gemm
        out = torch.empty(a.m, a.n, device="cuda", dtype=dt)
        fn = (lambda i: torch.nn.functional.linear(x, w)) if a.impl == "cublas" else \
            (lambda i: tcgen05_gemm.gemm_dense(x, w, out=out))
    else:
        q = qt.qtype_from_name(a.qtype)
        w = quantize_to_device_layout(torch.randn(a.n, a.k, device="cuda", dtype=dt) * 0.02, q)
        fn = lambda i: cuda_ops.gemm_lowbit(x, w, q, a.n, a.k)
    us = _time(fn, a.iters, a.warmup)
    return {"op": "gemm", "qtype": a.qtype, "n": a.n, "k": a.k, "m": a.m, "us": us, "tflops": flops / us / 1e6}


def bench_attn(a):
    from ..ops import cuda_ops
    dt = torch.float16 if a.dtype == "fp16" else torch.bfloat16
    B, Hq, Hkv, S, D = a.batch, a.heads, a.kv_heads, a.kv_len, a.head_dim
    n_sets = a.copies or max(2, int(300e6 // (2 * B * Hkv * S * D * (1 if a.fp8_kv else 2))) + 1)
    n_sets = min(n_sets, 64)
    q = torch.randn(B, Hq, 1, D, device="cuda", dtype=dt)
    if a.fp8_kv:
        ks = [torch.randint(0, 120, (B, Hkv, S, D), device="cuda", dtype=torch.uint8) for _ in range(n_sets)]
    else:
        ks = [torch.randn(B, Hkv, S, D, device="cuda", dtype=dt) for _ in range(n_sets)]
    us = _time(lambda i: cuda_ops.sdpa_decode(q, ks[i % n_sets], ks[(i + 1) % n_sets], None, D ** -0.5, None, None),
               a.iters, a.warmup)
    kvbytes = 2 * B * Hkv * S * D * ks[0].element_size()
    return {"op": "attn", "batch": B, "heads": Hq, "kv_heads": Hkv, "kv_len": S, "head_dim": D, "fp8_kv": a.fp8_kv,
            "us": us, "kv_bytes": kvbytes, "gbs": kvbytes / us / 1e3}


def bench_attn_prefill(a):
    """Causal prompt attention, ``--kv-len`` tokens: the tcgen05 kernel (``--impl tcgen05``, default) or the library
    SDPA (``--impl sdpa``) on the same token-major views of a fused qkv activation."""
    from ..ops import cuda_ops
    dt = torch.float16 if a.dtype == "fp16" else torch.bfloat16
    B, Hq, Hkv, S, D = a.batch, a.heads, a.kv_heads, a.kv_len, a.head_dim
    n_sets = min(16, max(2, int(300e6 // (B * S * (Hq + 2 * Hkv) * D * 2)) + 1))
    sets = []
    for _ in range(n_sets):
        qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device="cuda", dtype=dt)
        sets.append((qkv[:, :, :Hq].transpose(1, 2), qkv[:, :, Hq:Hq + Hkv].transpose(1, 2),
                     qkv[:, :, Hq + Hkv:].transpose(1, 2)))
    scale = D ** -0.5
    if a.impl == "sdpa":
        fn = lambda i: torch.nn.functional.scaled_dot_product_attention(*sets[i % n_sets], is_causal=True,
                                                                        scale=scale, enable_gqa=Hq != Hkv)
    else:
        fn = lambda i: cuda_ops.attn_prefill_tcgen05(*sets[i % n_sets], scale, True)
    us = _time(fn, a.iters, a.warmup)
    cuda_ops.check_error_flag(sets[0][0].device)
    flops = 4.0 * B * Hq * S * S * D / 2          # causal: half of the score matrix
    return {"op": "attn_prefill", "impl": a.impl or "tcgen05", "batch": B, "heads": Hq, "kv_heads": Hkv, "seq": S,
            "head_dim": D, "us": us, "tflops": flops / us / 1e6}


def bench_rmsnorm(a):
    from ..ops import cuda_ops
    dt = torch.float16 if a.dtype == "fp16" else torch.bfloat16
    rows = a.m
    n_sets = max(2, int(300e6 // (rows * a.k * 2)) + 1)
    xs = [torch.randn(rows, a.k, device="cuda", dtype=dt) for _ in range(min(n_sets, 64))]
    g = torch.ones(a.k, device="cuda", dtype=dt)
    us = _time(lambda i: cuda_ops.rms_norm(xs[i % len(xs)], g, 1e-5), a.iters, a.warmup)
    nbytes = 2 * rows * a.k * 2
    return {"op": "rmsnorm", "rows": rows, "k": a.k, "us": us, "gbs": nbytes / us / 1e3}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--op", default="gemv", choices=["gemv", "gemm", "attn", "attn_prefill", "rmsnorm"])
    ap.add_argument("--qtype", default="sym_int4")
    ap.add_argument("--dtype", default="fp16", choices=["fp16", "bf16"])
    ap.add_argument("--impl", default="", help="GEMV implementation override: v1 | tma | direct")
    ap.add_argument("--n", type=int, default=12288)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=32)
    ap.add_argument("--kv-len", type=int, default=1024)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--fp8-kv", action="store_true")
    ap.add_argument("--copies", type=int, default=0)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--graph", action="store_true", help="time a CUDA-graph replay of the launches")
    a = ap.parse_args(argv)
    global _GRAPH
    _GRAPH = a.graph
    if not torch.cuda.is_available():
        raise SystemExit("kernel_bench needs a CUDA device")
    res = {"gemv": bench_gemv, "gemm": bench_gemm, "attn": bench_attn, "attn_prefill": bench_attn_prefill,
           "rmsnorm": bench_rmsnorm}[a.op](a)
    pk = _peaks()
    if "gbs" in res and pk.get("hbm_gbs"):
        res["frac_of_measured_hbm"] = res["gbs"] / pk["hbm_gbs"]
    if "tflops" in res and pk.get("bf16_tflops"):
        res["frac_of_measured_bf16"] = res["tflops"] / pk["bf16_tflops"]
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
