"""Stress run: repeated long generations on one model, logging latency and reserved memory per round
(``python -m ipex_llm_b200.benchmark.stress_test --repo-id synthetic:llama2-7b --rounds 20``; reference
python/llm/dev/benchmark/all-in-one/run-stress-test.py:79-201).  Fails when a round's decode latency or the reserved
memory drifts above the first rounds' by more than the given factors."""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--repo-id", default="synthetic:llama2-7b")
    ap.add_argument("--test-api", default="transformer_int4_fp16_gpu")
    ap.add_argument("--low-bit", default="sym_int4")
    ap.add_argument("--in-out", default="1024-512")
    ap.add_argument("--rounds", type=int, default=20)
    ap.add_argument("--max-latency-drift", type=float, default=1.25)
    ap.add_argument("--max-memory-drift", type=float, default=1.10)
    a = ap.parse_args(argv)
    from .all_in_one import _load
    model, _, device, _ = _load(a.repo_id, a.test_api, a.low_bit, None, False)
    in_len, out_len = (int(v) for v in a.in_out.split("-"))
    ids = torch.randint(3, model.config.vocab_size, (1, in_len)).to(device)
    base_lat = base_mem = None
    ok = True
    for r in range(a.rounds):
        t = time.perf_counter()
        model.generate(ids, max_new_tokens=out_len, min_new_tokens=out_len, do_sample=False)
        if device == "cuda":
            torch.cuda.synchronize()
        total = time.perf_counter() - t
        rest = float(getattr(model, "rest_cost_mean", total / out_len))
        mem = torch.cuda.memory_reserved() / 2 ** 30 if device == "cuda" else 0.0
        if r == 1:                                      # the first pass pays graph capture and allocator growth
            base_lat, base_mem = rest, mem
        drift = base_lat is not None and (rest > base_lat * a.max_latency_drift or
                                          (base_mem and mem > base_mem * a.max_memory_drift))
        ok = ok and not drift
        print(json.dumps({"round": r, "total_s": round(total, 3), "ms_per_token": round(1e3 * rest, 3),
                          "memory_reserved_gib": round(mem, 2), "drift": bool(drift)}))
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
