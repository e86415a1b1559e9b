"""All-in-one latency benchmark: ``python -m ipex_llm_b200.benchmark.all_in_one [config.yaml]``.

Counterpart of python/llm/dev/benchmark/all-in-one/run.py:63-143 (timed ``generate`` in a loop), :145-205
(``test_api`` dispatch) and :599-601 (the CSV schema), driven by the same YAML keys as its ``config.yaml``
(``repo_id``, ``local_model_hub``, ``warm_up``, ``num_trials``, ``num_beams``, ``low_bit``, ``batch_size``,
``in_out_pairs``, ``test_api``, ``cpu_embedding``, ``streaming``).  A ``repo_id`` of the form ``synthetic:<arch>``
(``llama2-7b``, ``llama2-13b``, ``tiny``) builds a random-init model of that architecture, which is what runs where
no checkpoints exist; the prompt is then random token ids of the requested length.

test_api values served here: ``transformer_int4_gpu`` (fp32 activations in the reference, fp16 here),
``transformer_int4_fp16_gpu``, ``optimize_model_gpu``, ``bigdl_fp16_gpu``, ``speculative_gpu``,
``pipeline_parallel_gpu`` (under ``torchrun``), ``transformer_int4`` and ``optimize_model`` (CPU).
"""
from __future__ import annotations

import csv
import sys
import time
from datetime import date

import torch

CSV_COLUMNS = ["model", "1st token avg latency (ms)", "2+ avg latency (ms/token)", "encoder time (ms)",
               "input/output tokens", "batch_size", "actual input/output tokens", "num_beams", "low_bit",
               "cpu_embedding", "model loading time (s)", "peak mem (GB)", "streaming", "use_fp16_torch_dtype"]

SYNTHETIC = {
    "llama2-7b": dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=32, vocab_size=32000, max_position_embeddings=4096),
    "llama2-13b": dict(hidden_size=5120, intermediate_size=13824, num_hidden_layers=40, num_attention_heads=40,
                       num_key_value_heads=40, vocab_size=32000, max_position_embeddings=4096),
    "tiny": dict(hidden_size=256, intermediate_size=704, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=4, vocab_size=32000, max_position_embeddings=2048),
}

DEFAULT_CONFIG = {"repo_id": ["synthetic:llama2-7b"], "local_model_hub": None, "warm_up": 1, "num_trials": 3,
                  "num_beams": 1, "low_bit": "sym_int4", "batch_size": 1, "in_out_pairs": ["32-32", "1024-128"],
                  "test_api": ["transformer_int4_fp16_gpu"], "cpu_embedding": False, "streaming": False}


def _load(repo_id, test_api, low_bit, local_model_hub, cpu_embedding):
    """Returns (model, tokenizer or None, device, use_fp16)."""
    from ..transformers import AutoModelForCausalLM
    gpu = test_api.endswith("_gpu")
    device = "cuda" if gpu else "cpu"
    fp16 = gpu
    dtype = torch.float16 if fp16 else torch.float32
    bit = "fp16" if test_api == "bigdl_fp16_gpu" else low_bit
    kw = {}
    if test_api == "speculative_gpu":
        bit, kw = "fp16", {"speculative": True}
    if test_api == "pipeline_parallel_gpu":
        import torch.distributed as dist
        kw["pipeline_parallel_stages"] = dist.get_world_size() if dist.is_initialized() else 1
    if repo_id.startswith("synthetic:"):
        from transformers import LlamaConfig
        cfg = LlamaConfig(tie_word_embeddings=False, **SYNTHETIC[repo_id.split(":", 1)[1]])
        model = AutoModelForCausalLM.from_config(cfg, load_in_low_bit=bit, device=device, torch_dtype=dtype, **kw)
        return model, None, device, fp16
    import os
    from transformers import AutoTokenizer
    path = os.path.join(local_model_hub, repo_id.split("/")[-1]) if local_model_hub else repo_id
    if test_api in ("optimize_model", "optimize_model_gpu"):
        import transformers
        from ..optimize import optimize_model
        model = transformers.AutoModelForCausalLM.from_pretrained(path, dtype=dtype, trust_remote_code=True)
        model = optimize_model(model, low_bit=low_bit)
    else:
        model = AutoModelForCausalLM.from_pretrained(path, load_in_low_bit=bit, torch_dtype=dtype,
                                                     cpu_embedding=cpu_embedding, trust_remote_code=True, **kw)
    if gpu:
        model = model.to(dtype).to(device)
    return model, AutoTokenizer.from_pretrained(path, trust_remote_code=True), device, fp16


def run_model(repo_id, test_api, in_out_pairs, local_model_hub=None, warm_up=1, num_trials=3, num_beams=1,
              low_bit="sym_int4", cpu_embedding=False, batch_size=1, streaming=False):
    """One model through one ``test_api`` over every ``in-out`` pair; returns the CSV rows."""
    t0 = time.perf_counter()
    model, tokenizer, device, fp16 = _load(repo_id, test_api, low_bit, local_model_hub, cpu_embedding)
    load_time = time.perf_counter() - t0
    vocab = model.config.vocab_size
    rows = []
    for pair in in_out_pairs:
        in_len, out_len = (int(v) for v in pair.split("-"))
        g = torch.Generator().manual_seed(in_len)
        ids = torch.randint(3, vocab, (batch_size, in_len), generator=g).to(device)
        firsts, rests, actual_out = [], [], out_len
        if device == "cuda":
            torch.cuda.reset_peak_memory_stats()
        for trial in range(warm_up + num_trials):
            if device == "cuda":
                torch.cuda.synchronize()
            t = time.perf_counter()
            out = model.generate(ids, max_new_tokens=out_len, min_new_tokens=out_len, do_sample=False,
                                 num_beams=num_beams)
            if device == "cuda":
                torch.cuda.synchronize()
            total = time.perf_counter() - t
            actual_out = out.shape[1] - in_len
            first = float(getattr(model, "first_token_time", 0.0) or getattr(model, "first_cost", 0.0) or 0.0)
            rest = getattr(model, "rest_cost_mean", None)
            if test_api == "speculative_gpu" and getattr(model, "e2e_time_without_first", 0):
                rest = model.e2e_time_without_first / max(1, actual_out - 1)
            if not first or rest is None:            # a generate path without per-token timers: split the total
                first, rest = total / max(1, actual_out), total / max(1, actual_out)
            if trial >= warm_up:
                firsts.append(first)
                rests.append(float(rest))
        peak = torch.cuda.max_memory_allocated() / 2 ** 30 if device == "cuda" else 0.0
        rows.append([repo_id, round(1e3 * sum(firsts) / len(firsts), 2), round(1e3 * sum(rests) / len(rests), 2), 0.0,
                     pair, batch_size, f"{in_len}-{actual_out}", num_beams,
                     "fp16" if test_api in ("bigdl_fp16_gpu", "speculative_gpu") else low_bit, cpu_embedding,
                     round(load_time, 2), round(peak, 2), streaming, fp16])
    return rows


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    conf = dict(DEFAULT_CONFIG)
    if argv:
        import yaml
        with open(argv[0]) as f:
            conf.update(yaml.safe_load(f) or {})
    out_rows = []
    for api in conf["test_api"]:
        if api == "pipeline_parallel_gpu":
            import os
            import torch.distributed as dist
            if not dist.is_initialized():
                torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
                dist.init_process_group("nccl")
        rows = []
        for repo in conf["repo_id"]:
            rows += run_model(repo, api, conf["in_out_pairs"], conf.get("local_model_hub"), conf["warm_up"],
                              conf["num_trials"], conf["num_beams"], conf["low_bit"], conf.get("cpu_embedding", False),
                              conf["batch_size"], conf.get("streaming", False))
        name = f"{api}-results-{date.today()}.csv"
        rank0 = True
        if torch.distributed.is_available() and torch.distributed.is_initialized():
            rank0 = torch.distributed.get_rank() == 0
        if rank0:
            with open(name, "w", newline="") as f:
                w = csv.writer(f)
                w.writerow([""] + CSV_COLUMNS)
                for i, r in enumerate(rows):
                    w.writerow([i] + r)
            print(f"wrote {name}")
            for r in rows:
                print(dict(zip(CSV_COLUMNS, r)))
        out_rows += rows
    return out_rows


if __name__ == "__main__":
    main()
