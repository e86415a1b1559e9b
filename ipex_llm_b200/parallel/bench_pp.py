"""Pipeline-parallel decode throughput on synthetic data (Mixtral-8x7B architecture by default).

    torchrun --nproc-per-node N --master-addr 127.0.0.1 -m ipex_llm_b200.parallel.bench_pp --new-tokens 128

Random-init sym_int4 weights created stage by stage on each rank's GPU, batch 8, 1024 random prompt tokens,
greedy decoding through ``pipeline_parallel_generate`` (one graph-captured stage engine per micro-batch, NCCL p2p
between the stages).  Reports the first-token time and the decode throughput (CUDA events around the decode steps,
max over the stages).
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.distributed as dist

ARCH = {
    "mixtral-8x7b": dict(cls="MixtralConfig", hidden_size=4096, intermediate_size=14336, num_hidden_layers=32,
                         num_attention_heads=32, num_key_value_heads=8, vocab_size=32000, num_local_experts=8,
                         num_experts_per_tok=2, sliding_window=None, max_position_embeddings=4096),
    "llama2-7b": dict(cls="LlamaConfig", hidden_size=4096, intermediate_size=11008, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=32, vocab_size=32000, max_position_embeddings=4096),
    "tiny-moe": dict(cls="MixtralConfig", hidden_size=256, intermediate_size=512, num_hidden_layers=4,
                     num_attention_heads=4, num_key_value_heads=2, vocab_size=1000, num_local_experts=4,
                     num_experts_per_tok=2, sliding_window=None, max_position_embeddings=2048),
}


def run(argv=None, timed=None):
    """Run the benchmark; returns the result dictionary on rank 0 (None elsewhere).  ``timed``: optional pair of
    callables invoked right before and right after the measured generate call (clock sampling)."""
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="mixtral-8x7b", choices=list(ARCH))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--low-bit", default="sym_int4")
    a = ap.parse_args(argv)
    import transformers
    from ..transformers import AutoModelForCausalLM
    from .pp import init_pipeline_parallel
    init_pipeline_parallel()
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    arch = dict(ARCH[a.model])
    cfg = getattr(transformers, arch.pop("cls"))(tie_word_embeddings=False, **arch)
    model = AutoModelForCausalLM.from_config(cfg, load_in_low_bit=a.low_bit, torch_dtype=torch.float16, device=dev,
                                             seed=0, pipeline_parallel_stages=world)
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, cfg.vocab_size, (a.batch, a.prompt), generator=g).to(dev)
    model.generate(ids[:, :32], max_new_tokens=4, do_sample=False)            # warm-up
    if timed:
        timed[0]()
    out = model.generate(ids, max_new_tokens=a.new_tokens, do_sample=False)
    if timed:
        timed[1]()
    first, rest = model.first_token_time, model.rest_cost_mean
    t = torch.tensor([first, rest], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res = None
    if rank == 0:
        res = {"metric": "pipeline-parallel decode", "model": a.model, "n_gpus": world, "stages": world,
               "batch": a.batch, "prompt": a.prompt, "new_tokens": a.new_tokens, "low_bit": a.low_bit,
               "first_token_ms": round(float(t[0]) * 1e3, 2), "ms_per_step": round(float(t[1]) * 1e3, 3),
               "value": round(a.batch / float(t[1]), 2), "unit": "tokens/s", "out_shape": list(out.shape)}
    dist.barrier()
    dist.destroy_process_group()
    return res


def main(argv=None):
    res = run(argv)
    if res is not None:
        print(json.dumps(res))


if __name__ == "__main__":
    main()
