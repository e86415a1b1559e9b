"""QLoRA data-parallel training throughput on synthetic data.

    python -m ipex_llm_b200.train.bench_qlora --steps 8 --warmup 3                       (1 GPU)
    torchrun --nproc-per-node N --master-addr 127.0.0.1 -m ipex_llm_b200.train.bench_qlora ...

Llama-2-13B architecture (40 layers, hidden 5120, 40 heads, intermediate 13824, vocab 32000), frozen nf4 base created
directly on the device with random weights, LoRA r=8 alpha=16 dropout 0.05 on q/k/v/o/gate/up/down, bf16 compute,
sequence 512, micro-batch 4 per GPU, random token ids, causal-LM loss.  One step = forward + backward + fused
reduce-scatter/AdamW/all-gather kernel.  Timed with CUDA events around K steps after W warm-ups, max over ranks;
inputs come from pinned host memory every step and the loss is read back, as a training loop does.
``--optimizer torch`` swaps in ``dist.all_reduce`` + ``torch.optim.AdamW`` (the library baseline).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

ARCH = {
    "llama2-13b": dict(hidden_size=5120, intermediate_size=13824, num_hidden_layers=40, num_attention_heads=40,
                       num_key_value_heads=40, vocab_size=32000, max_position_embeddings=4096),
    "llama2-7b": dict(hidden_size=4096, intermediate_size=11008, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=32, vocab_size=32000, max_position_embeddings=4096),
    "tiny": dict(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=4, vocab_size=1000, max_position_embeddings=1024),
}


def run(argv=None, timed=None):
    """Run the benchmark; returns the result dictionary on rank 0 (None elsewhere).  ``timed``: optional pair of
    callables invoked right before and right after the measured steps (clock sampling)."""
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama2-13b", choices=list(ARCH))
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--optimizer", default="fused", choices=["fused", "torch"])
    ap.add_argument("--no-checkpointing", action="store_true")
    a = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from transformers import LlamaConfig
    from ..parallel.dp import FusedLoraAdamW
    from ..transformers import AutoModelForCausalLM
    from ..transformers.qlora import LoraConfig, cast_lora_weight, get_peft_model, prepare_model_for_kbit_training
    arch = dict(ARCH[a.model])
    if a.layers:
        arch["num_hidden_layers"] = a.layers
    cfg = LlamaConfig(tie_word_embeddings=False, **arch)
    model = AutoModelForCausalLM.from_config(cfg, load_in_low_bit="nf4", torch_dtype=torch.bfloat16, device=dev,
                                             modules_to_not_convert=["lm_head"], optimize_model=False, seed=0)
    model = prepare_model_for_kbit_training(model, use_gradient_checkpointing=not a.no_checkpointing)
    torch.manual_seed(0)
    pm = get_peft_model(model, LoraConfig(r=8, lora_alpha=16, lora_dropout=0.05, training_mode="qlora",
                                          target_modules=["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj",
                                                          "up_proj", "down_proj"]))
    cast_lora_weight(pm, torch.bfloat16)
    pm.train()
    params = [p for p in pm.parameters() if p.requires_grad]
    n_train = sum(p.numel() for p in params)
    if a.optimizer == "fused":
        opt = FusedLoraAdamW(params, lr=2e-4, max_grad_norm=0.0)
    else:
        opt = torch.optim.AdamW(params, lr=2e-4)
    g = torch.Generator().manual_seed(100 + rank)
    host = [torch.randint(0, cfg.vocab_size, (a.micro_batch, a.seq), generator=g).pin_memory()
            for _ in range(a.steps + a.warmup)]

    def step(i):
        ids = host[i].to(dev, non_blocking=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = pm(input_ids=ids, labels=ids).loss
        loss.backward()
        if a.optimizer == "torch" and world > 1:
            for p in params:
                dist.all_reduce(p.grad)
                p.grad.div_(world)
        opt.step()
        opt.zero_grad()
        return loss

    for i in range(a.warmup):
        step(i)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if timed:
        timed[0]()
    e0.record()
    last = 0.0
    for i in range(a.steps):
        last = float(step(a.warmup + i))          # device -> host read of the loss every step
    e1.record()
    if timed:
        torch.cuda.synchronize()
        timed[1]()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    res = None
    if rank == 0:
        ms = float(t[0])
        res = ({"metric": "QLoRA finetune throughput", "model": a.model, "n_gpus": world,
                          "value": round(world * a.micro_batch * 1000.0 / ms, 3), "unit": "samples/s",
                          "tokens_per_s": round(world * a.micro_batch * a.seq * 1000.0 / ms, 1),
                          "ms_per_step": round(ms, 3), "steps": a.steps, "warmup": a.warmup, "seq_len": a.seq,
                          "micro_batch_per_gpu": a.micro_batch, "trainable_params": n_train,
                          "optimizer": "fused reduce-scatter + AdamW + all-gather kernel" if a.optimizer == "fused"
                          else "NCCL all_reduce + torch.optim.AdamW", "base": "nf4", "compute": "bf16",
                          "gradient_checkpointing": not a.no_checkpointing, "last_loss": round(last, 4),
                          "h2d_bytes_per_step": a.micro_batch * a.seq * 8, "d2h_bytes_per_step": 4})
    if world > 1:
        dist.destroy_process_group()
    return res


def main(argv=None):
    res = run(argv)
    if res is not None:
        print(json.dumps(res))


if __name__ == "__main__":
    main()
