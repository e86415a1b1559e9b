"""python examples/qlora_finetune.py --repo-id-or-model-path <dir> --data <jsonl with a "text" field>
(torchrun --nproc-per-node N ... for data parallel)"""
import argparse
import json
import os

import torch
import torch.distributed as dist
from transformers import AutoTokenizer

from ipex_llm.transformers import AutoModelForCausalLM
from ipex_llm.transformers.qlora import LoraConfig, TrainingArguments, get_peft_model, prepare_model_for_kbit_training
from ipex_llm_b200.train import Trainer

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--repo-id-or-model-path", required=True)
    ap.add_argument("--data", required=True)
    ap.add_argument("--output-dir", default="outputs")
    ap.add_argument("--max-steps", type=int, default=200)
    ap.add_argument("--cutoff-len", type=int, default=256)
    a = ap.parse_args()
    if "RANK" in os.environ:
        local = int(os.environ.get("LOCAL_RANK", 0))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    tok = AutoTokenizer.from_pretrained(a.repo_id_or_model_path)
    model = AutoModelForCausalLM.from_pretrained(a.repo_id_or_model_path, load_in_low_bit="nf4", optimize_model=False,
                                                 torch_dtype=torch.bfloat16, modules_to_not_convert=["lm_head"])
    model = model.to("cuda")
    model = prepare_model_for_kbit_training(model)
    model = get_peft_model(model, LoraConfig(r=8, lora_alpha=32, lora_dropout=0.05, bias="none",
                                             target_modules=["q_proj", "k_proj", "v_proj"], task_type="CAUSAL_LM"))
    with open(a.data) as f:
        rows = [json.loads(line) for line in f if line.strip()]
    data = [{"input_ids": tok(r["text"], truncation=True, max_length=a.cutoff_len)["input_ids"]} for r in rows]
    for d in data:
        d["labels"] = list(d["input_ids"])
    args = TrainingArguments(output_dir=a.output_dir, per_device_train_batch_size=4, gradient_accumulation_steps=1,
                             warmup_steps=20, max_steps=a.max_steps, learning_rate=2e-4, save_steps=100, bf16=True,
                             logging_steps=20, optim="paged_adamw")
    trainer = Trainer(model, args, train_dataset=data)
    print(trainer.train())
    trainer.save_model(a.output_dir)
