"""A small causal-LM trainer for adapter finetuning (the reference drives HF ``Trainer``;
python/llm/example/GPU/LLM-Finetuning/QLoRA/alpaca-qlora/alpaca_qlora_finetuning.py:242-278).

One process per GPU.  Data parallelism is built in: every rank runs its micro-batches, the optimizer
(``FusedLoraAdamW``) averages gradients and updates parameters in one fused kernel.  Checkpoints hold the adapter
weights, the optimizer shards, the step, the RNG state and the data cursor, so ``resume_from_checkpoint`` continues
bit-for-bit on the same world size.
"""
from __future__ import annotations

import json
import math
import os
import time
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from ..parallel.dp import FusedLoraAdamW, PagedAdamW
from ..utils.common import invalidInputError


class TrainerCallback:
    """Hook points (same names as HF ``TrainerCallback`` for the ones used by ReLoRA / LISA)."""

    def on_train_begin(self, args, state, control, **kw): ...
    def on_step_begin(self, args, state, control, **kw): ...
    def on_step_end(self, args, state, control, **kw): ...
    def on_save(self, args, state, control, **kw): ...
    def on_train_end(self, args, state, control, **kw): ...


class TrainerState:
    def __init__(self):
        self.global_step = 0
        self.epoch = 0.0
        self.log_history: List[Dict] = []
        self.data_cursor = 0


class TrainerControl:
    def __init__(self):
        self.should_training_stop = False
        self.should_save = False


def _lr_lambda(kind: str, warmup: int, total: int) -> Callable[[int], float]:
    def f(step):
        if warmup > 0 and step < warmup:
            return (step + 1) / warmup
        if kind == "constant":
            return 1.0
        prog = (step - warmup) / max(1, total - warmup)
        if kind == "cosine":
            return 0.5 * (1.0 + math.cos(math.pi * min(1.0, prog)))
        return max(0.0, 1.0 - prog)   # linear
    return f


class Trainer:
    def __init__(self, model, args, train_dataset=None, data_collator=None, callbacks: Optional[list] = None,
                 optimizers=(None, None), tokenizer=None, eval_dataset=None):
        self.model, self.args = model, args
        self.train_dataset, self.collate = train_dataset, data_collator or default_collator
        self.callbacks = list(callbacks or [])
        self.optimizer, self.lr_scheduler = optimizers
        self.state, self.control = TrainerState(), TrainerControl()
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.device = next(p for p in model.parameters()).device

    # ------------------------------------------------------------------------------------------------
    def create_optimizer(self):
        a = self.args
        params = [p for p in self.model.parameters() if p.requires_grad]
        kw = dict(lr=a.learning_rate, betas=(a.adam_beta1, a.adam_beta2), eps=a.adam_epsilon,
                  weight_decay=a.weight_decay)
        if a.optim == "adamw_torch":
            invalidInputError(self.world == 1, "adamw_torch has no gradient averaging: use fused_lora_adamw")
            self.optimizer = torch.optim.AdamW(params, **kw)
        elif a.optim == "paged_adamw" and self.world == 1 and self.device.type == "cuda" and \
                sum(p.numel() for p in params) > (1 << 28):
            self.optimizer = PagedAdamW(params, **kw)
        else:
            self.optimizer = FusedLoraAdamW(params, max_grad_norm=a.max_grad_norm, **kw)
        return self.optimizer

    def _batches(self, start_cursor: int):
        """Rank-strided micro-batches over the dataset, resumable from a cursor (in samples)."""
        a = self.args
        n = len(self.train_dataset)
        bs = a.per_device_train_batch_size
        g = torch.Generator().manual_seed(a.seed)
        cursor = start_cursor
        epoch = cursor // n
        while True:
            g.manual_seed(a.seed + epoch)
            perm = torch.randperm(n, generator=g).tolist()
            pos = cursor % n
            while pos + bs * self.world <= n:
                idx = perm[pos + self.rank * bs: pos + (self.rank + 1) * bs]
                yield self.collate([self.train_dataset[i] for i in idx]), cursor + bs * self.world
                pos += bs * self.world
                cursor += bs * self.world
            cursor = (epoch + 1) * n
            epoch += 1

    def compute_loss(self, model, batch):
        batch = {k: v.to(self.device, non_blocking=True) for k, v in batch.items()}
        out = model(**batch)
        return out.loss if hasattr(out, "loss") and out.loss is not None else out[0]

    def train(self, resume_from_checkpoint: Optional[str] = None):
        a = self.args
        torch.manual_seed(a.seed + self.rank)
        if self.optimizer is None:
            self.create_optimizer()
        steps_per_epoch = max(1, len(self.train_dataset) // (a.per_device_train_batch_size * self.world *
                                                              a.gradient_accumulation_steps))
        total = a.max_steps if a.max_steps > 0 else int(math.ceil(a.num_train_epochs * steps_per_epoch))
        warmup = a.warmup_steps or int(a.warmup_ratio * total)
        sched = _lr_lambda(a.lr_scheduler_type, warmup, total)
        base_lr = a.learning_rate
        resume = resume_from_checkpoint or a.resume_from_checkpoint
        if resume:
            self._load_checkpoint(resume)
        for cb in self.callbacks:
            cb.on_train_begin(a, self.state, self.control, model=self.model, optimizer=self.optimizer)
        self.model.train()
        it = self._batches(self.state.data_cursor)
        t0 = time.time()
        tokens = 0
        self.optimizer.zero_grad()
        while self.state.global_step < total and not self.control.should_training_stop:
            for cb in self.callbacks:
                cb.on_step_begin(a, self.state, self.control, model=self.model, optimizer=self.optimizer)
            for g in self.optimizer.param_groups:
                # callbacks may install a per-group multiplier (ReLoRA's re-warm-up after each restart)
                g["lr"] = base_lr * sched(self.state.global_step) * g.get("relora_scale", 1.0)
            loss_acc = 0.0
            for _ in range(a.gradient_accumulation_steps):
                batch, cursor = next(it)
                ctx = torch.autocast("cuda", dtype=torch.bfloat16) if (self.device.type == "cuda" and a.bf16) \
                    else _null()
                with ctx:
                    loss = self.compute_loss(self.model, batch) / a.gradient_accumulation_steps
                loss.backward()
                loss_acc += float(loss.detach())
                tokens += int(batch["input_ids"].numel())
                self.state.data_cursor = cursor
            if not isinstance(self.optimizer, FusedLoraAdamW) and a.max_grad_norm and a.max_grad_norm > 0:
                torch.nn.utils.clip_grad_norm_([p for p in self.model.parameters() if p.requires_grad],
                                               a.max_grad_norm)
            self.optimizer.step()
            self.optimizer.zero_grad()
            self.state.global_step += 1
            self.state.epoch = self.state.global_step / steps_per_epoch
            if a.logging_steps and self.state.global_step % a.logging_steps == 0:
                rec = {"step": self.state.global_step, "loss": loss_acc, "lr": self.optimizer.param_groups[0]["lr"],
                       "epoch": round(self.state.epoch, 4)}
                self.state.log_history.append(rec)
                if self.rank == 0:
                    print(rec, flush=True)
            for cb in self.callbacks:
                cb.on_step_end(a, self.state, self.control, model=self.model, optimizer=self.optimizer)
            if (a.save_steps and self.state.global_step % a.save_steps == 0) or self.control.should_save:
                self.save_checkpoint()
                self.control.should_save = False
        dt = time.time() - t0
        for cb in self.callbacks:
            cb.on_train_end(a, self.state, self.control, model=self.model, optimizer=self.optimizer)
        metrics = {"train_runtime": dt, "train_steps_per_second": self.state.global_step / max(dt, 1e-9),
                   "train_tokens_per_second": tokens * self.world / max(dt, 1e-9),
                   "train_loss": self.state.log_history[-1]["loss"] if self.state.log_history else None}
        return metrics

    # ------------------------------------------------------------------------------------------------
    def _ckpt_dir(self):
        return os.path.join(self.args.output_dir, f"checkpoint-{self.state.global_step}")

    def save_checkpoint(self):
        d = self._ckpt_dir()
        os.makedirs(d, exist_ok=True)
        if self.rank == 0:
            if hasattr(self.model, "save_pretrained") and hasattr(self.model, "peft_config"):
                self.model.save_pretrained(d)
            else:
                torch.save({k: v.cpu() for k, v in self.model.state_dict().items()
                            if v.is_floating_point() and "lora_" in k}, os.path.join(d, "trainable.bin"))
            with open(os.path.join(d, "trainer_state.json"), "w") as f:
                json.dump({"global_step": self.state.global_step, "epoch": self.state.epoch,
                           "data_cursor": self.state.data_cursor, "log_history": self.state.log_history}, f)
        torch.save({"optimizer": self.optimizer.state_dict(), "rng": torch.get_rng_state(),
                    "cuda_rng": torch.cuda.get_rng_state() if self.device.type == "cuda" else None},
                   os.path.join(d, f"optimizer_rank{self.rank}.pt"))
        for cb in self.callbacks:
            cb.on_save(self.args, self.state, self.control, model=self.model)
        if dist.is_initialized():
            dist.barrier()
        self._rotate()
        return d

    def _rotate(self):
        lim = self.args.save_total_limit
        if not lim or self.rank != 0:
            return
        import shutil
        cks = sorted((int(n.split("-")[1]), n) for n in os.listdir(self.args.output_dir)
                     if n.startswith("checkpoint-") and n.split("-")[1].isdigit())
        for _, n in cks[:-lim]:
            shutil.rmtree(os.path.join(self.args.output_dir, n), ignore_errors=True)

    def _load_checkpoint(self, d):
        if d is True:
            cks = sorted(int(n.split("-")[1]) for n in os.listdir(self.args.output_dir) if n.startswith("checkpoint-"))
            invalidInputError(len(cks) > 0, f"no checkpoint under {self.args.output_dir}")
            d = os.path.join(self.args.output_dir, f"checkpoint-{cks[-1]}")
        with open(os.path.join(d, "trainer_state.json")) as f:
            st = json.load(f)
        self.state.global_step, self.state.epoch = st["global_step"], st["epoch"]
        self.state.data_cursor, self.state.log_history = st["data_cursor"], st["log_history"]
        from ..transformers.qlora import ADAPTER_WEIGHTS, set_peft_model_state_dict
        if os.path.exists(os.path.join(d, ADAPTER_WEIGHTS)):
            set_peft_model_state_dict(self.model, torch.load(os.path.join(d, ADAPTER_WEIGHTS), map_location="cpu",
                                                             weights_only=True))
        else:
            self.model.load_state_dict(torch.load(os.path.join(d, "trainable.bin"), map_location="cpu",
                                                  weights_only=True), strict=False)
        blob = torch.load(os.path.join(d, f"optimizer_rank{self.rank}.pt"), map_location="cpu", weights_only=False)
        self.optimizer.load_state_dict(blob["optimizer"])
        torch.set_rng_state(blob["rng"])
        if blob.get("cuda_rng") is not None and self.device.type == "cuda":
            torch.cuda.set_rng_state(blob["cuda_rng"])

    def save_model(self, output_dir=None):
        d = output_dir or self.args.output_dir
        if self.rank == 0 and hasattr(self.model, "save_pretrained"):
            self.model.save_pretrained(d)


class _null:
    def __enter__(self): return None
    def __exit__(self, *a): return False


def default_collator(samples):
    """Pads ``input_ids`` / ``labels`` / ``attention_mask`` lists to the longest sample (labels padded with -100)."""
    keys = samples[0].keys()
    n = max(len(s["input_ids"]) for s in samples)
    out = {}
    for k in keys:
        pad = -100 if k == "labels" else 0
        out[k] = torch.tensor([list(s[k]) + [pad] * (n - len(s[k])) for s in samples], dtype=torch.long)
    if "labels" not in out:
        out["labels"] = out["input_ids"].clone()
    return out
