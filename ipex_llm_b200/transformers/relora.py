"""ReLoRA: every ``relora_steps`` optimizer steps the adapters are folded into the (re-quantized) base weights,
re-initialised, the optimizer state is pruned and the learning rate re-warms.

Counterpart of python/llm/src/ipex_llm/transformers/relora.py (``ReLoRATrainer`` :64-108, ``reset_optimizer``
:128-146, ``ReLoRACallback`` :149-283, ``ReLoRAScheduler`` :286-316, ``lora_delta_weight`` :334-346,
``find_lora_modules`` :349-363, ``update_weights`` :366-380, ``merge_and_save`` :383-453,
``load_weight_checkpoint`` :455-471).  The reference reloads the fp16 checkpoint shards from disk for each merge;
here the merge dequantizes the packed base on the device, adds ``B @ A * scaling`` and re-quantizes in place with
the GPU quantizer (or the host one on CPU), so no full-precision copy of the model has to exist anywhere.
"""
from __future__ import annotations

import math
import os
from typing import Dict

import torch

from ..ops.linear import LowBitLinear
from ..quant.params import FP4Params
from ..train.trainer import Trainer, TrainerCallback
from .qlora import _LoraBase


def is_distributed() -> bool:
    return torch.distributed.is_available() and torch.distributed.is_initialized()


def is_main_process() -> bool:
    return not is_distributed() or torch.distributed.get_rank() == 0


def find_lora_modules(model) -> Dict[str, _LoraBase]:
    return {name: m for name, m in model.named_modules() if isinstance(m, _LoraBase)}


def lora_delta_weight(layer: _LoraBase, device=None) -> torch.Tensor:
    """``B @ A * scaling`` of the active adapter as fp32 ``[out, in]`` (QA-LoRA adapters are expanded over their
    quantization blocks)."""
    name = layer.active_adapters[0]
    a = layer.lora_A[name].weight.detach().float()
    b = layer.lora_B[name].weight.detach().float()
    if device is not None:
        a, b = a.to(device), b.to(device)
    pool = getattr(layer, "qa_pool", None)
    if pool is not None:
        qk = layer.in_features // a.shape[1]
        a = a.repeat_interleave(qk, dim=1) / qk
    return (b @ a) * layer.scaling[name]


def update_weights(target: _LoraBase, new_weight: torch.Tensor, reinit: bool, device):
    """Install ``new_weight`` (full precision ``[out, in]``) as the base weight; optionally restart the adapter."""
    if reinit:
        for name in list(target.lora_A.keys()):
            torch.nn.init.kaiming_uniform_(target.lora_A[name].weight, a=math.sqrt(5))
            torch.nn.init.zeros_(target.lora_B[name].weight)
    base = target.base_layer
    if isinstance(base, LowBitLinear):
        p = FP4Params(new_weight.to(torch.float32).cpu() if device == "cpu" or torch.device(device).type == "cpu"
                      else new_weight.to(torch.float16), requires_grad=False, quantized=False, _shape=None,
                      qtype=base.qtype)
        base._parameters["weight"] = p.to(device)
    else:
        base.weight.data.copy_(new_weight.to(base.weight.dtype))


@torch.no_grad()
def merge_and_requantize(model, reinit: bool = True):
    """Fold every adapter into its base layer (dequantize -> add -> quantize for low-bit bases)."""
    for _, layer in find_lora_modules(model).items():
        base = layer.base_layer
        dev = base.weight.device
        delta = lora_delta_weight(layer, dev)
        if isinstance(base, LowBitLinear):
            w = base.weight.dequantize(torch.float32)
        else:
            w = base.weight.detach().float()
        update_weights(layer, w + delta, reinit, dev)


def merge_and_save(model, dst_dir: str, reinit: bool = False, **_unused):
    """Merge, then write the merged model in the low-bit format (``save_low_bit``) when available."""
    merge_and_requantize(model, reinit=reinit)
    base = getattr(model, "base_model", model)
    os.makedirs(dst_dir, exist_ok=True)
    if hasattr(base, "save_low_bit"):
        # adapters are zero after a re-init and are skipped by the serializer of the base model
        base.save_low_bit(dst_dir)
    else:
        torch.save(base.state_dict(), os.path.join(dst_dir, "pytorch_model.bin"))


def load_weight_checkpoint(model, checkpoint_path: str):
    """Restore merged base weights written by ``merge_and_save`` (plain ``state_dict`` form)."""
    sd = torch.load(os.path.join(checkpoint_path, "pytorch_model.bin"), map_location="cpu", weights_only=False)
    getattr(model, "base_model", model).load_state_dict(sd, strict=False)


def reset_optimizer(optimizer, prune_ratio: float = 0.9):
    """Zero the smallest ``prune_ratio`` fraction (by magnitude) of the Adam moments after a restart."""
    from ..parallel.dp import FusedLoraAdamW
    if isinstance(optimizer, FusedLoraAdamW):
        tensors = [optimizer.exp_avg, optimizer.exp_avg_sq]
    else:
        tensors = [s[k] for s in optimizer.state.values() for k in ("exp_avg", "exp_avg_sq") if k in s]
    for t in tensors:
        if t.numel() == 0:
            continue
        k = int(prune_ratio * t.numel())
        if k <= 0:
            continue
        thresh = torch.kthvalue(t.abs().flatten().float().cpu(), max(1, k)).values.item()
        t.mul_((t.abs() > thresh).to(t.dtype))


class ReLoRAScheduler:
    """Multiplier on the learning rate that re-warms after every restart (jagged schedule)."""

    def __init__(self, relora_steps: int, warmup_steps: int, min_lr_scale: float = 0.001):
        self.relora_steps, self.warmup_steps, self.min_lr_scale = relora_steps, max(1, warmup_steps), min_lr_scale

    def scale(self, step: int) -> float:
        if step < self.relora_steps:
            return 1.0
        cycle_t = min(1.0, (step % self.relora_steps) / self.warmup_steps)
        return cycle_t * (1 - self.min_lr_scale) + self.min_lr_scale


class ReLoRACallback(TrainerCallback):
    def __init__(self, relora_steps=150, relora_warmup_steps=10, relora_cpu_offload=False, prune_ratio=0.9,
                 resume_from_checkpoint=None):
        self.relora_steps = relora_steps
        self.sched = ReLoRAScheduler(relora_steps, relora_warmup_steps)
        self.cpu_offload = relora_cpu_offload
        self.prune_ratio = prune_ratio
        self.last_full_model = resume_from_checkpoint
        self.num_restarts = 0
        self._base_lr = None

    def on_train_begin(self, args, state, control, **kw):
        self._base_lr = args.learning_rate

    def on_step_begin(self, args, state, control, model=None, optimizer=None, **kw):
        if state.global_step > 0 and state.global_step % self.relora_steps == 0 and \
                self.num_restarts < state.global_step // self.relora_steps:
            merge_and_requantize(model, reinit=True)
            reset_optimizer(optimizer, self.prune_ratio)
            from ..parallel.dp import FusedLoraAdamW
            if isinstance(optimizer, FusedLoraAdamW):
                # the adapters were re-initialised in place inside the flat parameter buffer
                lo = optimizer.rank * optimizer.shard
                optimizer.master.copy_(optimizer.flat_params[lo:lo + optimizer.shard].float())
            self.num_restarts = state.global_step // self.relora_steps
        # applied on top of the trainer's own schedule
        if optimizer is not None:
            s = self.sched.scale(state.global_step)
            for g in optimizer.param_groups:
                g["relora_scale"] = s

    def on_save(self, args, state, control, model=None, **kw):
        if model is not None and is_main_process():
            d = os.path.join(args.output_dir, f"checkpoint-{state.global_step}", "relora")
            os.makedirs(d, exist_ok=True)
            torch.save({"num_restarts": self.num_restarts}, os.path.join(d, "relora_state.pt"))


class ReLoRATrainer(Trainer):
    """``Trainer`` + ReLoRA restarts (reference relora.py:64-108)."""

    def __init__(self, *args, base_model=None, relora_steps=150, relora_warmup_steps=10, relora_cpu_offload=False,
                 resume_from_checkpoint=False, **kwargs):
        super().__init__(*args, **kwargs)
        self.relora = ReLoRACallback(relora_steps, relora_warmup_steps, relora_cpu_offload,
                                     resume_from_checkpoint=resume_from_checkpoint)
        self.callbacks.append(self.relora)
