"""QLoRA / LoRA / QA-LoRA / ReLoRA adapters on low-bit base models.

Covers the surface of python/llm/src/ipex_llm/transformers/qlora.py of the reference
(``LoraLowBitLinear`` :66-143, ``LoraBF16Linear`` :146-211, ``get_peft_model`` :282-301,
``prepare_model_for_kbit_training`` :304-352, ``LoraConfig`` :254-279, ``TrainingArguments`` :355-374,
``cast_lora_weight`` :377-391, ``PeftModel``).  The reference patches the ``peft`` package; this package carries its
own small adapter implementation with the same names, file formats (``adapter_config.json`` +
``adapter_model.bin`` with ``base_model.model.<path>.lora_A.weight`` keys) and semantics, so it works without peft
and adapters stay interchangeable.
"""
from __future__ import annotations

import json
import math
import os
import re
from dataclasses import asdict, dataclass, field
from typing import List, Optional, Union

import torch
from torch import nn

from ..ops.linear import BF16Linear, FP16Linear, LowBitLinear
from ..quant.params import get_block_size
from ..utils.common import invalidInputError

ADAPTER_WEIGHTS = "adapter_model.bin"
ADAPTER_CONFIG = "adapter_config.json"


@dataclass
class LoraConfig:
    """Adapter hyper-parameters (peft's ``LoraConfig`` fields that matter here + ``training_mode``)."""
    r: int = 8
    lora_alpha: int = 8
    lora_dropout: float = 0.0
    target_modules: Optional[Union[List[str], str]] = None
    bias: str = "none"
    task_type: str = "CAUSAL_LM"
    fan_in_fan_out: bool = False
    init_lora_weights: Union[bool, str] = True
    use_rslora: bool = False
    modules_to_save: Optional[List[str]] = None
    training_mode: str = "qlora"      # qlora | lora | qalora | relora
    base_model_name_or_path: Optional[str] = None
    inference_mode: bool = False
    peft_type: str = "LORA"

    def to_dict(self):
        return asdict(self)

    def save_pretrained(self, path):
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, ADAPTER_CONFIG), "w") as f:
            json.dump(self.to_dict(), f, indent=2, sort_keys=True)

    @classmethod
    def from_pretrained(cls, path):
        with open(os.path.join(path, ADAPTER_CONFIG)) as f:
            d = json.load(f)
        known = {k: v for k, v in d.items() if k in cls.__dataclass_fields__}
        return cls(**known)


class _LoraBase(nn.Module):
    """Shared adapter plumbing: per-adapter A/B, scaling, dropout, enable/disable, merge bookkeeping."""

    def __init__(self, base_layer, adapter_name, r, lora_alpha, lora_dropout, init_lora_weights, use_rslora,
                 lora_in_features):
        super().__init__()
        self.base_layer = base_layer
        self.in_features, self.out_features = base_layer.in_features, base_layer.out_features
        self.r, self.lora_alpha, self.scaling = {}, {}, {}
        self.lora_dropout = nn.ModuleDict()
        self.lora_A, self.lora_B = nn.ModuleDict(), nn.ModuleDict()
        self.disable_adapters = False
        self.merged = False
        self._active_adapter = adapter_name
        self._lora_in = lora_in_features
        self.update_layer(adapter_name, r, lora_alpha, lora_dropout, init_lora_weights, use_rslora)

    @property
    def active_adapters(self):
        a = self._active_adapter
        return [a] if isinstance(a, str) else list(a)

    @property
    def weight(self):
        return self.base_layer.weight

    @property
    def bias(self):
        return self.base_layer.bias

    def update_layer(self, name, r, lora_alpha, lora_dropout, init_lora_weights=True, use_rslora=False):
        invalidInputError(r > 0, f"`r` should be a positive integer value but the value passed is {r}")
        self.r[name], self.lora_alpha[name] = r, lora_alpha
        self.lora_dropout[name] = nn.Dropout(p=lora_dropout) if lora_dropout > 0.0 else nn.Identity()
        dev = self.base_layer.weight.device
        dev = dev if dev.type != "meta" else None
        self.lora_A[name] = nn.Linear(self._lora_in, r, bias=False, device=dev)
        self.lora_B[name] = nn.Linear(r, self.out_features, bias=False, device=dev)
        self.scaling[name] = lora_alpha / math.sqrt(r) if use_rslora else lora_alpha / r
        if init_lora_weights:
            if init_lora_weights == "gaussian":
                nn.init.normal_(self.lora_A[name].weight, std=1 / r)
            else:
                nn.init.kaiming_uniform_(self.lora_A[name].weight, a=math.sqrt(5))
            nn.init.zeros_(self.lora_B[name].weight)

    def _lora_delta(self, x, pool=None):
        out = None
        for name in self.active_adapters:
            if name not in self.lora_A:
                continue
            a, b = self.lora_A[name], self.lora_B[name]
            h = self.lora_dropout[name](x if pool is None else pool(x))
            d = b(a(h.to(a.weight.dtype))) * self.scaling[name]
            out = d if out is None else out + d
        return out


class LoraLowBitLinear(_LoraBase):
    """LoRA on a frozen ``LowBitLinear`` (reference qlora.py:66-143).  ``qa_lora`` average-pools the adapter input
    over each quantization block, so the merged update stays constant inside a block (QA-LoRA)."""

    def __init__(self, base_layer, adapter_name, r: int = 0, lora_alpha: int = 1, lora_dropout: float = 0.0,
                 qa_lora: bool = True, fan_in_fan_out: bool = False, init_lora_weights=True, use_rslora=False,
                 **kwargs):
        qtype = kwargs.get("qtype", getattr(base_layer, "qtype", None))
        qk = get_block_size(qtype) if qa_lora else 1
        super().__init__(base_layer, adapter_name, r, lora_alpha, lora_dropout, init_lora_weights, use_rslora,
                         base_layer.in_features // qk)
        self.fan_in_fan_out = fan_in_fan_out
        self.qa_pool = nn.AvgPool1d(qk) if qa_lora else None

    def forward(self, x: torch.Tensor):
        if x.is_cuda:
            x = x.to(torch.bfloat16)        # training on the GPU runs in bf16, as in the reference
        elif torch.is_autocast_enabled("cpu"):
            x = x.to(torch.get_autocast_dtype("cpu"))
        result = self.base_layer(x)
        if self.disable_adapters or self.merged:
            return result
        delta = self._lora_delta(x, self.qa_pool)
        return result if delta is None else result + delta.to(result.dtype)


class LoraBF16Linear(_LoraBase):
    """LoRA on a dense bf16 base layer (reference qlora.py:146-211)."""

    def __init__(self, base_layer, adapter_name, r: int = 0, lora_alpha: int = 1, lora_dropout: float = 0.0,
                 fan_in_fan_out: bool = False, init_lora_weights=True, use_rslora=False, **kwargs):
        super().__init__(base_layer, adapter_name, r, lora_alpha, lora_dropout, init_lora_weights, use_rslora,
                         base_layer.in_features)
        self.fan_in_fan_out = fan_in_fan_out

    def forward(self, x: torch.Tensor):
        if x.is_cuda:
            x = x.to(torch.bfloat16)
        result = self.base_layer(x)
        if self.disable_adapters or self.merged:
            return result
        delta = self._lora_delta(x)
        return result if delta is None else result + delta.to(result.dtype)

    def merge(self):
        """Fold the adapters into the dense base weight."""
        if self.merged:
            return
        w = self.base_layer.weight
        for name in self.active_adapters:
            w.data += (self.lora_B[name].weight.float() @ self.lora_A[name].weight.float()).to(w.dtype) * \
                self.scaling[name]
        self.merged = True


def _match_target(name: str, targets) -> bool:
    if isinstance(targets, str):
        return re.fullmatch(targets, name) is not None
    return any(name == t or name.endswith("." + t) for t in targets)


_DEFAULT_TARGETS = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


def _create_new_module(config: LoraConfig, adapter_name: str, target: nn.Module):
    """LowBitLinear -> LoraLowBitLinear, BF16Linear -> LoraBF16Linear (reference qlora.py:214-251)."""
    kw = dict(r=config.r, lora_alpha=config.lora_alpha, lora_dropout=config.lora_dropout,
              fan_in_fan_out=config.fan_in_fan_out, init_lora_weights=config.init_lora_weights,
              use_rslora=config.use_rslora)
    if isinstance(target, LowBitLinear):
        return LoraLowBitLinear(target, adapter_name, qa_lora=config.training_mode == "qalora", qtype=target.qtype,
                                **kw)
    if isinstance(target, (BF16Linear, FP16Linear, nn.Linear)):
        return LoraBF16Linear(target, adapter_name, **kw)
    invalidInputError(False, f"Target module {type(target).__name__} is not supported; only LowBitLinear, "
                             "BF16Linear and torch.nn.Linear are")


class PeftModel(nn.Module):
    """Base model + injected adapters.  Forward / generate go to the base model."""

    def __init__(self, model, peft_config: LoraConfig, adapter_name: str = "default"):
        super().__init__()
        self.base_model = model
        self.peft_config = {adapter_name: peft_config}
        self.active_adapter = adapter_name
        self.config = getattr(model, "config", None)
        self._inject(peft_config, adapter_name)
        mark_only_lora_as_trainable(self.base_model, peft_config.bias)

    # the reference's (peft's) checkpoints prefix keys with base_model.model.
    @property
    def model(self):
        return self.base_model

    def _inject(self, config, adapter_name):
        targets = config.target_modules or _DEFAULT_TARGETS
        replaced = 0
        for name, mod in list(self.base_model.named_modules()):
            if isinstance(mod, _LoraBase) or not isinstance(mod, nn.Linear) or not _match_target(name, targets):
                continue
            parent_name, _, child = name.rpartition(".")
            parent = self.base_model.get_submodule(parent_name) if parent_name else self.base_model
            setattr(parent, child, _create_new_module(config, adapter_name, mod))
            replaced += 1
        invalidInputError(replaced > 0, f"Target modules {targets} not found in the base model.")

    def forward(self, *args, **kwargs):
        return self.base_model(*args, **kwargs)

    def generate(self, *args, **kwargs):
        return self.base_model.generate(*args, **kwargs)

    def __getattr__(self, name):
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(self.base_model, name)

    def get_nb_trainable_parameters(self):
        trainable = sum(p.numel() for p in self.parameters() if p.requires_grad)
        total = 0
        for p in self.parameters():
            n = p.numel()
            shape = getattr(p, "_shape", None)
            if shape is not None and getattr(p, "quantized", False):
                n = int(shape[0]) * int(shape[1])
            total += n
        return trainable, total

    def print_trainable_parameters(self):
        t, a = self.get_nb_trainable_parameters()
        print(f"trainable params: {t:,d} || all params: {a:,d} || trainable%: {100 * t / max(a, 1):.4f}")

    def enable_input_require_grads(self):
        emb = self.base_model.get_input_embeddings()
        emb.register_forward_hook(lambda m, i, o: o.requires_grad_(True))

    def disable_adapter_layers(self, flag=True):
        for m in self.modules():
            if isinstance(m, _LoraBase):
                m.disable_adapters = flag

    def save_pretrained(self, save_directory, **kwargs):
        os.makedirs(save_directory, exist_ok=True)
        cfg = self.peft_config[self.active_adapter]
        cfg.save_pretrained(save_directory)
        torch.save(get_peft_model_state_dict(self), os.path.join(save_directory, ADAPTER_WEIGHTS))

    @classmethod
    def from_pretrained(cls, model, model_id, adapter_name="default", is_trainable=False, **kwargs):
        cfg = LoraConfig.from_pretrained(model_id)
        cfg.inference_mode = not is_trainable
        pm = cls(model, cfg, adapter_name)
        sd = torch.load(os.path.join(model_id, ADAPTER_WEIGHTS), map_location="cpu", weights_only=True)
        set_peft_model_state_dict(pm, sd, adapter_name)
        if not is_trainable:
            for p in pm.parameters():
                p.requires_grad_(False)
        return pm

    def merge_and_unload(self):
        """Dense bases only: fold adapters and return the plain model."""
        for name, mod in list(self.base_model.named_modules()):
            if isinstance(mod, LoraBF16Linear):
                mod.merge()
                parent_name, _, child = name.rpartition(".")
                parent = self.base_model.get_submodule(parent_name) if parent_name else self.base_model
                setattr(parent, child, mod.base_layer)
            elif isinstance(mod, LoraLowBitLinear):
                invalidInputError(False, "merging into a quantized base loses precision: dequantize the base first "
                                         "(see relora.merge_and_requantize) or export with a bf16 base")
        return self.base_model


def get_peft_model_state_dict(model: PeftModel, adapter_name="default"):
    out = {}
    for k, v in model.base_model.state_dict().items():
        if "lora_" in k:
            out["base_model.model." + k.replace(f".{adapter_name}.", ".")] = v.detach().cpu()
    return out


def set_peft_model_state_dict(model: PeftModel, sd, adapter_name="default"):
    own = model.base_model.state_dict()
    mapped = {}
    for k, v in sd.items():
        k = k[len("base_model.model."):] if k.startswith("base_model.model.") else k
        k = re.sub(r"\.(lora_[AB])\.weight$", rf".\1.{adapter_name}.weight", k)
        if k in own:
            mapped[k] = v
    invalidInputError(len(mapped) > 0, "no adapter weights in the checkpoint match this model")
    model.base_model.load_state_dict(mapped, strict=False)


def mark_only_lora_as_trainable(model, bias: str = "none"):
    for n, p in model.named_parameters():
        p.requires_grad_("lora_" in n)
    if bias == "all":
        for n, p in model.named_parameters():
            if n.endswith("bias") and p.is_floating_point():
                p.requires_grad_(True)


def get_peft_model(model, peft_config: LoraConfig, adapter_name: str = "default") -> PeftModel:
    """Wrap ``model`` with LoRA adapters on its target linears (reference qlora.py:282-301)."""
    peft_config.base_model_name_or_path = getattr(model, "name_or_path", None) or \
        getattr(getattr(model, "config", None), "_name_or_path", None)
    return PeftModel(model, peft_config, adapter_name)


def prepare_model_for_kbit_training(model, use_gradient_checkpointing=True, gradient_checkpointing_kwargs=None):
    """Freeze the base, keep 1-D parameters (norms) in fp32, make the embedding output require grad so that
    checkpointed blocks get gradients, and switch gradient checkpointing on (reference qlora.py:304-352)."""
    for _, p in model.named_parameters():
        p.requires_grad_(False)
    for p in model.parameters():
        if hasattr(p, "qtype"):
            continue    # packed low-bit bytes (some formats are viewed as bf16): not a floating-point tensor
        if p.dtype in (torch.float16, torch.bfloat16) and p.dim() == 1:
            p.data = p.data.to(torch.float32)
    if use_gradient_checkpointing:
        if hasattr(model, "enable_input_require_grads"):
            model.enable_input_require_grads()
        else:
            model.get_input_embeddings().register_forward_hook(lambda m, i, o: o.requires_grad_(True))
        if hasattr(model, "gradient_checkpointing_enable"):
            kw = gradient_checkpointing_kwargs or {"use_reentrant": False}
            try:
                model.gradient_checkpointing_enable(gradient_checkpointing_kwargs=kw)
            except TypeError:
                model.gradient_checkpointing_enable()
    for m in model.modules():
        if isinstance(m, LowBitLinear):
            m.compute_dtype = torch.bfloat16 if next(model.parameters()).is_cuda else torch.float32
    return model


def cast_lora_weight(model, dtype=torch.bfloat16):
    """LoRA A/B to ``dtype``, norms to fp32, lm_head/embeddings to ``dtype`` (reference qlora.py:377-391)."""
    for name, module in model.named_modules():
        if isinstance(module, LowBitLinear):
            module.compute_dtype = dtype
        if isinstance(module, _LoraBase):
            module.lora_A.to(dtype)
            module.lora_B.to(dtype)
        elif isinstance(module, BF16Linear):
            module.to(dtype)
            module.compute_dtype = dtype
        if "norm" in name:
            module.to(torch.float32)
        if ("lm_head" in name or "embed_tokens" in name) and hasattr(module, "weight") and \
                module.weight.dtype == torch.float32:
            module.to(dtype)
    return model


@dataclass
class TrainingArguments:
    """Arguments of ``ipex_llm_b200.train.Trainer`` with the reference's field names (HF ``TrainingArguments``
    subset; bf16 is forced on the GPU as in reference qlora.py:355-374)."""
    output_dir: str = "./outputs"
    per_device_train_batch_size: int = 4
    gradient_accumulation_steps: int = 1
    num_train_epochs: float = 1.0
    max_steps: int = -1
    learning_rate: float = 2e-4
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_epsilon: float = 1e-8
    max_grad_norm: float = 1.0
    warmup_steps: int = 0
    warmup_ratio: float = 0.0
    lr_scheduler_type: str = "linear"
    logging_steps: int = 10
    save_steps: int = 0
    save_total_limit: Optional[int] = None
    bf16: bool = True
    fp16: bool = False
    optim: str = "paged_adamw"          # adamw_torch | paged_adamw | fused_lora_adamw
    gradient_checkpointing: bool = False
    ddp_backend: str = "nccl"
    seed: int = 42
    resume_from_checkpoint: Optional[str] = None
    report_to: List[str] = field(default_factory=list)
    dataloader_num_workers: int = 0
    group_by_length: bool = False
    deepspeed: Optional[str] = None     # accepted for script compatibility; ZeRO-1 sharding is built in
