"""Finetuning: trainer, callbacks, optimizers (reference: HF Trainer + peft + DeepSpeed driven by the example
scripts under python/llm/example/GPU/LLM-Finetuning)."""
from .trainer import Trainer, TrainerCallback, TrainerControl, TrainerState, default_collator  # noqa: F401
from ..parallel.dp import FusedLoraAdamW, PagedAdamW  # noqa: F401
