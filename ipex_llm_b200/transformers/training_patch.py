"""Reference module path ``ipex_llm.transformers.training_patch`` (python/llm/src/ipex_llm/transformers/
training_patch.py:103-264): the reference replaces ``transformers.TrainingArguments`` device set-up so that a Trainer
lands on its device.  On CUDA the stock arguments already do; the patched class of ``qlora`` (bf16 forced, as the
reference's) is re-exported and ``patch()`` installs it."""
from .qlora import TrainingArguments  # noqa: F401


def patch():
    import transformers
    transformers.TrainingArguments = TrainingArguments
    return TrainingArguments
