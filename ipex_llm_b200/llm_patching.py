"""``llm_patch`` / ``llm_unpatch``: make third-party training scripts written for ``transformers`` + ``peft``
pick up the low-bit classes (reference: python/llm/src/ipex_llm/llm_patching.py:35-85).

``peft`` is not a dependency of this package: ``llm_patch(train=True)`` installs a minimal ``peft`` module
(``LoraConfig``, ``get_peft_model``, ``prepare_model_for_kbit_training``, ``PeftModel``) backed by
``ipex_llm_b200.transformers.qlora`` when the real one is absent, and patches the real one when present.
"""
from __future__ import annotations

import importlib
import sys
import types

import transformers

_is_patched = False
_saved = []


def _replace_attr(obj, name, value):
    _saved.append((obj, name, getattr(obj, name, None), hasattr(obj, name)))
    setattr(obj, name, value)


def llm_patch(train=False):
    """Must run before ``import peft`` in the training script."""
    global _is_patched
    if _is_patched:
        return
    from .transformers import AutoModel, AutoModelForCausalLM
    _replace_attr(transformers, "AutoModelForCausalLM", AutoModelForCausalLM)
    _replace_attr(transformers, "LlamaForCausalLM", AutoModelForCausalLM)
    _replace_attr(transformers, "AutoModel", AutoModel)
    if train:
        from .transformers import qlora
        try:
            peft = importlib.import_module("peft")
            real = True
        except ImportError:
            peft = types.ModuleType("peft")
            sys.modules["peft"] = peft
            _saved.append((sys.modules, "peft", None, False))
            real = False
        for name in ("get_peft_model", "prepare_model_for_kbit_training", "LoraConfig", "PeftModel",
                     "TrainingArguments"):
            if hasattr(qlora, name) and (real or name != "TrainingArguments"):
                _replace_attr(peft, name, getattr(qlora, name))
        _replace_attr(transformers, "TrainingArguments", qlora.TrainingArguments)
    _is_patched = True


def llm_unpatch():
    global _is_patched
    if not _is_patched:
        return
    for obj, name, old, existed in reversed(_saved):
        if obj is sys.modules:
            sys.modules.pop(name, None)
        elif existed:
            setattr(obj, name, old)
        else:
            try:
                delattr(obj, name)
            except AttributeError:
                pass
    _saved.clear()
    _is_patched = False
