"""Patch vLLM so that every model it loads has its linear layers replaced by ``vLLMLowBitLinear``.

Reference: python/llm/src/ipex_llm/vllm/xpu/model_convert.py:35-180 (``_ipex_llm_convert(load_in_low_bit)`` patches the
model runner's ``load_model`` to: load on the host, ``optimize_model(low_bit)`` with vLLM's parallel layers recognised
by the converter, move to the device; and patches ``LogitsProcessor._get_logits`` for the converted ``lm_head``).
The converter of this package already recognises vLLM's ``RowParallelLinear`` / ``ColumnParallelLinear`` /
``QKVParallelLinear`` / ``MergedColumnParallelLinear`` / ``ParallelLMHead`` (transformers/convert.py,
``is_linear_module``) and gives row-parallel layers the tensor-parallel group as ``mp_group``.
"""
from __future__ import annotations

import os

import torch

_PATCHED = {}


def convert_vllm_model(model, low_bit: str, torch_dtype=torch.float16):
    """Replace the linears of an already constructed vLLM model in place."""
    from ..optimize import optimize_model
    if low_bit in ("bf16", "fp16"):
        return model
    skip = ["lm_head"] if os.environ.get("IPEX_LLM_NOT_CONVERT_LM_HEAD", "0") == "1" else None
    return optimize_model(model, low_bit=low_bit, torch_dtype=torch_dtype, optimize_llm=False,
                          modules_to_not_convert=skip)


def _get_logits(self, hidden_states, lm_head, embedding_bias=None):
    """Logits through a converted ``lm_head`` (a ``LowBitLinear`` returns a tensor, not ``(out, bias)``)."""
    out = lm_head(hidden_states)
    logits = out[0] if isinstance(out, tuple) else out
    if embedding_bias is not None:
        logits = logits + embedding_bias
    try:
        from vllm.distributed import tensor_model_parallel_gather
        logits = tensor_model_parallel_gather(logits)
    except Exception:  # noqa: BLE001 - single process
        pass
    if logits is not None and getattr(self, "org_vocab_size", None):
        logits = logits[..., : self.org_vocab_size]
    return logits


def patch_runner_class(cls, load_in_low_bit: str):
    """Wrap ``cls.load_model``: the original loads the checkpoint, then the linears of ``self.model`` are packed."""
    if cls in _PATCHED:
        return
    orig = cls.load_model
    _PATCHED[cls] = orig

    def load_model(self, *args, _orig=orig, **kwargs):
        _orig(self, *args, **kwargs)
        model = getattr(self, "model", None)
        if model is not None:
            dtype = getattr(getattr(self, "model_config", None), "dtype", torch.float16)
            self.model = convert_vllm_model(model, load_in_low_bit, dtype)

    cls.load_model = load_model


def _ipex_llm_convert(load_in_low_bit: str):
    """Install the patches.  Call before constructing ``LLM`` / the engine."""
    from vllm.model_executor.layers.logits_processor import LogitsProcessor
    runners = []
    for mod_name, cls_name in (("vllm.worker.model_runner", "GPUModelRunnerBase"),
                               ("vllm.worker.model_runner", "ModelRunner"),
                               ("vllm.v1.worker.gpu_model_runner", "GPUModelRunner")):
        try:
            mod = __import__(mod_name, fromlist=[cls_name])
            runners.append(getattr(mod, cls_name))
        except Exception:  # noqa: BLE001 - layout differs between vLLM versions
            continue
    for cls in runners:
        patch_runner_class(cls, load_in_low_bit)
    if LogitsProcessor not in _PATCHED:
        _PATCHED[LogitsProcessor] = getattr(LogitsProcessor, "_get_logits", None)
        LogitsProcessor._get_logits = _get_logits
