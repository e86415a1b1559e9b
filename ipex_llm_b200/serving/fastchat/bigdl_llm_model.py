"""FastChat model adapters: how FastChat's stock ``model_worker`` / CLI load a path with this package.

Counterpart of python/llm/src/ipex_llm/serving/fastchat/bigdl_llm_model.py:42-289: ``BigDLLLMAdapter`` claims model
paths that contain ``bigdl`` (a Hugging Face checkpoint, packed to 4 bits on load), ``BigDLLMLOWBITAdapter`` those that
contain ``bigdl-lowbit`` (a ``save_low_bit`` directory), and ``patch_fastchat()`` puts both in front of FastChat's
adapter list and swaps its ``load_model`` for one that understands the ``xpu`` / ``cuda`` device names.  FastChat is
optional: without it the adapters are still usable directly and ``patch_fastchat`` reports that nothing was patched.
"""
from __future__ import annotations

import torch

try:                                               # pragma: no cover - depends on the optional package
    from fastchat.model.model_adapter import BaseModelAdapter as _Base
except Exception:  # noqa: BLE001
    class _Base:
        """Stand-in with FastChat's adapter contract."""
        use_fast_tokenizer = True

        def match(self, model_path: str):
            return True

        def get_default_conv_template(self, model_path: str):
            return {"name": "one_shot"}

is_fastchat_patched = False


def _tokenizer(model_path, **kw):
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(model_path, trust_remote_code=True, **kw)


class BigDLLLMAdapter(_Base):
    """Model paths containing ``bigdl``: Hugging Face checkpoint, ``load_in_4bit`` (or the ``load_in_low_bit`` given)."""

    def match(self, model_path: str):
        return "bigdl" in model_path.lower()

    def load_model(self, model_path: str, from_pretrained_kwargs: dict):
        from ...transformers import AutoModel, AutoModelForCausalLM
        kw = dict(from_pretrained_kwargs or {})
        kw.pop("revision", None)
        if "load_in_low_bit" not in kw:
            kw.setdefault("load_in_4bit", True)
        tok = _tokenizer(model_path, use_fast=False) if not self.use_fast_tokenizer else _tokenizer(model_path)
        cls = AutoModel if "chatglm" in model_path.lower() else AutoModelForCausalLM
        model = cls.from_pretrained(model_path, trust_remote_code=True, use_cache=True, **kw)
        return model, tok


class BigDLLMLOWBITAdapter(_Base):
    """Model paths containing ``bigdl-lowbit``: a directory written by ``save_low_bit``."""

    def match(self, model_path: str):
        return "bigdl-lowbit" in model_path.lower()

    def load_model(self, model_path: str, from_pretrained_kwargs: dict):
        from ...transformers import AutoModelForCausalLM
        kw = {k: v for k, v in (from_pretrained_kwargs or {}).items() if k in ("torch_dtype", "device")}
        return AutoModelForCausalLM.load_low_bit(model_path, **kw), _tokenizer(model_path)


ADAPTERS = [BigDLLMLOWBITAdapter(), BigDLLLMAdapter()]         # the more specific pattern first


def get_model_adapter(model_path: str):
    for a in ADAPTERS:
        if a.match(model_path):
            return a
    return None


def load_model(model_path: str, device: str = "cuda", num_gpus: int = 1, max_gpu_memory=None, dtype=None,
               load_8bit: bool = False, cpu_offloading: bool = False, gptq_config=None, awq_config=None,
               exllama_config=None, xft_config=None, revision: str = "main", debug: bool = False,
               load_in_low_bit: str = None):
    """FastChat's ``load_model`` signature.  Paths one of the adapters claims are loaded by it; any other path is
    loaded as a Hugging Face checkpoint packed to ``load_in_low_bit`` (default sym_int4)."""
    kwargs = {"torch_dtype": dtype or (torch.float32 if device == "cpu" else torch.float16)}
    if load_in_low_bit:
        kwargs["load_in_low_bit"] = load_in_low_bit
    adapter = get_model_adapter(model_path) or BigDLLLMAdapter()
    model, tok = adapter.load_model(model_path, kwargs)
    if device in ("cuda", "xpu", "gpu") and torch.cuda.is_available():
        model = model.to("cuda")
    if debug:
        print(model)
    return model.eval(), tok


def patch_fastchat() -> bool:
    """Register the adapters with an installed FastChat and route its ``load_model`` here.  Returns whether FastChat
    was found (idempotent)."""
    global is_fastchat_patched
    if is_fastchat_patched:
        return True
    try:
        import fastchat.model.model_adapter as ma
    except Exception:  # noqa: BLE001
        return False
    for a in reversed(ADAPTERS):
        ma.model_adapters.insert(0, a)
    ma.load_model = load_model
    try:
        import fastchat.serve.model_worker as mw
        mw.load_model = load_model
    except Exception:  # noqa: BLE001
        pass
    is_fastchat_patched = True
    return True
