"""``load_model``: one call that returns ``(model, tokenizer)`` for a path and a device, used by the FastChat worker
and the benchmark scripts (reference: python/llm/src/ipex_llm/transformers/loader.py:43-173)."""
from __future__ import annotations

import time

import torch

LLAMA_IDS = ["llama", "vicuna", "llama-2", "yi"]


def load_model(model_path: str, device: str = "cuda", low_bit: str = "sym_int4", trust_remote_code: bool = True,
               speculative: bool = False, load_low_bit_model: bool = False):
    from transformers import AutoTokenizer
    from . import AutoModel, AutoModelForCausalLM
    tokenizer = AutoTokenizer.from_pretrained(model_path, trust_remote_code=trust_remote_code)
    kw = dict(trust_remote_code=trust_remote_code, use_cache=True)
    if device in ("cuda", "xpu", "gpu"):
        kw["torch_dtype"] = torch.float16
    t0 = time.perf_counter()
    cls = AutoModel if "chatglm" in model_path.lower() else AutoModelForCausalLM
    if load_low_bit_model:
        model = cls.load_low_bit(model_path, **kw)
    else:
        if speculative:
            kw["speculative"] = True
            low_bit = "fp16"
        model = cls.from_pretrained(model_path, load_in_low_bit=low_bit, **kw)
    if device in ("cuda", "xpu", "gpu") and torch.cuda.is_available():
        model = model.to("cuda")
    print(f">> loading of model costs {time.perf_counter() - t0:.2f}s")
    return model.eval(), tokenizer
