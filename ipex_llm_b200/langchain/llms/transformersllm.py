"""``TransformersLLM``: a LangChain LLM over a low-bit model
(reference: python/llm/src/ipex_llm/langchain/llms/transformersllm.py:62-260, ``from_model_id`` /
``from_model_id_low_bit`` / ``_call`` with stop words and streaming)."""
from __future__ import annotations

from typing import Any, List, Optional

try:                                               # pragma: no cover - depends on the optional package
    from langchain_core.language_models.llms import LLM as _Base
    _HAS_LC = True
except Exception:  # noqa: BLE001
    _Base = object
    _HAS_LC = False

DEFAULT_MODEL_ID = "gpt2"


def _enforce_stop(text: str, stop: Optional[List[str]]) -> str:
    for s in stop or []:
        i = text.find(s)
        if i >= 0:
            text = text[:i]
    return text


class TransformersLLM(_Base):
    model_id: str = DEFAULT_MODEL_ID
    model_kwargs: Optional[dict] = None
    model: Any = None
    tokenizer: Any = None
    streaming: bool = False

    def __init__(self, model=None, tokenizer=None, model_id: str = DEFAULT_MODEL_ID, model_kwargs: Optional[dict] = None,
                 streaming: bool = False, **kwargs):
        if _HAS_LC:
            super().__init__(model=model, tokenizer=tokenizer, model_id=model_id, model_kwargs=model_kwargs,
                             streaming=streaming, **kwargs)
        else:
            self.model, self.tokenizer, self.model_id = model, tokenizer, model_id
            self.model_kwargs, self.streaming = model_kwargs, streaming

    # ---- constructors ---------------------------------------------------------------------------------
    @classmethod
    def from_model_id(cls, model_id: str, model_kwargs: Optional[dict] = None, device_map: str = "cuda",
                      tokenizer_id: Optional[str] = None, **kwargs):
        """Load a Hugging Face checkpoint with ``load_in_4bit=True``."""
        from transformers import AutoTokenizer
        from ...transformers import AutoModel, AutoModelForCausalLM
        kw = dict(model_kwargs or {})
        tok = AutoTokenizer.from_pretrained(tokenizer_id or model_id, **{k: v for k, v in kw.items()
                                                                         if k == "trust_remote_code"})
        load = dict(load_in_4bit=True) if "load_in_low_bit" not in kw else {}
        try:
            model = AutoModelForCausalLM.from_pretrained(model_id, **load, **kw)
        except Exception:  # noqa: BLE001
            model = AutoModel.from_pretrained(model_id, **load, **kw)
        model = cls._place(model, device_map)
        return cls(model=model, tokenizer=tok, model_id=model_id, model_kwargs=kw, **kwargs)

    @classmethod
    def from_model_id_low_bit(cls, model_id: str, model_kwargs: Optional[dict] = None, device_map: str = "cuda",
                              tokenizer_id: Optional[str] = None, **kwargs):
        """Load a checkpoint saved with ``save_low_bit``."""
        from transformers import AutoTokenizer
        from ...transformers import AutoModel, AutoModelForCausalLM
        kw = dict(model_kwargs or {})
        tok = AutoTokenizer.from_pretrained(tokenizer_id or model_id)
        try:
            model = AutoModelForCausalLM.load_low_bit(model_id, **kw)
        except Exception:  # noqa: BLE001
            model = AutoModel.load_low_bit(model_id, **kw)
        model = cls._place(model, device_map)
        return cls(model=model, tokenizer=tok, model_id=model_id, model_kwargs=kw, **kwargs)

    @staticmethod
    def _place(model, device_map):
        import torch
        if device_map in ("cuda", "xpu", "gpu") and torch.cuda.is_available():
            return model.to("cuda")
        return model

    # ---- LangChain protocol -------------------------------------------------------------------------------
    @property
    def _identifying_params(self):
        return {"model_id": self.model_id, "model_kwargs": self.model_kwargs}

    @property
    def _llm_type(self) -> str:
        return "IpexLLM"

    def _call(self, prompt: str, stop: Optional[List[str]] = None, run_manager=None, **kwargs) -> str:
        import torch
        dev = next(self.model.parameters()).device
        ids = self.tokenizer.encode(prompt, return_tensors="pt").to(dev)
        gen = dict(max_new_tokens=kwargs.pop("max_new_tokens", 64), do_sample=kwargs.pop("do_sample", False))
        gen.update(kwargs)
        if self.streaming and run_manager is not None:
            from threading import Thread
            from transformers import TextIteratorStreamer
            streamer = TextIteratorStreamer(self.tokenizer, skip_prompt=True, skip_special_tokens=True)
            th = Thread(target=lambda: self.model.generate(ids, streamer=streamer, **gen), daemon=True)
            th.start()
            text = ""
            for piece in streamer:
                text += piece
                run_manager.on_llm_new_token(piece)
            th.join()
        else:
            with torch.no_grad():
                out = self.model.generate(ids, **gen)
            text = self.tokenizer.decode(out[0][ids.shape[1]:], skip_special_tokens=True)
        return _enforce_stop(text, stop)

    if not _HAS_LC:
        def invoke(self, prompt: str, stop: Optional[List[str]] = None, **kwargs) -> str:
            return self._call(prompt, stop=stop, **kwargs)

        __call__ = invoke


class TransformersPipelineLLM(TransformersLLM):
    """The reference's pipeline flavour (same constructor surface; generation goes through ``generate``)."""

    @property
    def _llm_type(self) -> str:
        return "IpexLLM_pipeline"
