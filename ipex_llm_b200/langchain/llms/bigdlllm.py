"""LangChain LLMs over the llama-cpp-python style classes (``ipex_llm.models`` / ``ggml.model``).

Counterpart of python/llm/src/ipex_llm/langchain/llms/bigdlllm.py:58-693: ``BigdlNativeLLM(model_family=...)`` and
the per-family ``LlamaLLM`` / ``BloomLLM`` / ``GptneoxLLM`` / ``StarcoderLLM`` (plus ``ChatGLMLLM``), with the sampling
fields of the reference (``max_tokens``, ``temperature``, ``top_p``, ``top_k``, ``repeat_penalty``, ``stop``, ``echo``,
``streaming``), ``_call``, ``stream`` and ``get_num_tokens``.  The classes subclass LangChain's ``LLM`` when
``langchain_core`` is importable and are plain Python objects with the same methods otherwise.
"""
from __future__ import annotations

from typing import Any, Dict, Iterator, List, Optional

try:                                               # pragma: no cover - depends on the optional package
    from langchain_core.language_models.llms import LLM as _Base
    _HAS_LC = True
except Exception:  # noqa: BLE001
    _Base = object
    _HAS_LC = False

_FIELDS = dict(model_path=None, n_ctx=512, seed=-1, n_threads=2, n_batch=512, max_tokens=256, temperature=0.8,
               top_p=0.95, top_k=40, repeat_penalty=1.1, echo=False, stop=None, streaming=True, low_bit="sym_int4",
               device="auto")


def _native_class(family: str):
    from ...ggml.model import generic
    table = {"llama": generic.Llama, "bloom": generic.Bloom, "gptneox": generic.Gptneox,
             "starcoder": generic.Starcoder, "chatglm": generic.ChatGLM}
    if family not in table:
        raise ValueError(f"Unknown model family: {family}, expected one of {sorted(table)}")
    return table[family]


class _BaseCausalLM(_Base):
    """Shared implementation; ``ggml_family`` names the native class."""
    ggml_family: Optional[str] = None
    client: Any = None
    model_family: str = "llama"
    model_path: Optional[str] = None
    n_ctx: int = 512
    seed: int = -1
    n_threads: Optional[int] = 2
    n_batch: int = 512
    max_tokens: int = 256
    temperature: float = 0.8
    top_p: float = 0.95
    top_k: int = 40
    repeat_penalty: float = 1.1
    echo: bool = False
    stop: Optional[List[str]] = None
    streaming: bool = True
    low_bit: str = "sym_int4"
    device: str = "auto"

    def __init__(self, client=None, **kwargs):
        family = kwargs.pop("model_family", None) or type(self).ggml_family or "llama"
        fields = {k: kwargs.pop(k, v) for k, v in _FIELDS.items()}
        if client is None:
            if not fields["model_path"]:
                raise ValueError("model_path is required")
            client = _native_class(family)(fields["model_path"], n_ctx=fields["n_ctx"], n_threads=fields["n_threads"],
                                           seed=fields["seed"], n_batch=fields["n_batch"], low_bit=fields["low_bit"],
                                           device=fields["device"])
        if _HAS_LC:
            super().__init__(client=client, model_family=family, **fields, **kwargs)
        else:
            self.client, self.model_family = client, family
            for k, v in fields.items():
                setattr(self, k, v)

    # ---- LangChain contract -----------------------------------------------------------------------------
    @property
    def _default_params(self) -> Dict[str, Any]:
        return {"max_tokens": self.max_tokens, "temperature": self.temperature, "top_p": self.top_p,
                "top_k": self.top_k, "repeat_penalty": self.repeat_penalty, "echo": self.echo,
                "stop": list(self.stop or [])}

    @property
    def _identifying_params(self) -> Dict[str, Any]:
        return {"model_path": self.model_path, "model_family": self.model_family, **self._default_params}

    @property
    def _llm_type(self) -> str:
        return "BigDL"

    def _get_parameters(self, stop: Optional[List[str]] = None) -> Dict[str, Any]:
        if self.stop and stop is not None:
            raise ValueError("`stop` found in both the input and default params.")
        params = self._default_params
        params["stop"] = list(self.stop or stop or [])
        return params

    def _call(self, prompt: str, stop: Optional[List[str]] = None, run_manager=None, **kwargs) -> str:
        if self.streaming:
            return "".join(self.stream(prompt, stop=stop, run_manager=run_manager))
        params = {**self._get_parameters(stop), **kwargs}
        return self.client(prompt, **params)["choices"][0]["text"]

    def stream(self, prompt: str, stop: Optional[List[str]] = None, run_manager=None, **kwargs) -> Iterator[str]:
        """Text pieces as they are generated; every piece is also sent to ``run_manager.on_llm_new_token``."""
        params = {**self._get_parameters(stop), **kwargs}
        for chunk in self.client(prompt, stream=True, **params):
            piece = chunk["choices"][0]["text"]
            if run_manager is not None:
                run_manager.on_llm_new_token(token=piece, verbose=getattr(self, "verbose", False))
            yield piece

    def get_num_tokens(self, text: str) -> int:
        return len(self.client.tokenize(text.encode("utf-8")))

    def __call__(self, prompt: str, stop: Optional[List[str]] = None, **kwargs) -> str:
        if _HAS_LC:
            return super().__call__(prompt, stop=stop, **kwargs)
        return self._call(prompt, stop=stop, **kwargs)

    invoke = __call__ if not _HAS_LC else _Base.invoke


class BigdlNativeLLM(_BaseCausalLM):
    """``BigdlNativeLLM(model_family="llama", model_path=...)`` (deprecated spelling of the per-family classes)."""


class LlamaLLM(_BaseCausalLM):
    ggml_family = "llama"


class BloomLLM(_BaseCausalLM):
    ggml_family = "bloom"


class GptneoxLLM(_BaseCausalLM):
    ggml_family = "gptneox"


class StarcoderLLM(_BaseCausalLM):
    ggml_family = "starcoder"


class ChatGLMLLM(_BaseCausalLM):
    ggml_family = "chatglm"


__all__ = ["BigdlNativeLLM", "LlamaLLM", "BloomLLM", "GptneoxLLM", "StarcoderLLM", "ChatGLMLLM"]
