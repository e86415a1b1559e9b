"""LangChain LLMs over the vLLM adapter (reference: python/llm/src/ipex_llm/langchain/vllm/vllm.py:52-230).

``VLLM`` builds ``ipex_llm_b200.vllm.engine.IPEXLLMClass`` (``vllm.LLM`` whose workers convert the loaded model to
``load_in_low_bit``) and turns LangChain's generate call into ``SamplingParams`` + ``LLM.generate``; ``VLLMOpenAI``
points LangChain's OpenAI client at a vLLM OpenAI-compatible server.  Both import their dependencies lazily so the
package imports without LangChain or vLLM installed.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

try:                                               # pragma: no cover - depends on the optional package
    from langchain_core.language_models.llms import BaseLLM as _Base
    from langchain_core.outputs import Generation, LLMResult
    _HAS_LC = True
except Exception:  # noqa: BLE001
    _Base = object
    _HAS_LC = False

    class Generation:                                   # minimal stand-ins with the same fields
        def __init__(self, text: str):
            self.text = text

    class LLMResult:
        def __init__(self, generations):
            self.generations = generations

_SAMPLING_KEYS = ("n", "best_of", "presence_penalty", "frequency_penalty", "temperature", "top_p", "top_k", "stop",
                  "ignore_eos", "max_tokens", "logprobs", "use_beam_search")


class VLLM(_Base):
    model: str = ""
    tensor_parallel_size: int = 1
    trust_remote_code: bool = False
    n: int = 1
    best_of: Optional[int] = None
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    use_beam_search: bool = False
    stop: Optional[List[str]] = None
    ignore_eos: bool = False
    max_new_tokens: int = 512
    logprobs: Optional[int] = None
    dtype: str = "auto"
    download_dir: Optional[str] = None
    vllm_kwargs: Dict[str, Any] = {}
    load_in_low_bit: str = "sym_int4"
    device: str = "cuda"
    client: Any = None

    def __init__(self, **kwargs):
        if _HAS_LC:
            super().__init__(**kwargs)
        else:
            for k, v in kwargs.items():
                setattr(self, k, v)
        if self.client is None:
            from ...vllm.engine import IPEXLLMClass
            self.client = IPEXLLMClass(model=self.model, tensor_parallel_size=self.tensor_parallel_size,
                                       trust_remote_code=self.trust_remote_code, dtype=self.dtype,
                                       download_dir=self.download_dir, load_in_low_bit=self.load_in_low_bit,
                                       **(self.vllm_kwargs or {}))

    @property
    def _default_params(self) -> Dict[str, Any]:
        return {"n": self.n, "best_of": self.best_of, "max_tokens": self.max_new_tokens, "top_k": self.top_k,
                "top_p": self.top_p, "temperature": self.temperature, "presence_penalty": self.presence_penalty,
                "frequency_penalty": self.frequency_penalty, "stop": self.stop, "ignore_eos": self.ignore_eos,
                "use_beam_search": self.use_beam_search, "logprobs": self.logprobs}

    def _sampling_params(self, stop, kwargs):
        params = {**self._default_params, **{k: v for k, v in kwargs.items() if k in _SAMPLING_KEYS}}
        if stop:
            params["stop"] = stop
        params = {k: v for k, v in params.items() if v is not None}
        try:
            from vllm import SamplingParams
        except Exception:  # noqa: BLE001 (a client double in tests takes the plain dictionary)
            return params
        import inspect
        accepted = set(inspect.signature(SamplingParams).parameters)
        return SamplingParams(**{k: v for k, v in params.items() if k in accepted})

    def _generate(self, prompts: List[str], stop: Optional[List[str]] = None, run_manager=None, **kwargs):
        outputs = self.client.generate(prompts, self._sampling_params(stop, kwargs))
        return LLMResult(generations=[[Generation(text=o.text) for o in out.outputs] for out in outputs])

    def generate_texts(self, prompts: List[str], stop: Optional[List[str]] = None, **kwargs) -> List[str]:
        """Plain-Python convenience (also the path used without LangChain installed)."""
        return [g[0].text for g in self._generate(prompts, stop, **kwargs).generations]

    @property
    def _llm_type(self) -> str:
        return "vllm"


def VLLMOpenAI(**kwargs):
    """LangChain's OpenAI completion client configured for a vLLM OpenAI-compatible server (``openai_api_base``,
    ``openai_api_key``, ``model_name`` as in the reference class of the same name)."""
    try:
        from langchain_openai import OpenAI
    except Exception as e:  # noqa: BLE001
        raise ImportError("VLLMOpenAI needs the `langchain-openai` package") from e
    kwargs.setdefault("openai_api_key", "EMPTY")
    return OpenAI(**kwargs)
