"""``IpexLLM`` for LlamaIndex: ``complete`` / ``stream_complete`` / ``chat`` over a low-bit model
(reference: python/llm/src/ipex_llm/llamaindex/llms/bigdlllm.py:108-540).  Stand-alone when ``llama_index`` is not
installed: the response objects are small dataclasses with the same ``text`` / ``delta`` / ``message`` fields."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Iterator, List, Optional, Sequence

DEFAULT_HUGGINGFACE_MODEL = "meta-llama/Llama-2-7b-chat-hf"


@dataclass
class CompletionResponse:
    text: str
    delta: Optional[str] = None
    raw: Optional[dict] = None


@dataclass
class ChatMessage:
    role: str = "user"
    content: str = ""


@dataclass
class ChatResponse:
    message: ChatMessage = field(default_factory=ChatMessage)
    delta: Optional[str] = None


class IpexLLM:
    def __init__(self, model_name: str = DEFAULT_HUGGINGFACE_MODEL, model: Any = None, tokenizer: Any = None,
                 tokenizer_name: Optional[str] = None, context_window: int = 4096, max_new_tokens: int = 256,
                 load_in_4bit: bool = True, load_in_low_bit: Optional[str] = None, load_low_bit: bool = False,
                 device_map: str = "cuda", generate_kwargs: Optional[dict] = None, model_kwargs: Optional[dict] = None,
                 tokenizer_kwargs: Optional[dict] = None, messages_to_prompt: Optional[Callable] = None,
                 completion_to_prompt: Optional[Callable] = None, stopping_ids: Optional[List[int]] = None,
                 system_prompt: str = ""):
        import torch
        kw = dict(model_kwargs or {})
        if model is None:
            from ...transformers import AutoModelForCausalLM
            if load_low_bit:
                model = AutoModelForCausalLM.load_low_bit(model_name, **kw)
            elif load_in_low_bit:
                model = AutoModelForCausalLM.from_pretrained(model_name, load_in_low_bit=load_in_low_bit, **kw)
            else:
                model = AutoModelForCausalLM.from_pretrained(model_name, load_in_4bit=load_in_4bit, **kw)
            if device_map in ("cuda", "xpu", "gpu") and torch.cuda.is_available():
                model = model.to("cuda")
        if tokenizer is None:
            from transformers import AutoTokenizer
            tokenizer = AutoTokenizer.from_pretrained(tokenizer_name or model_name, **(tokenizer_kwargs or {}))
        self._model, self._tokenizer = model, tokenizer
        self.model_name, self.context_window, self.max_new_tokens = model_name, context_window, max_new_tokens
        self.generate_kwargs = dict(generate_kwargs or {})
        self.messages_to_prompt = messages_to_prompt or self._default_messages_to_prompt
        self.completion_to_prompt = completion_to_prompt or (lambda s: s)
        self.stopping_ids = list(stopping_ids or [])
        self.system_prompt = system_prompt

    @classmethod
    def from_model_id(cls, model_name: str, **kwargs):
        return cls(model_name=model_name, **kwargs)

    @classmethod
    def from_model_id_low_bit(cls, model_name: str, **kwargs):
        return cls(model_name=model_name, load_low_bit=True, **kwargs)

    @classmethod
    def class_name(cls) -> str:
        return "IpexLLM"

    @property
    def metadata(self):
        return {"context_window": self.context_window, "num_output": self.max_new_tokens,
                "model_name": self.model_name}

    @staticmethod
    def _default_messages_to_prompt(messages: Sequence[ChatMessage]) -> str:
        return "".join(f"{m.role}: {m.content}\n" for m in messages) + "assistant: "

    def _ids(self, prompt: str):
        dev = next(self._model.parameters()).device
        return self._tokenizer(prompt, return_tensors="pt")["input_ids"].to(dev)

    def complete(self, prompt: str, formatted: bool = False, **kwargs) -> CompletionResponse:
        import torch
        full = prompt if formatted else self.completion_to_prompt(self.system_prompt + prompt)
        ids = self._ids(full)
        with torch.no_grad():
            out = self._model.generate(ids, max_new_tokens=self.max_new_tokens, **{**self.generate_kwargs, **kwargs})
        toks = out[0][ids.shape[1]:]
        return CompletionResponse(text=self._tokenizer.decode(toks, skip_special_tokens=True),
                                  raw={"model_output": toks})

    def stream_complete(self, prompt: str, formatted: bool = False, **kwargs) -> Iterator[CompletionResponse]:
        from threading import Thread
        from transformers import TextIteratorStreamer
        full = prompt if formatted else self.completion_to_prompt(self.system_prompt + prompt)
        ids = self._ids(full)
        streamer = TextIteratorStreamer(self._tokenizer, skip_prompt=True, skip_special_tokens=True)
        th = Thread(target=lambda: self._model.generate(ids, streamer=streamer, max_new_tokens=self.max_new_tokens,
                                                        **{**self.generate_kwargs, **kwargs}), daemon=True)
        th.start()
        text = ""
        for piece in streamer:
            text += piece
            yield CompletionResponse(text=text, delta=piece)
        th.join()

    def chat(self, messages: Sequence[ChatMessage], **kwargs) -> ChatResponse:
        r = self.complete(self.messages_to_prompt(messages), formatted=True, **kwargs)
        return ChatResponse(message=ChatMessage(role="assistant", content=r.text))

    def stream_chat(self, messages: Sequence[ChatMessage], **kwargs) -> Iterator[ChatResponse]:
        for r in self.stream_complete(self.messages_to_prompt(messages), formatted=True, **kwargs):
            yield ChatResponse(message=ChatMessage(role="assistant", content=r.text), delta=r.delta)
