"""Request / response schemas of the HTTP server: OpenAI-compatible (``/v1/chat/completions``,
``/v1/completions``, ``/v1/models``) and TGI-style (``/generate``, ``/generate_stream``).

Field names follow the public OpenAI / text-generation-inference APIs, which is what the reference's
python/llm/src/ipex_llm/serving/fastapi/openai_protocol.py and tgi_protocol.py model as well.
"""
from __future__ import annotations

import time
import uuid
from typing import Dict, List, Literal, Optional, Union

from pydantic import BaseModel, Field


def _rid(prefix):
    return f"{prefix}-{uuid.uuid4().hex}"


class UsageInfo(BaseModel):
    prompt_tokens: int = 0
    total_tokens: int = 0
    completion_tokens: Optional[int] = 0


class ModelCard(BaseModel):
    id: str
    object: str = "model"
    created: int = Field(default_factory=lambda: int(time.time()))
    owned_by: str = "ipex-llm"


class ModelList(BaseModel):
    object: str = "list"
    data: List[ModelCard] = Field(default_factory=list)


class ChatMessage(BaseModel):
    role: str
    content: Union[str, List[Dict], None] = None


class _SamplingMixin(BaseModel):
    model: str = ""
    max_tokens: Optional[int] = 256
    temperature: Optional[float] = 1.0
    top_p: Optional[float] = 1.0
    top_k: Optional[int] = -1
    n: Optional[int] = 1
    stop: Optional[Union[str, List[str]]] = None
    stream: Optional[bool] = False
    presence_penalty: Optional[float] = 0.0
    frequency_penalty: Optional[float] = 0.0
    repetition_penalty: Optional[float] = 1.0
    seed: Optional[int] = None
    user: Optional[str] = None


class ChatCompletionRequest(_SamplingMixin):
    messages: List[ChatMessage]


class CompletionRequest(_SamplingMixin):
    prompt: Union[str, List[str]]
    echo: Optional[bool] = False


class ChatCompletionResponseChoice(BaseModel):
    index: int
    message: ChatMessage
    finish_reason: Optional[Literal["stop", "length"]] = None


class ChatCompletionResponse(BaseModel):
    id: str = Field(default_factory=lambda: _rid("chatcmpl"))
    object: str = "chat.completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str = ""
    choices: List[ChatCompletionResponseChoice]
    usage: UsageInfo = Field(default_factory=UsageInfo)


class DeltaMessage(BaseModel):
    role: Optional[str] = None
    content: Optional[str] = None


class ChatCompletionResponseStreamChoice(BaseModel):
    index: int
    delta: DeltaMessage
    finish_reason: Optional[Literal["stop", "length"]] = None


class ChatCompletionStreamResponse(BaseModel):
    id: str = Field(default_factory=lambda: _rid("chatcmpl"))
    object: str = "chat.completion.chunk"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str = ""
    choices: List[ChatCompletionResponseStreamChoice]


class CompletionResponseChoice(BaseModel):
    index: int
    text: str
    finish_reason: Optional[Literal["stop", "length"]] = None


class CompletionResponse(BaseModel):
    id: str = Field(default_factory=lambda: _rid("cmpl"))
    object: str = "text_completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str = ""
    choices: List[CompletionResponseChoice]
    usage: UsageInfo = Field(default_factory=UsageInfo)


class CompletionStreamResponse(BaseModel):
    id: str = Field(default_factory=lambda: _rid("cmpl"))
    object: str = "text_completion"
    created: int = Field(default_factory=lambda: int(time.time()))
    model: str = ""
    choices: List[CompletionResponseChoice]


# ---- TGI style -------------------------------------------------------------------------------------
class Parameters(BaseModel):
    max_new_tokens: int = 32
    do_sample: bool = False
    temperature: Optional[float] = None
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    repetition_penalty: Optional[float] = None
    stop: Optional[List[str]] = None
    seed: Optional[int] = None
    min_new_tokens: Optional[int] = None
    return_full_text: Optional[bool] = False


class GenerateRequest(BaseModel):
    inputs: str
    parameters: Parameters = Field(default_factory=Parameters)
    stream: bool = False
    req_type: str = "completion"


class GenerateResponse(BaseModel):
    generated_text: str
    generate_text: Optional[str] = None     # the key the reference's /generate returns
    prompt_tokens: int = 0
    generated_tokens: int = 0
    finish_reason: str = "length"


class StreamToken(BaseModel):
    text: str


class StreamResponse(BaseModel):
    token: StreamToken
    generated_text: Optional[str] = None
    finish_reason: Optional[str] = None
