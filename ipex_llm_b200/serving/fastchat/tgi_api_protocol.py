"""Request / response models of the TGI-style API server (reference:
python/llm/src/ipex_llm/serving/fastchat/tgi_api_protocol.py).  Field names follow text-generation-inference's
``/generate`` and ``/generate_stream`` schema."""
from __future__ import annotations

import time
import uuid
from typing import List, Optional

from pydantic import BaseModel, Field


class ErrorResponse(BaseModel):
    object: str = "error"
    message: str
    code: int


class Grammar(BaseModel):
    type: str = "json"
    value: str = "string"


class GenerateParameters(BaseModel):
    best_of: Optional[int] = 1
    decoder_input_details: Optional[bool] = False
    details: Optional[bool] = False
    do_sample: Optional[bool] = False
    frequency_penalty: Optional[float] = 0.0
    grammar: Optional[Grammar] = None
    max_new_tokens: Optional[int] = 256
    repetition_penalty: Optional[float] = 1.0
    return_full_text: Optional[bool] = False
    seed: Optional[int] = None
    stop: Optional[List[str]] = None
    temperature: Optional[float] = 1.0
    top_k: Optional[int] = -1
    top_n_tokens: Optional[int] = None
    top_p: Optional[float] = 1.0
    truncate: Optional[int] = None
    typical_p: Optional[float] = None
    watermark: Optional[bool] = False


class GenerateRequest(BaseModel):
    inputs: str
    parameters: GenerateParameters = Field(default_factory=GenerateParameters)
    model: Optional[str] = None
    stream: Optional[bool] = False


class Token(BaseModel):
    id: int = -1
    text: str = ""
    logprob: Optional[float] = None
    special: bool = False


class Details(BaseModel):
    finish_reason: Optional[str] = None
    generated_tokens: int = 0
    seed: Optional[int] = None
    prefill: List[Token] = []
    tokens: List[Token] = []


class GenerateResponse(BaseModel):
    generated_text: str
    details: Optional[Details] = None


class StreamResponse(BaseModel):
    token: Token
    generated_text: Optional[str] = None
    details: Optional[Details] = None


class ModelCard(BaseModel):
    id: str
    object: str = "model"
    created: int = Field(default_factory=lambda: int(time.time()))
    owned_by: str = "ipex-llm"
    root: Optional[str] = None


class ModelList(BaseModel):
    object: str = "list"
    data: List[ModelCard] = []


def request_id() -> str:
    return f"tgi-{uuid.uuid4().hex[:24]}"
