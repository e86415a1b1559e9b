"""Reference module path ``ipex_llm.serving.fastapi.tgi_protocol`` (python/llm/src/ipex_llm/serving/fastapi/tgi_protocol.py): the TGI ``/generate`` schemas."""
from ..protocol import GenerateRequest, GenerateResponse, Parameters, StreamResponse, StreamToken  # noqa: F401
