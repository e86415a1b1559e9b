"""TGI-style REST front (``/generate``, ``/generate_stream``, ``/v1/models``, ``/info``, ``/health``) for workers that
speak FastChat's worker protocol (reference: python/llm/src/ipex_llm/serving/fastchat/tgi_api_server.py).

The server owns no model.  For every request it finds a worker - a fixed ``--worker-address`` or, like FastChat's
API servers, by asking a controller (``/get_worker_address``) - and relays to the worker's ``/worker_generate_stream``
(a stream of NUL-separated JSON chunks carrying the text so far), turning that into TGI's response objects:
``/generate`` returns ``{"generated_text", "details"}``, ``/generate_stream`` server-sent events with one ``token`` per
event and the full text + details on the last one.  The transport is a small injectable class so the relay logic is
tested without sockets.

    python -m ipex_llm_b200.serving.fastchat.tgi_api_server --controller-address http://localhost:21001 --port 8000
"""
from __future__ import annotations

import argparse
import json
from typing import AsyncIterator, Dict, List, Optional

from fastapi import FastAPI
from fastapi.responses import JSONResponse, StreamingResponse

from .tgi_api_protocol import (Details, ErrorResponse, GenerateRequest, GenerateResponse, ModelCard, ModelList,
                               StreamResponse, Token)


class HttpTransport:
    """Plain HTTP to the controller / worker (``aiohttp``)."""

    async def post_json(self, url: str, payload: dict) -> dict:
        import aiohttp
        async with aiohttp.ClientSession() as s:
            async with s.post(url, json=payload, timeout=aiohttp.ClientTimeout(total=30)) as r:
                return await r.json()

    async def post_stream(self, url: str, payload: dict) -> AsyncIterator[bytes]:
        import aiohttp
        async with aiohttp.ClientSession() as s:
            async with s.post(url, json=payload, timeout=aiohttp.ClientTimeout(total=None)) as r:
                async for chunk in r.content.iter_any():
                    yield chunk


def worker_payload(req: GenerateRequest, model: str) -> dict:
    """FastChat ``worker_generate_stream`` parameters for a TGI request."""
    p = req.parameters
    temperature = float(p.temperature or 0.0) if p.do_sample else 0.0
    return {"model": model, "prompt": req.inputs, "temperature": temperature,
            "top_p": float(p.top_p if p.top_p is not None else 1.0), "top_k": int(p.top_k if p.top_k else -1),
            "repetition_penalty": float(p.repetition_penalty or 1.0),
            "frequency_penalty": float(p.frequency_penalty or 0.0), "max_new_tokens": int(p.max_new_tokens or 256),
            "stop": p.stop or [], "echo": bool(p.return_full_text), "best_of": p.best_of, "seed": p.seed}


async def worker_chunks(byte_stream: AsyncIterator[bytes]) -> AsyncIterator[dict]:
    """FastChat workers delimit their JSON chunks with NUL bytes; chunks may be split across reads."""
    buf = b""
    async for part in byte_stream:
        buf += part
        while b"\0" in buf:
            raw, buf = buf.split(b"\0", 1)
            if raw.strip():
                yield json.loads(raw.decode())
    if buf.strip():
        yield json.loads(buf.decode())


class TGIApp:
    def __init__(self, controller_address: Optional[str] = None, worker_address: Optional[str] = None,
                 model_names: Optional[List[str]] = None, transport=None):
        self.controller_address, self.worker_address = controller_address, worker_address
        self.model_names = model_names or []
        self.transport = transport or HttpTransport()
        self.app = FastAPI(title="ipex-llm TGI API server")
        self._routes()

    async def _worker_for(self, model: Optional[str]) -> str:
        if self.worker_address:
            return self.worker_address
        if not self.controller_address:
            raise RuntimeError("neither a worker address nor a controller address is configured")
        if not model:
            models = (await self.transport.post_json(self.controller_address + "/list_models", {})).get("models", [])
            model = models[0] if models else ""
        addr = (await self.transport.post_json(self.controller_address + "/get_worker_address",
                                               {"model": model})).get("address", "")
        if not addr:
            raise RuntimeError(f"no worker serves model '{model}'")
        return addr

    async def _relay(self, req: GenerateRequest) -> AsyncIterator[Dict]:
        addr = await self._worker_for(req.model)
        payload = worker_payload(req, req.model or (self.model_names[0] if self.model_names else ""))
        stream = self.transport.post_stream(addr + "/worker_generate_stream", payload)
        async for chunk in worker_chunks(stream):
            yield chunk

    def _routes(self):
        app = self.app

        @app.get("/health")
        async def health():
            return {"status": "ok"}

        @app.get("/info")
        async def info():
            return {"model_id": self.model_names[0] if self.model_names else None, "router": "ipex-llm-tgi",
                    "controller": self.controller_address, "worker": self.worker_address}

        @app.get("/v1/models")
        async def models():
            names = list(self.model_names)
            if not names and self.controller_address:
                names = (await self.transport.post_json(self.controller_address + "/list_models", {})).get("models", [])
            return ModelList(data=[ModelCard(id=n, root=n) for n in names])

        @app.post("/generate")
        async def generate(request: GenerateRequest):
            text, reason, n_tok = "", None, 0
            try:
                async for chunk in self._relay(request):
                    if chunk.get("error_code", 0):
                        return JSONResponse(ErrorResponse(message=str(chunk.get("text")),
                                                          code=int(chunk["error_code"])).model_dump(), status_code=400)
                    text = chunk.get("text", text)
                    reason = chunk.get("finish_reason", reason)
                    n_tok = int(chunk.get("usage", {}).get("completion_tokens", n_tok))
            except RuntimeError as e:
                return JSONResponse(ErrorResponse(message=str(e), code=404).model_dump(), status_code=404)
            details = Details(finish_reason=reason or "length", generated_tokens=n_tok, seed=request.parameters.seed) \
                if request.parameters.details else None
            return GenerateResponse(generated_text=text, details=details)

        @app.post("/generate_stream")
        async def generate_stream(request: GenerateRequest):
            async def sse():
                sent, reason, n_tok = "", None, 0
                try:
                    async for chunk in self._relay(request):
                        if chunk.get("error_code", 0):
                            err = ErrorResponse(message=str(chunk.get("text")), code=int(chunk["error_code"]))
                            yield f"data: {err.model_dump_json()}\n\n"
                            return
                        text = chunk.get("text", sent)
                        reason = chunk.get("finish_reason", reason)
                        n_tok = int(chunk.get("usage", {}).get("completion_tokens", n_tok))
                        piece = text[len(sent):] if text.startswith(sent) else text
                        sent = text
                        if piece and reason is None:
                            yield f"data: {StreamResponse(token=Token(text=piece)).model_dump_json()}\n\n"
                        elif reason is not None:
                            last = StreamResponse(token=Token(text=piece), generated_text=sent,
                                                  details=Details(finish_reason=reason, generated_tokens=n_tok,
                                                                  seed=request.parameters.seed))
                            yield f"data: {last.model_dump_json()}\n\n"
                except RuntimeError as e:
                    yield f"data: {ErrorResponse(message=str(e), code=404).model_dump_json()}\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--controller-address", default=None)
    ap.add_argument("--worker-address", default=None)
    ap.add_argument("--model-names", default=None, help="comma separated")
    a = ap.parse_args(argv)
    import uvicorn
    tgi = TGIApp(a.controller_address, a.worker_address, a.model_names.split(",") if a.model_names else None)
    uvicorn.run(tgi.app, host=a.host, port=a.port, log_level="info")


if __name__ == "__main__":
    main()
