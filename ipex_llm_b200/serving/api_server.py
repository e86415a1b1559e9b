"""``FastApp``: the HTTP front of a ``ModelWorker`` (or ``PPModelWorker``).

Endpoints (same set as python/llm/src/ipex_llm/serving/fastapi/api_server.py:103-437):
  POST /generate, /generate_stream      TGI-style
  POST /v1/chat/completions, /v1/completions   OpenAI-compatible (streaming with server-sent events)
  POST /v1/audio/transcriptions                OpenAI-compatible speech-to-text (workers started with model_type "audio")
  GET  /v1/models, /health, /metrics
``IPEX_LLM_FASTAPI_TIMEOUT`` bounds the time a request may wait for its next piece.
"""
from __future__ import annotations

import asyncio
import json
import os
import time
from typing import AsyncIterator, List, Optional

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from .model_worker import ModelWorker, SamplingParams
from .protocol import (ChatCompletionRequest, ChatCompletionResponse, ChatCompletionResponseChoice,
                       ChatCompletionResponseStreamChoice, ChatCompletionStreamResponse, ChatMessage,
                       CompletionRequest, CompletionResponse, CompletionResponseChoice, CompletionStreamResponse,
                       DeltaMessage, GenerateRequest, GenerateResponse, ModelCard, ModelList, StreamResponse,
                       StreamToken, UsageInfo)


def _timeout() -> float:
    return float(os.environ.get("IPEX_LLM_FASTAPI_TIMEOUT", "600"))


def _params_from_openai(req) -> SamplingParams:
    stop = [req.stop] if isinstance(req.stop, str) else list(req.stop or [])
    t = 1.0 if req.temperature is None else req.temperature
    return SamplingParams(max_new_tokens=req.max_tokens or 256, do_sample=t > 1e-5 and t != 1.0 or
                          (req.top_p or 1.0) < 1.0 or (req.top_k or -1) > 0, temperature=max(t, 1e-5),
                          top_p=req.top_p or 1.0, top_k=max(req.top_k or 0, 0),
                          repetition_penalty=req.repetition_penalty or 1.0, stop=stop, seed=req.seed)


def _params_from_tgi(p) -> SamplingParams:
    return SamplingParams(max_new_tokens=p.max_new_tokens, do_sample=p.do_sample, temperature=p.temperature or 1.0,
                          top_p=p.top_p or 1.0, top_k=p.top_k or 0, repetition_penalty=p.repetition_penalty or 1.0,
                          stop=list(p.stop or []), seed=p.seed)


def chat_prompt(tokenizer, messages: List[ChatMessage]) -> str:
    """The tokenizer's chat template when it has one, a plain role-tagged transcript otherwise."""
    msgs = [{"role": m.role, "content": m.content if isinstance(m.content, str) else
             " ".join(part.get("text", "") for part in (m.content or []) if isinstance(part, dict))} for m in messages]
    if getattr(tokenizer, "chat_template", None):
        try:
            return tokenizer.apply_chat_template(msgs, tokenize=False, add_generation_prompt=True)
        except Exception:  # noqa: BLE001 - malformed template: fall through to the generic form
            pass
    return "".join(f"{m['role']}: {m['content']}\n" for m in msgs) + "assistant:"


class FastApp:
    def __init__(self, local_model: ModelWorker, served_model_name: Optional[str] = None):
        self.worker = local_model
        self.name = served_model_name or os.path.basename(str(local_model.model_name).rstrip("/")) or "model"
        self.app = FastAPI(title="ipex-llm serving")
        self._routes()

    # ------------------------------------------------------------------------------------------------
    async def _pieces(self, req) -> AsyncIterator:
        """Yields str pieces, then the final summary dict."""
        while True:
            try:
                item = await asyncio.wait_for(req.out.get(), timeout=_timeout())
            except asyncio.TimeoutError:
                raise HTTPException(status_code=504, detail="generation timed out")
            yield item
            if isinstance(item, dict):
                return

    async def _collect(self, req):
        final = None
        async for item in self._pieces(req):
            if isinstance(item, dict):
                final = item
        if final is None or "error" in final:
            raise HTTPException(status_code=500, detail=(final or {}).get("error", "generation failed"))
        return final

    def _routes(self):
        app, w = self.app, self.worker

        @app.get("/health")
        async def health():
            return PlainTextResponse("OK")

        @app.get("/v1/models")
        async def models():
            return ModelList(data=[ModelCard(id=self.name)])

        @app.get("/metrics")
        async def metrics():
            s = w.stats
            ft, nt = s["first_token_s"], s["next_token_s"]
            lines = [f"ipex_llm_requests_total {s['requests']}", f"ipex_llm_batches_total {s['batches']}",
                     f"ipex_llm_generated_tokens_total {s['generated_tokens']}",
                     f"ipex_llm_first_token_seconds_avg {sum(ft) / len(ft) if ft else 0.0}",
                     f"ipex_llm_next_token_seconds_avg {sum(nt) / len(nt) if nt else 0.0}",
                     f"ipex_llm_waiting_requests {w.waiting.qsize()}"]
            return PlainTextResponse("\n".join(lines) + "\n")

        @app.post("/generate")
        async def generate(request: GenerateRequest):
            req = await w.submit(request.inputs, _params_from_tgi(request.parameters))
            fin = await self._collect(req)
            text = (request.inputs if request.parameters.return_full_text else "") + fin["generated_text"]
            return GenerateResponse(generated_text=text, generate_text=text, prompt_tokens=fin["prompt_tokens"],
                                    generated_tokens=fin["generated_tokens"], finish_reason=fin["finish_reason"])

        @app.post("/generate_stream")
        async def generate_stream(request: GenerateRequest):
            req = await w.submit(request.inputs, _params_from_tgi(request.parameters))

            async def sse():
                async for item in self._pieces(req):
                    if isinstance(item, dict):
                        out = StreamResponse(token=StreamToken(text=""), generated_text=item.get("generated_text"),
                                             finish_reason=item.get("finish_reason"))
                    else:
                        out = StreamResponse(token=StreamToken(text=item))
                    yield f"data: {out.model_dump_json()}\n\n"
            return StreamingResponse(sse(), media_type="text/event-stream")

        @app.post("/v1/chat/completions")
        async def chat(request: ChatCompletionRequest):
            prompt = chat_prompt(w.tokenizer, request.messages)
            req = await w.submit(prompt, _params_from_openai(request))
            if request.stream:
                async def sse():
                    first = ChatCompletionStreamResponse(model=self.name, choices=[
                        ChatCompletionResponseStreamChoice(index=0, delta=DeltaMessage(role="assistant"))])
                    rid = first.id
                    yield f"data: {first.model_dump_json(exclude_unset=False)}\n\n"
                    async for item in self._pieces(req):
                        if isinstance(item, dict):
                            ch = ChatCompletionResponseStreamChoice(index=0, delta=DeltaMessage(),
                                                                    finish_reason=_reason(item))
                        else:
                            ch = ChatCompletionResponseStreamChoice(index=0, delta=DeltaMessage(content=item))
                        yield f"data: {ChatCompletionStreamResponse(id=rid, model=self.name, choices=[ch]).model_dump_json()}\n\n"
                    yield "data: [DONE]\n\n"
                return StreamingResponse(sse(), media_type="text/event-stream")
            fin = await self._collect(req)
            usage = UsageInfo(prompt_tokens=fin["prompt_tokens"], completion_tokens=fin["generated_tokens"],
                              total_tokens=fin["prompt_tokens"] + fin["generated_tokens"])
            return ChatCompletionResponse(model=self.name, usage=usage, choices=[ChatCompletionResponseChoice(
                index=0, message=ChatMessage(role="assistant", content=fin["generated_text"]),
                finish_reason=_reason(fin))])

        @app.post("/v1/completions")
        async def completions(request: CompletionRequest):
            prompts = [request.prompt] if isinstance(request.prompt, str) else list(request.prompt)
            params = _params_from_openai(request)
            reqs = [await w.submit(p, params) for p in prompts]
            if request.stream:
                if len(reqs) != 1:
                    raise HTTPException(status_code=400, detail="streaming supports one prompt per request")

                async def sse():
                    rid = None
                    async for item in self._pieces(reqs[0]):
                        if isinstance(item, dict):
                            ch = CompletionResponseChoice(index=0, text="", finish_reason=_reason(item))
                        else:
                            ch = CompletionResponseChoice(index=0, text=item)
                        resp = CompletionStreamResponse(model=self.name, choices=[ch])
                        rid = rid or resp.id
                        resp.id = rid
                        yield f"data: {resp.model_dump_json()}\n\n"
                    yield "data: [DONE]\n\n"
                return StreamingResponse(sse(), media_type="text/event-stream")
            fins = [await self._collect(r) for r in reqs]
            choices = [CompletionResponseChoice(index=i, text=(prompts[i] if request.echo else "") +
                                                f["generated_text"], finish_reason=_reason(f))
                       for i, f in enumerate(fins)]
            pt, ct = sum(f["prompt_tokens"] for f in fins), sum(f["generated_tokens"] for f in fins)
            return CompletionResponse(model=self.name, choices=choices,
                                      usage=UsageInfo(prompt_tokens=pt, completion_tokens=ct, total_tokens=pt + ct))

        @app.post("/v1/audio/transcriptions")
        async def transcriptions(request: Request):
            """multipart/form-data with ``file`` (PCM WAV) and optional ``model``, ``language``, ``prompt``,
            ``response_format`` (json | text), as the reference's endpoint (api_server.py:403-425)."""
            from .audio import decode_wav, parse_multipart, resample
            form = parse_multipart(await request.body(), request.headers.get("content-type", ""))
            if not isinstance(form.get("file"), tuple):
                raise HTTPException(status_code=400, detail="multipart field 'file' with a WAV file is required")
            if not hasattr(w, "transcribe"):
                raise HTTPException(status_code=400, detail="this worker serves no speech model")
            try:
                samples, rate = decode_wav(form["file"][1])
            except Exception as e:  # noqa: BLE001
                raise HTTPException(status_code=400, detail=f"cannot decode the audio file: {e}")
            loop = asyncio.get_running_loop()
            try:
                text = await asyncio.wait_for(
                    loop.run_in_executor(None, w.transcribe, resample(samples, rate), form.get("language") or None),
                    timeout=_timeout())
            except asyncio.TimeoutError:
                raise HTTPException(status_code=504, detail="transcription timed out")
            if (form.get("response_format") or "json") == "text":
                return PlainTextResponse(text)
            return JSONResponse({"text": text})

def _reason(item) -> Optional[str]:
    r = item.get("finish_reason")
    return r if r in ("stop", "length") else "stop"


def main(argv=None):
    """``python -m ipex_llm_b200.serving.api_server --repo-id-or-model-path <dir> --low-bit sym_int4 --port 8000``
    (the flags of the reference's Lightweight-Serving example)."""
    import argparse

    import uvicorn
    ap = argparse.ArgumentParser()
    ap.add_argument("--repo-id-or-model-path", type=str, required=True)
    ap.add_argument("--low-bit", type=str, default="sym_int4")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--host", type=str, default="0.0.0.0")
    ap.add_argument("--max-num-seqs", type=int, default=8)
    ap.add_argument("--model-type", type=str, default="normal")
    ap.add_argument("--pipeline-parallel-stages", type=int, default=int(os.environ.get("WORLD_SIZE", "1")),
                    help="under torchrun: one stage per rank; rank 0 serves HTTP, the others follow its batches "
                         "(the reference's Pipeline-Parallel-Serving/pipeline_serving.py)")
    a = ap.parse_args(argv)
    if a.pipeline_parallel_stages > 1:
        from .pp_worker import PPModelWorker
        worker = PPModelWorker(a.repo_id_or_model_path, low_bit=a.low_bit, max_num_seqs=a.max_num_seqs)
        if worker.rank != 0:
            worker._serve_forever()                 # stages without the HTTP side follow rank 0 until it stops
            return
    else:
        worker = ModelWorker(a.repo_id_or_model_path, a.low_bit, a.model_type, max_num_seqs=a.max_num_seqs)
    uvicorn.run(FastApp(worker).app, host=a.host, port=a.port)


if __name__ == "__main__":
    main()
