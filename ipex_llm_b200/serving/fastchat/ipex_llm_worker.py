"""``BigDLLLMWorker``: a model worker that speaks FastChat's controller / worker HTTP protocol.

Reference: python/llm/src/ipex_llm/serving/fastchat/ipex_llm_worker.py (``BigDLLLMWorker`` with
``generate_stream_gate`` / ``generate_gate``, heart-beats to the controller, ``/worker_generate_stream``,
``/worker_generate``, ``/worker_get_embeddings``, ``/worker_get_status``, ``/count_token``, ``/model_details``).  FastChat itself is not a
dependency: the endpoints and JSON payloads are implemented here on FastAPI, generation runs on this package's
``ModelWorker``, and registration with a controller is a plain HTTP POST when ``controller_addr`` is given.

    python -m ipex_llm_b200.serving.fastchat.ipex_llm_worker --model-path <dir> --low-bit sym_int4 --port 21002
"""
from __future__ import annotations

import argparse
import asyncio
import json
import threading
import time
import uuid
from typing import Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, StreamingResponse

from ..model_worker import ModelWorker, SamplingParams

HEART_BEAT_INTERVAL = 45


class BigDLLLMWorker:
    def __init__(self, controller_addr: Optional[str], worker_addr: str, worker_id: str, model_path: str,
                 model_names=None, limit_worker_concurrency: int = 8, low_bit: str = "sym_int4", device: str = "cuda",
                 no_register: bool = False, worker: Optional[ModelWorker] = None, speculative: bool = False,
                 load_low_bit_model: bool = False, stream_interval: int = 2, **kwargs):
        self.controller_addr, self.worker_addr, self.worker_id = controller_addr, worker_addr, worker_id
        self.model_names = model_names or [model_path.rstrip("/").split("/")[-1]]
        self.limit_worker_concurrency = limit_worker_concurrency
        self.stream_interval = stream_interval
        self.worker = worker or ModelWorker(model_path, low_bit, max_num_seqs=limit_worker_concurrency,
                                            device=None if device in ("cuda", "xpu") else device)
        self.tokenizer = self.worker.tokenizer
        self.context_len = getattr(self.worker.model.config, "max_position_embeddings", 2048)
        self.call_ct = 0
        self.in_flight = 0
        if controller_addr and not no_register:
            self.register_to_controller()
            threading.Thread(target=self._heart_beat_loop, daemon=True).start()

    # ---- controller protocol ---------------------------------------------------------------------------
    def _post(self, path, payload):
        import requests
        return requests.post(self.controller_addr + path, json=payload, timeout=5)

    def register_to_controller(self):
        self._post("/register_worker", {"worker_name": self.worker_addr, "check_heart_beat": True,
                                        "worker_status": self.get_status()})

    def _heart_beat_loop(self):
        while True:
            time.sleep(HEART_BEAT_INTERVAL)
            try:
                r = self._post("/receive_heart_beat", {"worker_name": self.worker_addr,
                                                       "queue_length": self.get_queue_length()})
                if not r.json().get("exist", True):
                    self.register_to_controller()
            except Exception:  # noqa: BLE001 - controller away: keep serving, try again later
                pass

    def get_queue_length(self):
        return self.in_flight + self.worker.waiting.qsize()

    def get_status(self):
        return {"model_names": self.model_names, "speed": 1, "queue_length": self.get_queue_length()}

    def count_token(self, params):
        return {"count": len(self.tokenizer(params["prompt"])["input_ids"]), "error_code": 0}

    def get_conv_template(self):
        return {"conv": {"name": "ipex-llm", "system_message": "", "roles": ["USER", "ASSISTANT"], "messages": [],
                         "sep": "\n", "stop_str": None}}

    # ---- generation --------------------------------------------------------------------------------------
    @staticmethod
    def _params(p) -> SamplingParams:
        t = float(p.get("temperature", 1.0))
        stop = p.get("stop") or []
        stop = [stop] if isinstance(stop, str) else list(stop)
        return SamplingParams(max_new_tokens=int(p.get("max_new_tokens", 256)), do_sample=t > 1e-5 and t != 1.0,
                              temperature=max(t, 1e-5), top_p=float(p.get("top_p", 1.0)),
                              top_k=max(int(p.get("top_k", -1)), 0),
                              repetition_penalty=float(p.get("repetition_penalty", 1.0)), stop=stop)

    async def generate_stream_gate(self, params):
        self.call_ct += 1
        self.in_flight += 1
        try:
            req = await self.worker.submit(params["prompt"], self._params(params))
            echo = params.get("echo", True)
            text = params["prompt"] if echo else ""
            n = 0
            while True:
                item = await asyncio.wait_for(req.out.get(), timeout=600)
                if isinstance(item, dict):
                    if "error" in item:
                        yield json.dumps({"text": item["error"], "error_code": 50001}).encode() + b"\0"
                        return
                    out = {"text": (params["prompt"] if echo else "") + item["generated_text"], "error_code": 0,
                           "usage": {"prompt_tokens": item["prompt_tokens"],
                                     "completion_tokens": item["generated_tokens"],
                                     "total_tokens": item["prompt_tokens"] + item["generated_tokens"]},
                           "finish_reason": item["finish_reason"]}
                    yield json.dumps(out).encode() + b"\0"
                    return
                text += item
                n += 1
                if n % self.stream_interval == 0:
                    yield json.dumps({"text": text, "error_code": 0, "finish_reason": None}).encode() + b"\0"
        finally:
            self.in_flight -= 1

    def get_embeddings(self, params):
        """FastChat's ``/worker_get_embeddings``: mean of the last hidden states over the real tokens of every input,
        L2-normalised; ``token_num`` counts the tokens that were embedded."""
        import torch
        texts = params["input"]
        texts = [texts] if isinstance(texts, str) else list(texts)
        tok, model = self.tokenizer, self.worker.model
        enc = tok(texts, return_tensors="pt", padding=True, truncation=True, max_length=self.context_len)
        dev = next(model.parameters()).device
        ids, mask = enc["input_ids"].to(dev), enc["attention_mask"].to(dev)
        with torch.no_grad():
            out = model(input_ids=ids, attention_mask=mask, output_hidden_states=True)
        h = out.hidden_states[-1].float()
        m = mask.unsqueeze(-1).float()
        emb = (h * m).sum(1) / m.sum(1).clamp_min(1.0)
        emb = torch.nn.functional.normalize(emb, p=2, dim=1)
        return {"embedding": emb.cpu().tolist(), "token_num": int(mask.sum())}

    async def generate_gate(self, params):
        last = None
        async for chunk in self.generate_stream_gate(params):
            last = chunk
        return json.loads(last[:-1].decode())


def create_app(w: BigDLLLMWorker) -> FastAPI:
    app = FastAPI()

    @app.post("/worker_generate_stream")
    async def api_generate_stream(request: Request):
        return StreamingResponse(w.generate_stream_gate(await request.json()))

    @app.post("/worker_generate")
    async def api_generate(request: Request):
        return JSONResponse(await w.generate_gate(await request.json()))

    @app.post("/worker_get_embeddings")
    async def api_get_embeddings(request: Request):
        return JSONResponse(w.get_embeddings(await request.json()))

    @app.post("/worker_get_status")
    async def api_get_status(request: Request):
        return w.get_status()

    @app.post("/count_token")
    async def api_count_token(request: Request):
        return w.count_token(await request.json())

    @app.post("/worker_get_conv_template")
    async def api_get_conv(request: Request):
        return w.get_conv_template()

    @app.post("/model_details")
    async def api_model_details(request: Request):
        return {"context_length": w.context_len}

    return app


def main(argv=None):
    import uvicorn
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="localhost")
    ap.add_argument("--port", type=int, default=21002)
    ap.add_argument("--worker-address", default="http://localhost:21002")
    ap.add_argument("--controller-address", default="http://localhost:21001")
    ap.add_argument("--model-path", required=True)
    ap.add_argument("--low-bit", default="sym_int4")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--model-names", type=lambda s: s.split(","))
    ap.add_argument("--limit-worker-concurrency", type=int, default=8)
    ap.add_argument("--no-register", action="store_true")
    a = ap.parse_args(argv)
    w = BigDLLLMWorker(a.controller_address, a.worker_address, str(uuid.uuid4())[:8], a.model_path, a.model_names,
                       a.limit_worker_concurrency, a.low_bit, a.device, a.no_register)
    uvicorn.run(create_app(w), host=a.host, port=a.port, log_level="info")


if __name__ == "__main__":
    main()
