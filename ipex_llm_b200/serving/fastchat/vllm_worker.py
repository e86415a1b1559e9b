"""``VLLMWorker``: FastChat's worker protocol in front of the vLLM adapter (reference:
python/llm/src/ipex_llm/serving/fastchat/vllm_worker.py).

Same HTTP surface as ``BigDLLLMWorker`` (``/worker_generate_stream``, ``/worker_generate``, ``/worker_get_status``,
``/count_token``, ``/model_details``), but generation goes through ``IPEXLLMAsyncLLMEngine`` - vLLM's async engine whose
workers convert the loaded model to ``load_in_low_bit`` - so continuous batching and paged KV come from vLLM.  vLLM
is imported only when a worker is built without an injected engine.

    python -m ipex_llm_b200.serving.fastchat.vllm_worker --model-path <dir> --load-in-low-bit sym_int4 --port 21002
"""
from __future__ import annotations

import argparse
import json
import uuid
from typing import Optional

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, StreamingResponse

_SAMPLING_KEYS = ("n", "best_of", "presence_penalty", "frequency_penalty", "temperature", "top_p", "top_k", "stop",
                  "stop_token_ids", "max_tokens", "use_beam_search")


class VLLMWorker:
    def __init__(self, controller_addr: Optional[str], worker_addr: str, worker_id: str, model_path: str,
                 model_names=None, limit_worker_concurrency: int = 64, no_register: bool = True, engine=None,
                 tokenizer=None, context_len: int = 2048, load_in_low_bit: str = "sym_int4", **engine_kwargs):
        self.controller_addr, self.worker_addr, self.worker_id = controller_addr, worker_addr, worker_id
        self.model_names = model_names or [model_path.rstrip("/").split("/")[-1]]
        self.limit_worker_concurrency = limit_worker_concurrency
        if engine is None:
            from vllm.engine.arg_utils import AsyncEngineArgs
            from ...vllm.engine import IPEXLLMAsyncLLMEngine
            args = AsyncEngineArgs(model=model_path, **engine_kwargs)
            engine = IPEXLLMAsyncLLMEngine.from_engine_args(args, load_in_low_bit=load_in_low_bit)
        self.engine = engine
        self.tokenizer = tokenizer
        self.context_len = context_len
        self.call_ct = 0
        self.in_flight = 0
        if controller_addr and not no_register:
            self.register_to_controller()

    def register_to_controller(self):
        import requests
        requests.post(self.controller_addr + "/register_worker",
                      json={"worker_name": self.worker_addr, "check_heart_beat": True,
                            "worker_status": self.get_status()}, timeout=5)

    def get_status(self):
        return {"model_names": self.model_names, "speed": 1, "queue_length": self.in_flight}

    def count_token(self, params):
        if self.tokenizer is None:
            return {"count": len(params["prompt"].split()), "error_code": 0}
        return {"count": len(self.tokenizer(params["prompt"])["input_ids"]), "error_code": 0}

    @staticmethod
    def sampling_kwargs(params: dict) -> dict:
        """FastChat request parameters -> keyword arguments of vLLM's ``SamplingParams``."""
        t = float(params.get("temperature", 1.0))
        top_p = float(params.get("top_p", 1.0))
        stop = params.get("stop") or []
        stop = [stop] if isinstance(stop, str) else list(stop)
        kw = {"n": 1, "temperature": max(t, 0.0), "top_p": top_p if t > 1e-5 else 1.0,
              "top_k": int(params.get("top_k", -1)), "presence_penalty": float(params.get("presence_penalty", 0.0)),
              "frequency_penalty": float(params.get("frequency_penalty", 0.0)),
              "max_tokens": int(params.get("max_new_tokens", 256)), "stop": stop,
              "stop_token_ids": list(params.get("stop_token_ids") or [])}
        if params.get("best_of") is not None:
            kw["best_of"] = int(params["best_of"])
        return kw

    def _sampling_params(self, params: dict):
        kw = self.sampling_kwargs(params)
        try:
            import inspect

            from vllm import SamplingParams
            accepted = set(inspect.signature(SamplingParams).parameters)
            return SamplingParams(**{k: v for k, v in kw.items() if k in accepted})
        except Exception:  # noqa: BLE001 (an injected engine double takes the plain dictionary)
            return kw

    async def generate_stream(self, params):
        self.call_ct += 1
        self.in_flight += 1
        try:
            prompt = params["prompt"]
            echo = params.get("echo", True)
            request_id = params.get("request_id") or uuid.uuid4().hex
            async for out in self.engine.generate(prompt, self._sampling_params(params), request_id):
                texts = [(prompt if echo else "") + o.text for o in out.outputs]
                n_prompt = len(getattr(out, "prompt_token_ids", None) or [])
                n_gen = sum(len(getattr(o, "token_ids", None) or []) for o in out.outputs)
                finished = bool(getattr(out, "finished", False))
                ret = {"text": " ".join(texts), "error_code": 0,
                       "usage": {"prompt_tokens": n_prompt, "completion_tokens": n_gen,
                                 "total_tokens": n_prompt + n_gen},
                       "cumulative_logprob": [getattr(o, "cumulative_logprob", None) for o in out.outputs],
                       "finish_reason": (getattr(out.outputs[0], "finish_reason", None) if finished else None)}
                yield json.dumps(ret).encode() + b"\0"
        finally:
            self.in_flight -= 1

    async def generate(self, params):
        last = None
        async for chunk in self.generate_stream(params):
            last = chunk
        return json.loads(last[:-1].decode())


def create_app(w: VLLMWorker) -> FastAPI:
    app = FastAPI()

    @app.post("/worker_generate_stream")
    async def api_generate_stream(request: Request):
        return StreamingResponse(w.generate_stream(await request.json()))

    @app.post("/worker_generate")
    async def api_generate(request: Request):
        return JSONResponse(await w.generate(await request.json()))

    @app.post("/worker_get_status")
    async def api_get_status(request: Request):
        return w.get_status()

    @app.post("/count_token")
    async def api_count_token(request: Request):
        return w.count_token(await request.json())

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
    ap.add_argument("--model-names", type=lambda s: s.split(","))
    ap.add_argument("--load-in-low-bit", default="sym_int4")
    ap.add_argument("--limit-worker-concurrency", type=int, default=64)
    ap.add_argument("--no-register", action="store_true")
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    a = ap.parse_args(argv)
    w = VLLMWorker(a.controller_address, a.worker_address, str(uuid.uuid4())[:8], a.model_path, a.model_names,
                   a.limit_worker_concurrency, a.no_register, load_in_low_bit=a.load_in_low_bit,
                   tensor_parallel_size=a.tensor_parallel_size)
    uvicorn.run(create_app(w), host=a.host, port=a.port, log_level="info")


if __name__ == "__main__":
    main()
