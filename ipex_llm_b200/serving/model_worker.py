"""``ModelWorker``: one model, one generation thread, dynamic batching of waiting requests.

Reference behaviour (python/llm/src/ipex_llm/serving/fastapi/model_worker.py:27-210): requests wait in an asyncio
queue; the worker takes one, runs ``model.generate`` in a thread with a ``TextIteratorStreamer`` and the HTTP layer
forwards the pieces.  Here the worker takes up to ``max_num_seqs`` compatible requests at once, left-pads them into
one batch and streams every sequence separately through ``BatchTextIteratorStreamer``; a request whose stop string
or EOS has been reached is closed immediately while the rest of its batch keeps going.
"""
from __future__ import annotations

import asyncio
import logging
import queue
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import List, Optional

import torch

logger = logging.getLogger("ipex_llm.serving")


@dataclass
class SamplingParams:
    max_new_tokens: int = 32
    do_sample: bool = False
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    repetition_penalty: float = 1.0
    stop: List[str] = field(default_factory=list)
    seed: Optional[int] = None

    def key(self):
        """Requests are batched together only when generate() would be configured identically."""
        return (self.do_sample, round(self.temperature, 4), round(self.top_p, 4), self.top_k,
                round(self.repetition_penalty, 4))


@dataclass
class ServingRequest:
    prompt: str
    params: SamplingParams
    request_id: str = field(default_factory=lambda: uuid.uuid4().hex)
    arrival: float = field(default_factory=time.perf_counter)
    loop: Optional[asyncio.AbstractEventLoop] = None
    out: Optional[asyncio.Queue] = None          # receives str pieces, then a final dict
    prompt_tokens: int = 0
    generated_tokens: int = 0
    text: str = ""
    finished: bool = False

    def emit(self, item):
        if self.loop is not None and self.out is not None:
            self.loop.call_soon_threadsafe(self.out.put_nowait, item)


class ModelWorker:
    def __init__(self, checkpoint: Optional[str] = None, low_bit: str = "sym_int4", model_type: str = "normal",
                 torch_dtype=torch.float16, model=None, tokenizer=None, max_num_seqs: int = 8, device=None):
        self.dtype = torch_dtype
        self.model_name = checkpoint or getattr(getattr(model, "config", None), "_name_or_path", "model")
        t0 = time.perf_counter()
        if model is None:
            model, tokenizer = self.load_model(checkpoint, low_bit, model_type, device)
        self.model, self.tokenizer = model, tokenizer
        if self.tokenizer.pad_token_id is None:
            self.tokenizer.pad_token = self.tokenizer.eos_token
        self.tokenizer.padding_side = "left"
        logger.info("Time to load weights: %.2fs", time.perf_counter() - t0)
        self.max_num_seqs = max_num_seqs
        self.waiting: "queue.Queue[ServingRequest]" = queue.Queue()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.stats = {"requests": 0, "batches": 0, "generated_tokens": 0, "first_token_s": [], "next_token_s": []}

    # ------------------------------------------------------------------------------------------------
    def load_model(self, model_path, low_bit="sym_int4", model_type="normal", device=None):
        from transformers import AutoTokenizer
        from ..transformers import AutoModel, AutoModelForCausalLM, AutoModelForSpeechSeq2Seq
        kw = dict(load_in_low_bit=low_bit, torch_dtype=self.dtype, optimize_model=True, trust_remote_code=True,
                  use_cache=True)
        if model_type == "audio":
            model = AutoModelForSpeechSeq2Seq.from_pretrained(model_path, **kw)
            try:
                from transformers import AutoProcessor
                self.processor = AutoProcessor.from_pretrained(model_path)
            except Exception:  # noqa: BLE001 - the feature extractor alone is enough
                from transformers import AutoFeatureExtractor
                self.processor = AutoFeatureExtractor.from_pretrained(model_path)
        else:
            try:
                model = AutoModelForCausalLM.from_pretrained(model_path, **kw)
            except Exception:  # noqa: BLE001 - checkpoints that only register with AutoModel (chatglm family)
                model = AutoModel.from_pretrained(model_path, **kw)
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        model = model.eval().to(device)
        tok = AutoTokenizer.from_pretrained(model_path, trust_remote_code=True, padding_side="left")
        return model, tok

    # ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def transcribe(self, samples, language: Optional[str] = None, max_new_tokens: int = 128) -> str:
        """Speech-to-text for one 16 kHz mono waveform (numpy float32) with a speech sequence-to-sequence model
        (reference model_worker.py:100-118)."""
        proc = getattr(self, "processor", None)
        fe = getattr(proc, "feature_extractor", proc)
        if fe is None:
            raise RuntimeError("transcribe needs a worker created with model_type='audio'")
        feats = fe(samples, sampling_rate=16000, return_tensors="pt").input_features
        dev = next(self.model.parameters()).device
        feats = feats.to(dev, self.dtype if dev.type == "cuda" else torch.float32)
        kw = {}
        if language and hasattr(proc, "get_decoder_prompt_ids"):
            try:
                kw["forced_decoder_ids"] = proc.get_decoder_prompt_ids(language=language, task="transcribe")
            except Exception:  # noqa: BLE001 - tokenizers without language tokens
                pass
        ids = self.model.generate(input_features=feats, max_new_tokens=max_new_tokens, do_sample=False, **kw)
        tok = getattr(proc, "tokenizer", None) or self.tokenizer
        return tok.batch_decode(ids, skip_special_tokens=True)[0].strip()

    # ------------------------------------------------------------------------------------------------
    def start(self):
        if self._thread is None or not self._thread.is_alive():
            self._stop.clear()
            self._thread = threading.Thread(target=self._serve_forever, name="ipex-llm-worker", daemon=True)
            self._thread.start()

    def shutdown(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    async def submit(self, prompt: str, params: SamplingParams) -> ServingRequest:
        req = ServingRequest(prompt=prompt, params=params, loop=asyncio.get_running_loop(), out=asyncio.Queue())
        self.waiting.put(req)
        self.start()
        return req

    def submit_blocking(self, prompt: str, params: SamplingParams) -> ServingRequest:
        """For callers without an event loop (tests, scripts): the finished request is returned."""
        req = ServingRequest(prompt=prompt, params=params)
        self._run_batch([req])
        return req

    # ------------------------------------------------------------------------------------------------
    def _next_batch(self) -> List[ServingRequest]:
        try:
            first = self.waiting.get(timeout=0.05)
        except queue.Empty:
            return []
        batch, rest = [first], []
        while len(batch) < self.max_num_seqs:
            try:
                r = self.waiting.get_nowait()
            except queue.Empty:
                break
            (batch if r.params.key() == first.params.key() else rest).append(r)
        for r in rest:
            self.waiting.put(r)
        return batch

    def _serve_forever(self):
        while not self._stop.is_set():
            batch = self._next_batch()
            if not batch:
                continue
            try:
                self._run_batch(batch)
            except Exception as e:  # noqa: BLE001 - a failed batch must not kill the server
                logger.exception("generation failed")
                for r in batch:
                    if not r.finished:
                        r.finished = True
                        r.emit({"error": str(e), "finish_reason": "error"})

    @torch.no_grad()
    def _run_batch(self, batch: List[ServingRequest]):
        from transformers import StoppingCriteria, StoppingCriteriaList
        from ..transformers.streamer import BatchTextIteratorStreamer
        tok, p = self.tokenizer, batch[0].params
        enc = tok([r.prompt for r in batch], return_tensors="pt", padding=True)
        dev = next(self.model.parameters()).device
        ids, mask = enc["input_ids"].to(dev), enc["attention_mask"].to(dev)
        for r, m in zip(batch, enc["attention_mask"]):
            r.prompt_tokens = int(m.sum())
        max_new = max(r.params.max_new_tokens for r in batch)
        streamer = BatchTextIteratorStreamer(len(batch), tok, skip_prompt=True, skip_special_tokens=True)
        done = [False] * len(batch)
        eos = tok.eos_token_id

        class _AllDone(StoppingCriteria):
            def __call__(self, input_ids, scores, **kw):
                return torch.full((input_ids.shape[0],), all(done), dtype=torch.bool, device=input_ids.device)

        kw = dict(max_new_tokens=max_new, do_sample=p.do_sample, streamer=streamer, attention_mask=mask,
                  pad_token_id=tok.pad_token_id, stopping_criteria=StoppingCriteriaList([_AllDone()]))
        if p.do_sample:
            kw.update(temperature=p.temperature, top_p=p.top_p)
            if p.top_k and p.top_k > 0:
                kw["top_k"] = p.top_k
            if p.seed is not None:
                torch.manual_seed(p.seed)
        if p.repetition_penalty and p.repetition_penalty != 1.0:
            kw["repetition_penalty"] = p.repetition_penalty
        result = {}

        def _gen():
            try:
                result["ids"] = self.model.generate(ids, **kw)
            except Exception as e:  # noqa: BLE001
                result["error"] = e
                streamer.end()

        th = threading.Thread(target=_gen, daemon=True)
        t0 = time.perf_counter()
        th.start()
        first_seen = False
        t_prev = t0
        for pieces in streamer:
            now = time.perf_counter()
            if not first_seen:
                self.stats["first_token_s"].append(now - t0)
                first_seen = True
            else:
                self.stats["next_token_s"].append(now - t_prev)
            t_prev = now
            for i, (r, piece) in enumerate(zip(batch, pieces)):
                if done[i]:
                    continue
                r.generated_tokens = streamer.generated_tokens[i]
                if piece:
                    r.text += piece
                    cut = _first_stop(r.text, r.params.stop)
                    if cut >= 0:
                        emit = piece[: max(0, len(piece) - (len(r.text) - cut))]
                        r.text = r.text[:cut]
                        if emit:
                            r.emit(emit)
                        self._finish(r, "stop")
                        done[i] = True
                        continue
                    r.emit(piece)
                if r.generated_tokens >= r.params.max_new_tokens:
                    self._finish(r, "length")
                    done[i] = True
        th.join()
        if "error" in result:
            raise result["error"]
        out = result["ids"]
        for i, r in enumerate(batch):
            if not done[i]:
                new = out[i, ids.shape[1]:]
                hit_eos = eos is not None and bool((new == eos).any())
                self._finish(r, "stop" if hit_eos else "length")
        self.stats["requests"] += len(batch)
        self.stats["batches"] += 1

    def _finish(self, r: ServingRequest, reason: str):
        r.finished = True
        self.stats["generated_tokens"] += r.generated_tokens
        r.emit({"finish_reason": reason, "prompt_tokens": r.prompt_tokens, "generated_tokens": r.generated_tokens,
                "generated_text": r.text})
        r.finish_reason = reason


def _first_stop(text: str, stops: List[str]) -> int:
    best = -1
    for s in stops or []:
        if not s:
            continue
        i = text.find(s)
        if i >= 0 and (best < 0 or i < best):
            best = i
    return best
