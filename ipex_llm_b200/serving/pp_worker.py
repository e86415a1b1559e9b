"""``PPModelWorker``: pipeline-parallel serving.  Every rank runs one worker; rank 0 owns the request queue and the
HTTP layer, the other ranks follow the batches it announces.

Reference: python/llm/src/ipex_llm/transformers/pipeline_parallel.py:482-927 (``PPModelWorker`` with a ring of
in-flight ``BatchTask``s, ``max_num_seqs``, ``max_prefilled_seqs``, ``dist.broadcast_object_list`` for the schedule
and ``isend`` hand-offs).  Here the schedule message is a small ``BatchTask`` broadcast per batch, and the
token loop is ``pipeline_parallel_generate`` (micro-batches keep every stage busy inside one batch), with a
per-step callback on rank 0 that feeds the streams.
"""
from __future__ import annotations

import queue
import time
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from .model_worker import ModelWorker, SamplingParams, ServingRequest, _first_stop


@dataclass
class BatchTask:
    batch_id: str
    request_ids: List[str]
    max_tokens: int
    batch_size: int
    input_len: int
    prompt_lengths: List[int]
    stopped: bool = False
    input_ids: Optional[List[List[int]]] = None


class _TokenEmitter:
    """Streamer of the pipeline loop on the first stage: one ``put`` per decoding step with every sequence's
    token; each request gets the text its tokens add, as they arrive (the reference streams per token through
    its ring as well, pipeline_parallel.py:837-927).  Text that may still change is held back: an incomplete
    UTF-8 sequence, and a tail that is the beginning of one of the request's stop strings."""

    def __init__(self, tokenizer, requests):
        self.tok = tokenizer
        self.reqs = list(requests)
        n = len(self.reqs)
        self.tokens = [[] for _ in range(n)]
        self.done = [False] * n
        self.sent = [0] * n          # characters already emitted per request
        self.prefix = [""] * n       # the emitted text itself (to check it is a prefix of the final text)
        self._first = True

    def put(self, value):
        if self._first and value.dim() == 2:
            self._first = False      # the prompt
            return
        self._first = False
        ids = value.reshape(-1).tolist()
        eos = self.tok.eos_token_id
        for i, r in enumerate(self.reqs):
            if self.done[i] or i >= len(ids):
                continue
            t = ids[i]
            if (eos is not None and t == eos) or len(self.tokens[i]) >= r.params.max_new_tokens:
                self.done[i] = True
                continue
            self.tokens[i].append(t)
            text = self.tok.decode(self.tokens[i], skip_special_tokens=True)
            cut = _first_stop(text, r.params.stop)
            if cut >= 0:
                text, self.done[i] = text[:cut], True
            else:
                if text.endswith("�"):
                    continue
                hold = 0
                for s in r.params.stop or []:
                    for k in range(min(len(s) - 1, len(text)), 0, -1):
                        if text.endswith(s[:k]):
                            hold = max(hold, k)
                            break
                text = text[: len(text) - hold] if hold else text
            if len(text) > self.sent[i]:
                r.emit(text[self.sent[i]:])
                self.prefix[i] = text
                self.sent[i] = len(text)

    def end(self):
        pass


class PPModelWorker(ModelWorker):
    def __init__(self, checkpoint=None, rank=None, world_size=None, low_bit="sym_int4", max_num_seqs=4,
                 max_prefilled_seqs=0, torch_dtype=torch.float16, model=None, tokenizer=None):
        from ..parallel.pp import init_pipeline_parallel
        init_pipeline_parallel()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world_size is None else world_size
        self.max_prefilled_seqs = max_prefilled_seqs
        self._low_bit = low_bit
        super().__init__(checkpoint, low_bit, torch_dtype=torch_dtype, model=model, tokenizer=tokenizer,
                         max_num_seqs=max_num_seqs)

    def load_model(self, model_path, low_bit="sym_int4", model_type="normal", device=None):
        from transformers import AutoTokenizer
        from ..transformers import AutoModel, AutoModelForCausalLM
        kw = dict(load_in_low_bit=low_bit, torch_dtype=self.dtype, optimize_model=True, trust_remote_code=True,
                  use_cache=True, pipeline_parallel_stages=self.world)
        try:
            model = AutoModelForCausalLM.from_pretrained(model_path, **kw)
        except Exception:  # noqa: BLE001
            model = AutoModel.from_pretrained(model_path, **kw)
        tok = AutoTokenizer.from_pretrained(model_path, trust_remote_code=True, padding_side="left")
        return model.eval(), tok

    # ------------------------------------------------------------------------------------------------
    def _announce(self, task: Optional[BatchTask]) -> Optional[BatchTask]:
        box = [task]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    def serve_step(self) -> bool:
        """One scheduling round on every rank.  Returns False when rank 0 announced shutdown."""
        batch: List[ServingRequest] = []
        task = None
        if self.rank == 0:
            batch = self._next_batch()
            if self._stop.is_set():
                task = BatchTask("stop", [], 0, 0, 0, [], stopped=True)
            elif batch:
                enc = self.tokenizer([r.prompt for r in batch], return_tensors="pt", padding=True)
                for r, m in zip(batch, enc["attention_mask"]):
                    r.prompt_tokens = int(m.sum())
                task = BatchTask(batch[0].request_id, [r.request_id for r in batch],
                                 max(r.params.max_new_tokens for r in batch), len(batch), enc["input_ids"].shape[1],
                                 [r.prompt_tokens for r in batch], input_ids=enc["input_ids"].tolist())
        task = self._announce(task)
        if task is None:
            return True
        if task.stopped:
            return False
        ids = torch.tensor(task.input_ids, dtype=torch.long)
        # prompts are left-padded to the longest of the batch: the mask follows from the announced lengths
        cols = torch.arange(ids.shape[1]).unsqueeze(0)
        attn = (cols >= ids.shape[1] - torch.tensor(task.prompt_lengths).unsqueeze(1)).long()
        t0 = time.perf_counter()
        emitter = _TokenEmitter(self.tokenizer, batch) if self.rank == 0 else None
        out = self.model.generate(ids, max_new_tokens=task.max_tokens, do_sample=False, streamer=emitter,
                                  attention_mask=attn, eos_token_id=self.tokenizer.eos_token_id, pad_token_id=self.tokenizer.pad_token_id)
        if self.rank == 0:
            self.stats["first_token_s"].append(getattr(self.model, "first_token_time", 0.0))
            self.stats["next_token_s"].extend(getattr(self.model, "next_token_time", []))
            new = out[:, task.input_len:].cpu()
            eos = self.tokenizer.eos_token_id
            for i, r in enumerate(batch):
                toks = new[i, : r.params.max_new_tokens].tolist()
                reason = "length"
                if eos is not None and eos in toks:
                    toks = toks[: toks.index(eos)]
                    reason = "stop"
                r.generated_tokens = len(toks)
                r.text = self.tokenizer.decode(toks, skip_special_tokens=True)
                cut = _first_stop(r.text, r.params.stop)
                if cut >= 0:
                    r.text, reason = r.text[:cut], "stop"
                # whatever the per-token stream has not delivered yet (held-back partial characters, or everything
                # when the model's generate did not stream)
                rest = r.text[emitter.sent[i]:] if r.text.startswith(emitter.prefix[i]) else ""
                if rest:
                    r.emit(rest)
                self._finish(r, reason)
            self.stats["requests"] += len(batch)
            self.stats["batches"] += 1
            self.stats["batch_seconds"] = self.stats.get("batch_seconds", 0.0) + time.perf_counter() - t0
        return True

    def _serve_forever(self):
        while self.serve_step():
            pass

    def submit_blocking(self, prompt: str, params: SamplingParams) -> ServingRequest:
        req = ServingRequest(prompt=prompt, params=params)
        self.waiting.put(req)
        return req
