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
from dataclasses import dataclass, field
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
        t0 = time.perf_counter()
        out = self.model.generate(ids, max_new_tokens=task.max_tokens, do_sample=False,
                                  eos_token_id=self.tokenizer.eos_token_id, pad_token_id=self.tokenizer.pad_token_id)
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
                if r.text:
                    r.emit(r.text)
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
