"""Pipeline-parallel inference: contiguous layer slices over the ranks, NCCL (or gloo) p2p between stages.

Counterpart of python/llm/src/ipex_llm/transformers/pipeline_parallel.py of the reference
(``init_pipeline_parallel`` :108-112, ``pipeline_parallel`` :166-234, ``pipeline_parallel_generate`` :300-445).
Same partitioning rule (``ceil(L / stages)`` layers per rank, other layers replaced by pass-through dummies,
embedding only on the first rank, final norm + lm_head only on the last) and the same greedy-only contract.

What differs: the reference runs strictly serially — one stage busy at a time, blocking send/recv per token,
``next_ids`` broadcast to every rank.  Here the batch is split into micro-batches (one per stage when the batch
allows) that travel through the stages back to back, stage hand-offs are ``isend``/``irecv`` so a stage starts
its next micro-batch while the previous activation is still in flight, and sampled ids go only from the last
stage to the first (a ring), the full output being gathered once at the end.
"""
from __future__ import annotations

import math
import os
import time
from typing import List, Optional

import torch
import torch.distributed as dist
from torch import nn

from ..ops.kv_cache import DynamicFp8Cache, DynamicNormalCache
from ..utils.common import invalidInputError


def init_pipeline_parallel():
    """Create the default process group from the launcher's environment (torchrun or mpirun)."""
    if dist.is_initialized():
        return
    if "RANK" not in os.environ and "PMI_RANK" in os.environ:
        os.environ["RANK"] = os.environ["PMI_RANK"]
        os.environ["WORLD_SIZE"] = os.environ.get("PMI_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if torch.cuda.is_available():
        local = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
        torch.cuda.set_device(local % torch.cuda.device_count())
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    else:
        dist.init_process_group("gloo")


class Dummy_DecoderLayer(nn.Module):
    """Stands in for a decoder layer owned by another stage: returns its input."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        self.input_layernorm = nn.Identity()

    def forward(self, hidden_states, *args, **kwargs):
        return hidden_states


class Dummy_Embedding(nn.Module):
    def forward(self, input_ids):  # pragma: no cover - stages > 0 always receive inputs_embeds
        raise RuntimeError("this pipeline stage has no embedding table; it receives hidden states")


class Dummy_Norm(nn.Module):
    def forward(self, hidden_states):
        return hidden_states


class Dummy_Head(nn.Module):
    """Replaces lm_head on stages that are not last: the "logits" are the hidden states to hand on."""

    def forward(self, hidden_states):
        return hidden_states


def stage_layer_range(num_layers: int, stages: int, rank: int):
    per = math.ceil(num_layers / stages)
    return per * rank, min(per * (rank + 1), num_layers)


def pipeline_parallel(model, pipeline_parallel_stages: int, torch_dtype=torch.float16, device=None):
    """Keep only this rank's slice of ``model`` (in place) and move it to the rank's device."""
    invalidInputError(dist.is_initialized(), "call init_pipeline_parallel() first")
    world, rank = dist.get_world_size(), dist.get_rank()
    invalidInputError(world == pipeline_parallel_stages,
                      "Please make sure world size is same as `pipeline_parallel_stages`")
    base = model.model
    n_layers = model.config.num_hidden_layers
    start, end = stage_layer_range(n_layers, pipeline_parallel_stages, rank)
    for i in range(n_layers):
        if i < start or i >= end:
            base.layers[i] = Dummy_DecoderLayer()
        else:
            # the stage's own cache starts at index 0, so its length / mask bookkeeping sees a real layer first
            attn = getattr(base.layers[i], "self_attn", None)
            if attn is not None and hasattr(attn, "layer_idx"):
                attn.layer_idx = i - start
    if rank != 0:
        base.embed_tokens = Dummy_Embedding()
    if rank != world - 1:
        base.norm = Dummy_Norm()
        model.lm_head = Dummy_Head()
    model.pipeline_parallel_stages = pipeline_parallel_stages
    model.layer_start, model.layer_end = start, end
    model.num_layers = n_layers
    model.pp_rank, model.pp_world = rank, world
    if device is None and torch.cuda.is_available():
        device = torch.device("cuda", torch.cuda.current_device())
    if device is not None:
        model = model.to(device)
    import gc
    gc.collect()
    return model


def _new_cache(model, batch_rows: int, device):
    from ..models.utils import use_quantize_kv_cache
    probe = torch.empty(batch_rows, 1, device=device)
    cfg = model.config
    flag = getattr(model, "_pp_kv_fp8", None)
    if flag is None:
        # every stage must take the same decision (reference pipeline_parallel.py:143-163): decide on rank 0
        # and broadcast it
        local = use_quantize_kv_cache(None, probe, cfg.num_attention_heads,
                                      getattr(cfg, "num_key_value_heads", 1) or 1)
        t = torch.tensor([int(local)], device=device)
        dist.broadcast(t, src=0)
        flag = bool(int(t.item()))
        model._pp_kv_fp8 = flag
    return DynamicFp8Cache(cfg) if flag else DynamicNormalCache(cfg)


@torch.no_grad()
def pipeline_parallel_generate(self, inputs: Optional[torch.Tensor] = None, max_new_tokens: int = 32,
                               generation_config=None, streamer=None, attention_mask=None, **kwargs):
    """Greedy generation over the pipeline.  Every rank calls it with the same ``inputs``; every rank returns the
    same ``[B, S + max_new_tokens]`` tensor."""
    invalidInputError(inputs is not None and inputs.dim() == 2, "inputs must be [batch, seq] token ids")
    gc = generation_config or getattr(self, "generation_config", None)
    if kwargs.get("do_sample", False):
        invalidInputError(False, "pipeline-parallel generation supports greedy search only")
    max_new_tokens = kwargs.get("max_new_tokens", max_new_tokens) or max_new_tokens
    eos = kwargs.get("eos_token_id", getattr(gc, "eos_token_id", None) if gc is not None else None)
    eos_ids = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
    pad = kwargs.get("pad_token_id", getattr(gc, "pad_token_id", None) if gc is not None else None)
    if pad is None:
        pad = eos_ids[0] if eos_ids else 0

    rank, world = self.pp_rank, self.pp_world
    dev = next(p for p in self.parameters()).device
    dtype = next((p.dtype for p in self.parameters() if p.is_floating_point() and p.dim() == 1), torch.float32)
    input_ids = inputs.to(dev)
    B, S = input_ids.shape
    H = self.config.hidden_size
    first, last = rank == 0, rank == world - 1
    n_mb = max(1, min(B, world))
    bounds = [(B * i) // n_mb for i in range(n_mb + 1)]
    rows = [bounds[i + 1] - bounds[i] for i in range(n_mb)]
    caches = [_new_cache(self, rows[m], dev) for m in range(n_mb)]
    out_new = torch.full((B, max_new_tokens), pad, dtype=torch.long, device=dev)
    finished = torch.zeros(B, dtype=torch.bool, device=dev)
    eos_t = torch.tensor(eos_ids, device=dev) if eos_ids else None
    pending = []          # outstanding isend handles (+ the tensors they read)
    self.first_token_time = 0.0
    self.next_token_time = []

    def sync():
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)

    def send(t, dst):
        if dst == rank:
            return
        t = t.contiguous()
        pending.append((dist.isend(t, dst), t))

    def drain(keep=0):
        while len(pending) > keep:
            h, _ = pending.pop(0)
            h.wait()

    local_ids = {}        # world == 1: ids pass through this dict instead of the ring
    t_start = time.perf_counter()
    for step in range(max_new_tokens):
        s_len = S if step == 0 else 1
        pos = torch.arange(S) if step == 0 else torch.tensor([S + step - 1])
        for m in range(n_mb):
            b0, b1 = bounds[m], bounds[m + 1]
            position_ids = pos.to(dev).unsqueeze(0).expand(rows[m], -1)
            if first:
                if step == 0:
                    ids = input_ids[b0:b1]
                elif world == 1:
                    ids = local_ids[m]
                else:
                    ids = torch.empty((rows[m], 1), dtype=torch.long, device=dev)
                    dist.recv(ids, src=world - 1)
                    out_new[b0:b1, step - 1] = ids[:, 0]
                out = self(input_ids=ids, position_ids=position_ids, past_key_values=caches[m], use_cache=True)
            else:
                hid = torch.empty((rows[m], s_len, H), dtype=dtype, device=dev)
                dist.recv(hid, src=rank - 1)
                out = self(inputs_embeds=hid, position_ids=position_ids, past_key_values=caches[m], use_cache=True)
            res = out.logits
            if last:
                nxt = torch.argmax(res[:, -1, :], dim=-1)
                if eos_t is not None:
                    nxt = torch.where(finished[b0:b1], torch.full_like(nxt, pad), nxt)
                    finished[b0:b1] |= torch.isin(nxt, eos_t)
                out_new[b0:b1, step] = nxt
                if step < max_new_tokens - 1:
                    if world == 1:
                        local_ids[m] = nxt.view(-1, 1)
                    else:
                        send(nxt.view(-1, 1), 0)
            else:
                send(res.to(dtype), rank + 1)
            drain(keep=2 * n_mb)
        # token-level streaming from the first stage: the ring has just delivered every sequence's token of the
        # previous step (on a single stage, of this step)
        if streamer is not None and first:
            if step == 0:
                streamer.put(input_ids.cpu())
            if world == 1:
                streamer.put(out_new[:, step].cpu())
            elif step > 0:
                streamer.put(out_new[:, step - 1].cpu())
        if step == 0:
            sync()
            self.first_token_time = time.perf_counter() - t_start
            t_prev = time.perf_counter()
        else:
            sync()
            now = time.perf_counter()
            self.next_token_time.append(now - t_prev)
            t_prev = now
    drain()
    # the last stage owns the sampled ids: share them so that every rank returns the same result
    if world > 1:
        dist.broadcast(out_new, src=world - 1)
    self.rest_cost_mean = sum(self.next_token_time) / max(1, len(self.next_token_time))
    result = torch.cat([input_ids, out_new], dim=1)
    if streamer is not None and first:
        if world > 1:
            streamer.put(out_new[:, max_new_tokens - 1].cpu())     # the last step's tokens came with the broadcast
        streamer.end()
    return result
