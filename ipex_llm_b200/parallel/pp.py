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
from typing import Optional

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
    os.environ.setdefault("RANK", "0")             # plain `python` start: a pipeline of one stage
    os.environ.setdefault("WORLD_SIZE", "1")
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
    base = getattr(model, "model", None)
    invalidInputError(base is not None and hasattr(base, "layers") and hasattr(base, "embed_tokens"),
                      f"pipeline parallelism slices `model.model.layers`; {type(model).__name__} is laid out "
                      "differently (GPT-2 / GPT-J / Bloom style `transformer.h`)")
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
        # models that scale their input embeddings inside the model forward (Granite, and MiniCPM checkpoints mapped
        # to it) would scale the hidden states a later stage receives as `inputs_embeds` once more
        if hasattr(base, "embedding_multiplier"):
            base.embedding_multiplier = 1.0
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


def _back_group(model):
    """Process group of the ids ring (last stage -> first stage).  With two stages the ring shares its rank pair
    with the hidden-state hand-over; on one communicator the two directions would be queued on one stream in an
    order the peer does not mirror (stage 0: send h0, send h1, recv ids0; stage 1: recv h0, send ids0, recv h1), which
    only works while the messages fit the transport's buffers.  A second communicator keeps them independent."""
    g = model.__dict__.get("_pp_back_group")
    if g is None and model.pp_world > 1:
        g = dist.new_group(ranks=list(range(model.pp_world)))
        model.__dict__["_pp_back_group"] = g
    return g


def _stage_engines_ok(model, dev, attention_mask) -> bool:
    """True when EVERY stage can run its slice on the flattened graph engine (all ranks take the same decision)."""
    ok = dev.type == "cuda" and os.environ.get("IPEX_LLM_PP_ENGINE", "1") != "0" and \
        (attention_mask is None or bool(attention_mask.all()))
    if ok:
        from ..engine import supports
        ok = supports(model, {})
    if model.pp_world > 1:
        t = torch.tensor([int(ok)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        ok = bool(int(t.item()))
    return ok


@torch.no_grad()
def _generate_with_stage_engines(model, input_ids, max_new_tokens, eos_ids, pad, streamer):
    """Greedy pipeline generation on the flattened engines: every stage runs its slice of the layers as one
    CUDA-graph replay per (micro-batch, token), hidden states travel stage to stage with NCCL p2p enqueued on the
    stream, sampled ids go from the last stage back to the first, and the host never waits for the device between
    tokens (one synchronisation after the prompt pass for the first-token time, one at the end).  Each micro-batch
    has its own engine (activations, KV cache, graph) over the stage's shared flattened weights."""
    from ..engine import DecoderEngine
    rank, world = model.pp_rank, model.pp_world
    dev = input_ids.device
    B, S = input_ids.shape
    H = model.config.hidden_size
    first, last = rank == 0, rank == world - 1
    n_mb = max(1, min(B, world))
    bounds = [(B * i) // n_mb for i in range(n_mb + 1)]
    rows = [bounds[i + 1] - bounds[i] for i in range(n_mb)]
    need_len = (max(S + max_new_tokens + 1, 2048) + 255) // 256 * 256
    engs = model.__dict__.get("_pp_engines") or []
    if len(engs) < n_mb or engs[0].max_batch < max(rows) or engs[0].max_len < need_len:
        base = DecoderEngine(model, max_batch=max(rows), max_len=need_len)
        engs = [base] + [base.clone_for_microbatch() for _ in range(n_mb - 1)]
        model.__dict__["_pp_engines"] = engs
    dtype = engs[0].dtype
    back = _back_group(model)
    out_new = torch.full((B, max_new_tokens), pad, dtype=torch.long, device=dev)
    finished = torch.zeros(B, dtype=torch.bool, device=dev)
    eos_t = torch.tensor(eos_ids, device=dev) if eos_ids else None
    sends = [None] * n_mb            # the isend that still reads each engine's hand-over buffer
    keep = []                         # prompt-pass tensors an isend still reads
    model.first_token_time = 0.0
    model.next_token_time = []
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start = time.perf_counter()
    t_first = t_start
    for step in range(max_new_tokens):
        for m in range(n_mb):
            e, r, b0, b1 = engs[m], rows[m], bounds[m], bounds[m + 1]
            if sends[m] is not None:
                sends[m].wait()               # stream-level: the next write of the buffer comes after the send
                sends[m] = None
            if step == 0:
                if first:
                    x = input_ids[b0:b1]
                else:
                    x = torch.empty((r, S, H), dtype=dtype, device=dev)
                    dist.recv(x, src=rank - 1)
                out = e.prefill_stage(x)
                if last:
                    e.tokens[:r] = torch.argmax(out, dim=-1)
                else:
                    out = out.contiguous()
                    keep.append(out)
                    sends[m] = dist.isend(out, rank + 1)
            else:
                if first and world > 1:
                    dist.recv(e.tokens[:r], src=world - 1, group=back)
                    out_new[b0:b1, step - 1] = e.tokens[:r]
                elif not first:
                    dist.recv(e.h[0][:r], src=rank - 1)
                e.decode_step(r, use_graph=True)
                if not last:
                    sends[m] = dist.isend(e.h[0][:r], rank + 1)
            if last:
                nxt = e.tokens[:r]
                if eos_t is not None:
                    nxt = torch.where(finished[b0:b1], torch.full_like(nxt, pad), nxt)
                    finished[b0:b1] |= torch.isin(nxt, eos_t)
                    e.tokens[:r] = nxt
                out_new[b0:b1, step] = nxt
                if step < max_new_tokens - 1 and world > 1:
                    ids = nxt.clone()
                    keep.append(ids)
                    sends[m] = dist.isend(ids, 0, group=back)
        if len(keep) > 4 * n_mb:
            del keep[:len(keep) - 4 * n_mb]   # older sends were waited for when their engine came round again
        if streamer is not None and first:
            if step == 0:
                streamer.put(input_ids.cpu())
            if world == 1:
                streamer.put(out_new[:, step].cpu())
            elif step > 0:
                streamer.put(out_new[:, step - 1].cpu())
        if step == 0:
            torch.cuda.synchronize(dev)
            t_first = time.perf_counter()
            model.first_token_time = t_first - t_start
            ev0.record()
    for h in sends:
        if h is not None:
            h.wait()
    ev1.record()                      # decode steps timed on the device (the caller takes the max over the stages)
    if world > 1:
        dist.broadcast(out_new, src=world - 1)
    torch.cuda.synchronize(dev)
    rest = ev0.elapsed_time(ev1) * 1e-3 / max(1, max_new_tokens - 1) if max_new_tokens > 1 else 0.0
    model.next_token_time = [rest] * max(0, max_new_tokens - 1)
    model.rest_cost_mean = rest
    result = torch.cat([input_ids, out_new], dim=1)
    if streamer is not None and first:
        if world > 1:
            streamer.put(out_new[:, max_new_tokens - 1].cpu())
        streamer.end()
    return result


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
    if _stage_engines_ok(self, dev, attention_mask):
        return _generate_with_stage_engines(self, input_ids, max_new_tokens, eos_ids, pad, streamer)
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

    back = _back_group(self)

    def send(t, dst, group=None):
        if dst == rank:
            return
        t = t.contiguous()
        pending.append((dist.isend(t, dst, group=group), t))

    def drain(keep=0):
        while len(pending) > keep:
            h, _ = pending.pop(0)
            h.wait()

    local_ids = {}        # world == 1: ids pass through this dict instead of the ring
    # padded prompts: every stage masks the padding and counts positions from each row's first real token
    mask = None
    if attention_mask is not None and not bool(attention_mask.all()):
        mask = torch.ones((B, S + max_new_tokens), dtype=torch.long, device=dev)
        mask[:, :S] = attention_mask.to(dev)
        prompt_pos = (mask[:, :S].cumsum(-1) - 1).clamp_(min=0)
        prompt_len = mask[:, :S].sum(-1, keepdim=True)
    t_start = time.perf_counter()
    for step in range(max_new_tokens):
        s_len = S if step == 0 else 1
        pos = torch.arange(S) if step == 0 else torch.tensor([S + step - 1])
        for m in range(n_mb):
            b0, b1 = bounds[m], bounds[m + 1]
            if mask is None:
                position_ids = pos.to(dev).unsqueeze(0).expand(rows[m], -1)
                mkw = {}
            else:
                position_ids = prompt_pos[b0:b1] if step == 0 else prompt_len[b0:b1] + (step - 1)
                mkw = dict(attention_mask=mask[b0:b1, :S + step])
            if first:
                if step == 0:
                    ids = input_ids[b0:b1]
                elif world == 1:
                    ids = local_ids[m]
                else:
                    ids = torch.empty((rows[m], 1), dtype=torch.long, device=dev)
                    dist.recv(ids, src=world - 1, group=back)
                    out_new[b0:b1, step - 1] = ids[:, 0]
                kw = dict(input_ids=ids)
            else:
                hid = torch.empty((rows[m], s_len, H), dtype=dtype, device=dev)
                dist.recv(hid, src=rank - 1)
                kw = dict(inputs_embeds=hid)
            if last:
                res = self(position_ids=position_ids, past_key_values=caches[m], use_cache=True, **kw, **mkw).logits
            else:
                # the hidden states themselves: a causal-LM wrapper may scale or soft-cap what it takes for logits
                # (Cohere, Granite, Gemma-2), which must happen on the last stage only
                res = self.model(position_ids=position_ids, past_key_values=caches[m], use_cache=True,
                                 **kw, **mkw).last_hidden_state
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
                        send(nxt.view(-1, 1), 0, group=back)
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
