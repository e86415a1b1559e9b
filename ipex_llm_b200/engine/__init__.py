"""Native decode engine: selection and the ``generate`` loop built on it.

``engine_generate`` is what ``model.generate`` runs for a converted CUDA model of a supported family: the engine's
prompt pass (flattened tcgen05 pass for unmasked prompts, module tree otherwise), then one CUDA-graph replay per
token.  Per-token timing follows the reference's
``BenchmarkWrapper`` definitions (first token = prompt pass + first sampling, rest = mean of the remaining steps;
python/llm/src/ipex_llm/utils/benchmark_util_4_47.py:3376-3393) and is left on the model as
``first_token_time`` / ``rest_cost_mean`` / ``last_token_time``.
"""
from __future__ import annotations

import time

import torch

from ..models.registry import family_for
from ..ops import cuda_ops
from ..ops.linear import LowBitLinear
from ..utils.tracing import nvtx_range
from .decoder_engine import DecoderEngine

_UNSUPPORTED_KW = ("num_beams", "penalty_alpha", "num_return_sequences", "constraints", "force_words_ids",
                   "output_scores", "output_attentions", "output_hidden_states", "return_dict_in_generate",
                   "inputs_embeds", "past_key_values")


def supports(model, kwargs) -> bool:
    fam = family_for(model)
    if fam is None or fam.engine not in ("llama", "mixtral"):
        return False
    if getattr(model, "_ipex_engine_disabled", False):
        return False
    if getattr(getattr(model, "config", None), "ipex_alibi", False):
        return False            # linear attention biases instead of rotary positions: module path
    from .. import config as _cfg
    if _cfg.kv_cache_format() == "int4":
        return False            # the 4-bit KV cache lives on the module path (the fused kernels read fp16 / e5m2)
    for k in _UNSUPPORTED_KW:
        v = kwargs.get(k)
        if v is not None and v not in (False, 1):
            return False
    try:
        # (a pipeline stage keeps only its slice of the layers; the others are parameter-free stand-ins)
        blk = next(b for b in model.model.layers if hasattr(b, "self_attn"))
    except Exception:  # noqa: BLE001
        return False
    if not hasattr(blk.self_attn, "qkv_proj"):
        return False
    mlp_mods = ()
    if hasattr(blk.mlp, "experts"):
        # sparse mixture-of-experts layers: the expert bank must be the packed one the MoE kernels read
        ex = blk.mlp.experts
        if not (hasattr(ex, "intermediate_dim") and hasattr(blk.mlp, "gate") and cuda_ops.moe_supported(ex)) or \
                getattr(ex, "_tp_group", None) is not None or getattr(blk.mlp, "shared_expert", None) is not None:
            return False
    elif hasattr(blk.mlp, "gate_proj"):
        mlp_mods = (blk.mlp.gate_proj, blk.mlp.down_proj)
    else:
        return False
    for mod in (blk.self_attn.qkv_proj, blk.self_attn.o_proj) + mlp_mods:
        if isinstance(mod, LowBitLinear) and not cuda_ops.is_tiled(mod.weight.qtype):
            return False
    hd = getattr(model.config, "head_dim", None) or model.config.hidden_size // model.config.num_attention_heads
    if hd not in (64, 128, 256):
        return False
    if getattr(model.config, "sliding_window", None) and getattr(model.config, "use_sliding_window", True) and \
            model.config.model_type in ("mistral",) and model.config.sliding_window < 4096:
        return False
    return True


def get_engine(model, batch: int, need_len: int) -> DecoderEngine:
    eng = getattr(model, "_ipex_engine", None)
    if eng is None or eng.max_batch < batch or eng.max_len < need_len:
        max_len = max(need_len, 2048)
        max_len = (max_len + 255) // 256 * 256
        eng = DecoderEngine(model, max_batch=max(batch, 1), max_len=max_len)
        model._ipex_engine = eng
    return eng


def _sample(logits, do_sample, temperature, top_k, top_p):
    if not do_sample:
        return torch.argmax(logits, dim=-1)
    logits = logits.float()
    if temperature and temperature != 1.0:
        logits = logits / temperature
    if top_k:
        kth = torch.topk(logits, min(top_k, logits.shape[-1]), dim=-1).values[..., -1, None]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p and top_p < 1.0:
        sorted_logits, sorted_idx = torch.sort(logits, descending=True, dim=-1)
        cum = torch.softmax(sorted_logits, dim=-1).cumsum(dim=-1)
        remove = cum - torch.softmax(sorted_logits, dim=-1) > top_p
        sorted_logits = sorted_logits.masked_fill(remove, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, sorted_idx, sorted_logits)
    return torch.multinomial(torch.softmax(logits, dim=-1), 1).squeeze(-1)


@torch.no_grad()
def engine_generate(model, input_ids, generation_config=None, streamer=None, attention_mask=None, **kwargs):
    gc = generation_config or model.generation_config
    max_new = kwargs.get("max_new_tokens", None)
    if max_new is None:
        max_len_kw = kwargs.get("max_length", None) or getattr(gc, "max_length", None)
        max_new = getattr(gc, "max_new_tokens", None) or (max_len_kw - input_ids.shape[1] if max_len_kw else 20)
    min_new = kwargs.get("min_new_tokens", getattr(gc, "min_new_tokens", None)) or 0
    do_sample = kwargs.get("do_sample", getattr(gc, "do_sample", False))
    temperature = kwargs.get("temperature", getattr(gc, "temperature", 1.0))
    top_k = kwargs.get("top_k", getattr(gc, "top_k", None)) if do_sample else None
    top_p = kwargs.get("top_p", getattr(gc, "top_p", None)) if do_sample else None
    rep_pen = kwargs.get("repetition_penalty", getattr(gc, "repetition_penalty", None))
    eos = kwargs.get("eos_token_id", getattr(gc, "eos_token_id", None))
    pad = kwargs.get("pad_token_id", getattr(gc, "pad_token_id", None))
    eos_ids = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
    if pad is None:
        pad = eos_ids[0] if eos_ids else 0
    B, S = input_ids.shape
    if attention_mask is not None and not bool(attention_mask.all()):
        # left-padded batches need per-row positions: use the module path
        model._ipex_engine_disabled = True
        try:
            return model.generate(input_ids, generation_config=generation_config, streamer=streamer,
                                  attention_mask=attention_mask, **kwargs)
        finally:
            model._ipex_engine_disabled = False
    eng = get_engine(model, B, S + max_new + 1)

    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with nvtx_range("ipex_llm.prefill"):
        logits = eng.prefill(input_ids)
    if rep_pen and rep_pen != 1.0:
        cuda_ops.repetition_penalty_inplace(logits, input_ids, rep_pen)
    nxt = _sample(logits, do_sample, temperature, top_k, top_p)
    out = torch.full((B, S + max_new), pad, dtype=input_ids.dtype, device=input_ids.device)
    out[:, :S] = input_ids
    out[:, S] = nxt
    finished = torch.zeros(B, dtype=torch.bool, device=input_ids.device)
    eos_t = torch.tensor(eos_ids, device=input_ids.device) if eos_ids else None
    if eos_t is not None and min_new <= 1:
        finished |= torch.isin(nxt, eos_t)
    if streamer is not None:
        streamer.put(input_ids.cpu())
        streamer.put(nxt.cpu())
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    model.first_token_time = t1 - t0

    eng.tokens[:B] = nxt
    n_gen = 1
    graph_greedy = not do_sample and not (rep_pen and rep_pen != 1.0)
    step_times = []
    check_every = 16 if streamer is None else 1
    while n_gen < max_new:
        ts = time.perf_counter()
        with nvtx_range("ipex_llm.decode_step"):
            eng.decode_step(B)
        if graph_greedy:
            nxt = eng.tokens[:B]
        else:
            lg = eng.gather_logits(B).clone()      # a no-op unless the lm_head is vocabulary-parallel
            if rep_pen and rep_pen != 1.0:
                cuda_ops.repetition_penalty_inplace(lg, out[:, :S + n_gen], rep_pen)
            nxt = _sample(lg, do_sample, temperature, top_k, top_p)
            eng.tokens[:B] = nxt
        if eos_t is not None:
            nxt = torch.where(finished, torch.full_like(nxt, pad), nxt)
            if n_gen + 1 > min_new:
                finished = finished | torch.isin(nxt, eos_t)
        out[:, S + n_gen] = nxt
        n_gen += 1
        if streamer is not None:
            streamer.put(nxt.cpu())
        if eos_t is not None and (n_gen % check_every == 0) and bool(finished.all()):
            break
        step_times.append(time.perf_counter() - ts)
    torch.cuda.synchronize()
    t2 = time.perf_counter()
    if streamer is not None:
        streamer.end()
    eng.sync_cache_length(S + n_gen - 1)
    model.rest_cost_mean = (t2 - t1) / max(1, n_gen - 1)
    model.last_token_time = step_times
    model.n_generated = n_gen
    return out[:, :S + n_gen]


@torch.no_grad()
def prefill_host(model, input_ids, max_new_tokens: int = 256):
    """Serving-style API, step 1: run the prompt (host or device token ids ``[B, S]``) and return the first
    sampled (greedy) token of every sequence as a pinned host tensor.  Sets up the decode engine for up to
    ``max_new_tokens`` further ``decode_step`` calls."""
    dev = next(model.parameters()).device
    ids = input_ids.to(dev, non_blocking=True)
    B, S = ids.shape
    eng = get_engine(model, B, S + max_new_tokens + 1)
    logits = eng.prefill(ids)
    nxt = torch.argmax(logits, dim=-1)
    eng.tokens[:B] = nxt
    out = torch.empty(B, dtype=torch.int64).pin_memory()
    out.copy_(nxt, non_blocking=True)
    torch.cuda.current_stream().synchronize()
    return out


@torch.no_grad()
def decode_step_host(model, tokens_host):
    """Serving-style API, step 2..n: feed the token chosen for every sequence (pinned host tensor ``[B]``, e.g.
    after host-side sampling or stop-word handling), run one decode step, return the next greedy tokens as a
    pinned host tensor.  Both copies are part of the call."""
    eng = getattr(model, "_ipex_engine", None)
    if eng is None or eng.cache is None:
        raise RuntimeError("call model.prefill(input_ids) (or generate) before decode_step")
    B = tokens_host.shape[0]
    eng.tokens[:B].copy_(tokens_host, non_blocking=True)
    eng.decode_step(B)
    out = eng.__dict__.get("_host_out")
    if out is None or out.shape[0] != B:
        out = torch.empty(B, dtype=torch.int64).pin_memory()
        eng._host_out = out
    out.copy_(eng.tokens[:B], non_blocking=True)
    torch.cuda.current_stream().synchronize()
    return out
