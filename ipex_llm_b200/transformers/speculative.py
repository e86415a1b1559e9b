"""Self-speculative decoding: a half-precision target verified against a sym_int4 draft of the same weights.

Counterpart of python/llm/src/ipex_llm/transformers/speculative.py of the reference (``speculative_generate``
:803-1269, adaptive ``th_stop_draft`` :1225-1236, KV cropping :478-496, sampling acceptance :1162-1188).

Both models share ONE KV cache (the package's block-grown cache with O(1) ``crop``):
  1. the draft appends its own K/V while it proposes up to ``max_step_draft`` tokens, stopping early when its
     confidence drops below ``th_stop_draft`` (after ``min_step_draft`` tokens);
  2. the cache is cropped back, the target scores ``[last accepted token, drafts...]`` in one forward (a short
     query against the long cache: the split-KV decode kernel on the GPU) and rewrites those K/V entries;
  3. greedy: the longest matching prefix is accepted plus the target's own next token; sampling: each draft
     token is accepted with probability ``min(1, p_target / p_draft)``, the first rejected position is
     resampled from ``max(0, p_target - p_draft)``;
  4. the cache is cropped to the accepted length and ``th_stop_draft`` adapts to the running acceptance rate.
"""
from __future__ import annotations

import time
from typing import Optional

import torch

from ..ops.kv_cache import DynamicFp8Cache, DynamicNormalCache
from ..utils.common import invalidInputError


def attach_draft_model(model, draft):
    """``from_pretrained(..., speculative=True)``: keep the draft on the target and expose the generate method."""
    import types
    model.draft_model = draft
    model.speculative_generate = types.MethodType(speculative_generate, model)
    clear_benchmarks(model)
    return model


def clear_benchmarks(self):
    self.first_token_time = 0
    self.generate_time = []
    self.draft_time = []
    self.verify_time = []
    self.draft_num = []
    self.accept_num = []
    self.n_drafted = 0
    self.n_matched = 0
    self.n_token_generated = 0
    self.e2e_time_without_first = 0


def _sync(device):
    if device.type == "cuda":
        torch.cuda.synchronize(device)


def _warp_logits(logits, temperature, top_k, top_p):
    logits = logits.float()
    if temperature is not None and temperature > 0 and temperature != 1.0:
        logits = logits / temperature
    if top_k:
        kth = torch.topk(logits, min(int(top_k), logits.shape[-1]), dim=-1).values[..., -1, None]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p is not None and top_p < 1.0:
        sl, si = torch.sort(logits, descending=True, dim=-1)
        probs = torch.softmax(sl, dim=-1)
        remove = probs.cumsum(dim=-1) - probs > top_p
        sl = sl.masked_fill(remove, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, si, sl)
    return logits


def _new_cache(model, x):
    from ..models.utils import use_quantize_kv_cache
    cfg = model.config
    if use_quantize_kv_cache(None, x, cfg.num_attention_heads, getattr(cfg, "num_key_value_heads", 1) or 1):
        return DynamicFp8Cache(cfg)
    return DynamicNormalCache(cfg)


def _crop(cache, length: int):
    cache.crop(length)


def _engine_pair(target, draft, need_len: int):
    """Flattened graph engines of target and draft with equal geometry (they share one cache), or None when
    either model is outside the engine's coverage."""
    import os
    if os.environ.get("IPEX_LLM_SPEC_ENGINE", "1") == "0":
        return None
    dev = next(target.parameters()).device
    if dev.type != "cuda" or next(draft.parameters()).device != dev:
        return None
    try:
        from ..engine import DecoderEngine, supports
        if not supports(target, {}) or not supports(draft, {}):
            return None
        max_len = (max(need_len, 2048) + 255) // 256 * 256
        pair = []
        for m, mb in ((target, 8), (draft, 1)):
            eng = getattr(m, "_ipex_engine", None)
            if eng is None or eng.max_batch < mb or eng.max_len != max_len:
                eng = DecoderEngine(m, max_batch=mb, max_len=max_len)
                m._ipex_engine = eng
            pair.append(eng)
        t, d = pair
        if t.kv_fp8 != d.kv_fp8 or t.dtype != d.dtype or t.n_kv != d.n_kv or t.hd != d.hd or \
                len(t.layers) != len(d.layers) or t.layers[0].o.tp is not None:
            return None
        return t, d
    except NotImplementedError:
        return None


def _speculative_generate_engine(self, t, d, input_ids, max_new_tokens, max_step_draft, th_stop_draft,
                                 auto_th_stop_draft, auto_parameters, hf_adjust, min_step_draft, do_sample,
                                 temperature, top_k, top_p, eos_ids, streamer):
    """The same algorithm on the two graph engines: every draft token is one graph replay of the int4 engine, the
    verification is ONE graph replay of the target engine scoring up to 8 tokens (multi-row GEMVs, the split-KV
    attention kernel with the new rows causal among themselves), and rejecting drafts is just not advancing the
    device-side length.  Host work per iteration: one read of the draft's confidence per proposal (the early
    stop needs it) and one read of the target's tokens."""
    device = input_ids.device
    clear_benchmarks(self)
    max_step_draft = max(1, min(max_step_draft, 7))       # current token + drafts are scored as <= 8 GEMV rows
    min_step_draft = min(min_step_draft, max_step_draft)
    out_ids = []
    tmp_matchness = 0.0
    step_verify = 0

    _sync(device)
    tic = time.time()
    logits = t.prefill(input_ids)                          # [1, V]; K/V of the prompt in t.cache
    d.bind_cache(t.cache, 1)
    if do_sample:
        probs = torch.softmax(_warp_logits(logits[0], temperature, top_k, top_p), dim=-1)
        current = int(torch.multinomial(probs, 1))
    else:
        current = int(torch.argmax(logits[0]))
    out_ids.append(current)
    n_past = input_ids.shape[1]
    _sync(device)
    self.first_token_time = time.time() - tic
    e2e_tic = time.time()
    if streamer is not None:
        streamer.put(input_ids.cpu())
        streamer.put(torch.tensor([[current]]))
    finished = bool(eos_ids) and current in eos_ids

    while len(out_ids) < max_new_tokens and not finished:
        _sync(device)
        t0 = time.time()
        # ---- 1. draft: graph replays of the int4 engine on the shared cache ----
        d.past_len[:1].fill_(n_past)
        d.tokens[:1].fill_(current)
        drafts, draft_probs = [], []
        for _ in range(max_step_draft):
            d.decode_step(1)
            row = d.logits[0]
            if do_sample:
                probs = torch.softmax(_warp_logits(row, temperature, top_k, top_p), dim=-1)
                nt = torch.multinomial(probs, 1).view(-1)
                d.tokens[:1].copy_(nt)
                conf = float(probs[nt[0]])
                tok = int(nt[0])
                draft_probs.append(probs)
            else:
                # confidence of the arg-max token = 1 / sum(exp(l - l_max))
                lf = row.float()
                conf, tok = float(1.0 / torch.exp(lf - lf.max()).sum()), int(d.tokens[0])
            drafts.append(tok)
            if len(out_ids) + len(drafts) >= max_new_tokens:
                break
            if conf < th_stop_draft and len(drafts) >= min_step_draft:
                break
        drafted_n = len(drafts)
        _sync(device)
        t1 = time.time()
        self.draft_time.append(t1 - t0)

        # ---- 2. verify: one pass of the target over [current, drafts] ----
        S = drafted_n + 1
        t.vtokens[:S].copy_(torch.tensor([current] + drafts, dtype=torch.int64), non_blocking=False)
        t.past_len[:1].fill_(n_past)
        t.verify_step(S)
        if not do_sample:
            target_tokens = t.vout[:S].tolist()
            n_match = 0
            while n_match < drafted_n and target_tokens[n_match] == drafts[n_match]:
                n_match += 1
            accepted = target_tokens[: n_match + 1]
        else:
            v_logits = t.logits[:S]
            n_match, accepted = 0, []
            for i in range(drafted_n):
                p_t = torch.softmax(_warp_logits(v_logits[i], temperature, top_k, top_p), dim=-1)
                p_d = draft_probs[i]
                ratio = float((p_t[drafts[i]] / p_d[drafts[i]].clamp_min(1e-20)).clamp(max=1.0))
                if float(torch.rand(())) <= ratio:
                    accepted.append(drafts[i])
                    n_match += 1
                else:
                    resid = (p_t - p_d).clamp_min(0)
                    resid = resid / resid.sum().clamp_min(1e-20)
                    accepted.append(int(torch.multinomial(resid, 1)))
                    break
            if n_match == drafted_n:
                p_t = torch.softmax(_warp_logits(v_logits[drafted_n], temperature, top_k, top_p), dim=-1)
                accepted.append(int(torch.multinomial(p_t, 1)))
        _sync(device)
        t2 = time.time()
        self.verify_time.append(t2 - t1)
        self.generate_time.append(t2 - t0)

        # ---- 3. commit: rows of [current, matched drafts] stay, the rest is dead storage past the length ----
        n_past += n_match + 1
        room = max_new_tokens - len(out_ids)
        accepted = accepted[:room]
        out_ids.extend(accepted)
        if streamer is not None:
            streamer.put(torch.tensor([accepted]))
        current = accepted[-1]
        self.draft_num.append(drafted_n)
        self.accept_num.append(n_match)
        self.n_drafted += drafted_n
        self.n_matched += n_match
        step_verify += 1

        # ---- 4. adapt the early-stop threshold to the observed acceptance ----
        if auto_th_stop_draft and step_verify % auto_parameters[0] == 0:
            tmp_matchness = auto_parameters[1] * tmp_matchness + (1 - auto_parameters[1]) * (n_match / drafted_n)
            if tmp_matchness < auto_parameters[2]:
                new_th = th_stop_draft + auto_parameters[3]
            elif drafted_n == max_step_draft:
                new_th = th_stop_draft
            else:
                new_th = th_stop_draft - auto_parameters[3]
            th_stop_draft = auto_parameters[4] * th_stop_draft + (1 - auto_parameters[4]) * new_th
        if hf_adjust:
            max_step_draft = min(7, max_step_draft + 1) if n_match == max_step_draft else max(1, max_step_draft - 1)
        for e in eos_ids:
            if e in out_ids:
                out_ids = out_ids[: out_ids.index(e) + 1]
                finished = True
                break

    if streamer is not None:
        streamer.end()
    t.past_len[:1].fill_(n_past)
    t.sync_cache_length(n_past)
    _sync(device)
    self.n_token_generated = len(out_ids)
    self.e2e_time_without_first = time.time() - e2e_tic
    self.th_stop_draft = th_stop_draft
    new = torch.tensor([out_ids], dtype=input_ids.dtype, device=device)
    return torch.cat([input_ids, new], dim=-1)


@torch.no_grad()
def speculative_generate(self, inputs: Optional[torch.Tensor] = None, draft_model=None, max_new_tokens=10,
                         max_step_draft=8, th_stop_draft=0.8, auto_th_stop_draft=True,
                         auto_parameters=(1, 0.5, 0.9, 1e-2, 0.9), hf_adjust=False, min_step_draft=3,
                         generation_config=None, attention_mask=None, streamer=None, **sampling_kwargs):
    invalidInputError(draft_model is not None, "Draft model should be provided.")
    invalidInputError(inputs is not None and inputs.dim() == 2, "inputs must be a [batch, seq] tensor of token ids")
    invalidInputError(inputs.shape[0] == 1, "speculative decoding supports batch size 1")
    min_step_draft = max(1, min_step_draft)
    if inputs.device.type == "cuda" and (attention_mask is None or bool(attention_mask.all())):
        pair = _engine_pair(self, draft_model, inputs.shape[1] + max_new_tokens + 16)
        if pair is not None:
            gc_ = generation_config or self.generation_config
            sample_ = sampling_kwargs.get("do_sample", getattr(gc_, "do_sample", False))
            eos_ = sampling_kwargs.get("eos_token_id", getattr(gc_, "eos_token_id", None))
            return _speculative_generate_engine(
                self, pair[0], pair[1], inputs, max_new_tokens, max_step_draft, th_stop_draft, auto_th_stop_draft,
                auto_parameters, hf_adjust, min_step_draft, sample_,
                sampling_kwargs.get("temperature", getattr(gc_, "temperature", 1.0)),
                (sampling_kwargs.get("top_k", getattr(gc_, "top_k", None)) if sample_ else None),
                (sampling_kwargs.get("top_p", getattr(gc_, "top_p", None)) if sample_ else None),
                [] if eos_ is None else ([eos_] if isinstance(eos_, int) else list(eos_)), streamer)
    gc = generation_config or self.generation_config
    do_sample = sampling_kwargs.get("do_sample", getattr(gc, "do_sample", False))
    temperature = sampling_kwargs.get("temperature", getattr(gc, "temperature", 1.0))
    top_k = sampling_kwargs.get("top_k", getattr(gc, "top_k", None)) if do_sample else None
    top_p = sampling_kwargs.get("top_p", getattr(gc, "top_p", None)) if do_sample else None
    eos = sampling_kwargs.get("eos_token_id", getattr(gc, "eos_token_id", None))
    eos_ids = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))

    device = inputs.device
    input_ids = inputs
    clear_benchmarks(self)
    draft_gen_length = max_step_draft + 6 if hf_adjust else max_step_draft + 1
    generate_ids = torch.empty((1, max_new_tokens + draft_gen_length + 1), dtype=torch.long, device=device)
    cache = _new_cache(self, input_ids)
    tmp_matchness = 0.0
    step = 0
    step_verify = 0
    e2e_tic = 0.0
    n_past = 0
    finished = False

    def pick(logits_row):
        if do_sample:
            probs = torch.softmax(_warp_logits(logits_row, temperature, top_k, top_p), dim=-1)
            return torch.multinomial(probs, 1).view(-1), probs
        return torch.argmax(logits_row, dim=-1).view(-1), None

    # ---- step 0: the target consumes the prompt ----
    _sync(device)
    tic = time.time()
    out = self(input_ids=input_ids, past_key_values=cache, use_cache=True)
    cache = out.past_key_values if out.past_key_values is not None else cache
    tok, _ = pick(out.logits[0, -1])
    generate_ids[0, 0] = tok[0]
    current = tok.view(1, 1)
    n_past = input_ids.shape[1]
    step = 1
    _sync(device)
    self.first_token_time = time.time() - tic
    e2e_tic = time.time()
    if streamer is not None:
        streamer.put(input_ids.cpu())
        streamer.put(current.cpu())
    if eos_ids and int(tok[0]) in eos_ids:
        finished = True

    while step < max_new_tokens and not finished:
        # ---- 1. draft ----
        _sync(device)
        t0 = time.time()
        if hasattr(cache, "reserve"):
            cache.reserve(max_step_draft + 2)
        drafts, draft_probs = [], []
        d_in = current
        for step_draft in range(max_step_draft):
            d_out = draft_model(input_ids=d_in, past_key_values=cache, use_cache=True)
            row = d_out.logits[0, -1]
            if do_sample:
                probs = torch.softmax(_warp_logits(row, temperature, top_k, top_p), dim=-1)
                nt = torch.multinomial(probs, 1).view(-1)
                conf = probs[nt[0]]
                draft_probs.append(probs)
            else:
                probs = torch.softmax(row.float(), dim=-1)
                nt = torch.argmax(row, dim=-1).view(-1)
                conf = probs[nt[0]]
            drafts.append(nt)
            d_in = nt.view(1, 1)
            if step + len(drafts) >= max_new_tokens:
                break
            # early stop when the draft is not confident (after a minimum number of proposals)
            if float(conf) < th_stop_draft and len(drafts) >= min_step_draft:
                break
        drafted_n = len(drafts)
        draft_tokens = torch.stack(drafts, dim=1)  # [1, n]
        _sync(device)
        t1 = time.time()
        self.draft_time.append(t1 - t0)

        # ---- 2. verify: the target scores the last accepted token and every draft in one forward ----
        _crop(cache, n_past)
        verify_in = torch.cat([current, draft_tokens], dim=1)      # [1, n+1]
        v_out = self(input_ids=verify_in, past_key_values=cache, use_cache=True)
        v_logits = v_out.logits[0]
        if v_logits.shape[0] != verify_in.shape[1]:
            invalidInputError(False, "the target returned logits for the last position only; disable lm_head "
                                     "slicing (IPEX_LLM_LAST_LM_HEAD=0) is not needed for <= 10 tokens")
        if not do_sample:
            target_tokens = torch.argmax(v_logits, dim=-1)          # [n+1]
            match = (target_tokens[:drafted_n] == draft_tokens[0]).int()
            n_match = int(match.cumprod(dim=0).sum())
            accepted = target_tokens[: n_match + 1]
        else:
            n_match = 0
            accepted_list = []
            for i in range(drafted_n):
                p_t = torch.softmax(_warp_logits(v_logits[i], temperature, top_k, top_p), dim=-1)
                p_d = draft_probs[i]
                tok_i = draft_tokens[0, i]
                ratio = (p_t[tok_i] / p_d[tok_i].clamp_min(1e-20)).clamp(max=1.0)
                if torch.rand((), device=device) <= ratio:
                    accepted_list.append(tok_i.view(1))
                    n_match += 1
                else:
                    resid = (p_t - p_d).clamp_min(0)
                    resid = resid / resid.sum().clamp_min(1e-20)
                    accepted_list.append(torch.multinomial(resid, 1).view(1))
                    break
            if n_match == drafted_n:
                p_t = torch.softmax(_warp_logits(v_logits[drafted_n], temperature, top_k, top_p), dim=-1)
                accepted_list.append(torch.multinomial(p_t, 1).view(1))
            accepted = torch.cat(accepted_list)
        _sync(device)
        t2 = time.time()
        self.verify_time.append(t2 - t1)
        self.generate_time.append(t2 - t0)

        # ---- 3. commit: keep the K/V of [current, matched drafts]; the new last token has none yet ----
        n_new = accepted.shape[0]
        n_past = n_past + n_match + 1
        _crop(cache, n_past)
        room = max_new_tokens - step
        accepted = accepted[:room] if n_new > room else accepted
        n_new = accepted.shape[0]
        generate_ids[0, step: step + n_new] = accepted
        if streamer is not None:
            streamer.put(accepted.view(1, -1).cpu())
        step += n_new
        current = accepted[-1:].view(1, 1)
        self.draft_num.append(drafted_n)
        self.accept_num.append(n_match)
        self.n_drafted += drafted_n
        self.n_matched += n_match
        step_verify += 1

        # ---- 4. adapt the early-stop threshold to the observed acceptance ----
        if auto_th_stop_draft and step_verify % auto_parameters[0] == 0:
            tmp_matchness = auto_parameters[1] * tmp_matchness + (1 - auto_parameters[1]) * (n_match / drafted_n)
            if tmp_matchness < auto_parameters[2]:
                new_th = th_stop_draft + auto_parameters[3]
            elif drafted_n == max_step_draft:
                new_th = th_stop_draft
            else:
                new_th = th_stop_draft - auto_parameters[3]
            th_stop_draft = auto_parameters[4] * th_stop_draft + (1 - auto_parameters[4]) * new_th
        if hf_adjust:
            if n_match == max_step_draft:
                max_step_draft = min(draft_gen_length - 1, max_step_draft + 1)
            else:
                max_step_draft = max(1, max_step_draft - 1)

        if eos_ids:
            out_list = generate_ids[0, :step].tolist()
            for e in eos_ids:
                if e in out_list:
                    step = out_list.index(e) + 1
                    finished = True
                    break

    if streamer is not None:
        streamer.end()
    step = min(step, max_new_tokens)
    _sync(device)
    self.n_token_generated = step
    self.e2e_time_without_first = time.time() - e2e_tic
    self.th_stop_draft = th_stop_draft
    return torch.cat([input_ids, generate_ids[:, :step]], dim=-1)
