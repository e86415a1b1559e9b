"""Prompt-lookup decoding: draft tokens come from n-gram matches in the text seen so far, no draft model.

Counterpart of python/llm/src/ipex_llm/transformers/lookup.py of the reference (candidate generator :145-270,
``lookup_generate`` :274-457; ``IPEX_LLM_PERFORMANCE_MODE=1`` turns it on with ``lookahead=2`` for prompts of 100+
tokens, :50-136).  The verification forward scores ``1 + lookahead`` tokens against the cache, which is the
short-query case of the split-KV decode kernel.
"""
from __future__ import annotations

import random
import time
from typing import Optional

import torch

from ..utils.common import invalidInputError
from .speculative import _new_cache, _sync, _warp_logits


class PromptLookupCandidateGenerator:
    """Keeps a table ``n-gram -> first position where it occurred`` over prompt + generated tokens and proposes
    the ``num_output_tokens`` tokens that followed the longest matching suffix n-gram."""

    def __init__(self, num_output_tokens: int = 10, max_matching_ngram_size: int = None, device: str = "b200"):
        self.num_output_tokens = num_output_tokens
        self.max_matching_ngram_size = max_matching_ngram_size if max_matching_ngram_size else 2
        self.max_candidates = 9
        self.min_candidates = 0
        self.lookup_table = {}
        invalidInputError(self.max_matching_ngram_size > 0 and self.num_output_tokens > 0,
                          "Invalid max_matching_ngram_size or num_output_tokens")

    def init_look_up_table(self, input_ids: torch.LongTensor):
        ids = input_ids[0].tolist()
        for n in range(min(self.max_matching_ngram_size, len(ids)), 0, -1):
            for idx in range(len(ids) - n + 1):
                self.lookup_table.setdefault(tuple(ids[idx: idx + n]), idx)

    def update_look_up_table(self, new_input_ids: torch.LongTensor):
        ids = new_input_ids[0].tolist()
        m = self.max_matching_ngram_size
        window = ids[-m:]
        for k in range(len(window)):
            key = tuple(window[k:])
            self.lookup_table.setdefault(key, len(ids) - len(key))

    def get_candidates(self, input_ids: torch.LongTensor):
        """Returns ``input_ids`` extended by the proposed continuation (unchanged when nothing matches)."""
        if self.num_output_tokens == 0:
            return input_ids, None
        ids = input_ids[0].tolist()
        L = len(ids)
        for n in range(min(self.max_matching_ngram_size, L - 1), 0, -1):
            idx = self.lookup_table.get(tuple(ids[-n:]))
            if idx is None:
                continue
            start, end = idx + n, min(idx + n + self.num_output_tokens, L)
            if start < end:
                chosen = input_ids[0, start:end].unsqueeze(0)
                return torch.cat((input_ids, chosen), dim=1), None
        return input_ids, None

    def update_candidate_strategy(self, candidate_num: int, num_matches: int, accept_rate: float):
        """More candidates after a full match, fewer (randomised by the running accept rate) after misses."""
        if self.num_output_tokens == 0:
            if random.random() - 0.15 <= accept_rate:
                self.num_output_tokens = 1
        elif num_matches == self.num_output_tokens:
            self.num_output_tokens = min(self.num_output_tokens + 1, self.max_candidates)
        elif candidate_num > num_matches:
            if random.random() + 0.1 * (candidate_num - num_matches) > accept_rate:
                self.num_output_tokens = max(self.num_output_tokens - 1, self.min_candidates)


@torch.no_grad()
def lookup_generate(self, inputs: Optional[torch.Tensor] = None, max_new_tokens: int = 10, num_output_tokens: int = 10,
                    max_matching_ngram_size: int = None, generation_config=None, attention_mask=None, streamer=None,
                    lookahead: int = None, **sampling_kwargs):
    if lookahead:
        num_output_tokens = lookahead
    invalidInputError(inputs is not None and inputs.shape[0] == 1, "lookup decoding supports batch size 1")
    gc = generation_config or self.generation_config
    do_sample = sampling_kwargs.get("do_sample", getattr(gc, "do_sample", False))
    temperature = sampling_kwargs.get("temperature", getattr(gc, "temperature", 1.0))
    top_k = sampling_kwargs.get("top_k", getattr(gc, "top_k", None)) if do_sample else None
    top_p = sampling_kwargs.get("top_p", getattr(gc, "top_p", None)) if do_sample else None
    eos = sampling_kwargs.get("eos_token_id", getattr(gc, "eos_token_id", None))
    eos_ids = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
    max_new_tokens = sampling_kwargs.get("max_new_tokens_override", max_new_tokens)

    device = inputs.device
    input_ids = inputs
    gen = PromptLookupCandidateGenerator(num_output_tokens=num_output_tokens,
                                         max_matching_ngram_size=max_matching_ngram_size)
    gen.init_look_up_table(input_ids)
    cache = _new_cache(self, input_ids)
    self.first_token_time = 0
    self.generate_time, self.verify_time, self.draft_time = [], [], []
    self.n_matched = self.n_drafted = 0
    self.draft_num, self.accept_num = [], []

    def choose(logits):
        if do_sample:
            probs = torch.softmax(_warp_logits(logits, temperature, top_k, top_p), dim=-1)
            return torch.multinomial(probs, 1).squeeze(-1)
        return torch.argmax(logits, dim=-1)

    _sync(device)
    tic = time.time()
    out = self(input_ids=input_ids, past_key_values=cache, use_cache=True)
    cache = out.past_key_values if out.past_key_values is not None else cache
    nxt = choose(out.logits[0, -1:]).view(1, 1)
    all_ids = torch.cat([input_ids, nxt], dim=1)
    n_past = input_ids.shape[1]
    step = 1
    _sync(device)
    self.first_token_time = time.time() - tic
    e2e_tic = time.time()
    if streamer is not None:
        streamer.put(input_ids.cpu())
        streamer.put(nxt.cpu())
    gen.update_look_up_table(all_ids)
    finished = bool(eos_ids) and int(nxt) in eos_ids
    accept_rate = 0.0
    n_verify = 0

    while step < max_new_tokens and not finished:
        t0 = time.time()
        cand_ids, _ = gen.get_candidates(all_ids)
        cand_len = cand_ids.shape[1] - all_ids.shape[1]
        cand_len = min(cand_len, max_new_tokens - step - 1) if max_new_tokens - step - 1 >= 0 else 0
        cand_len = max(cand_len, 0)
        verify_in = cand_ids[:, all_ids.shape[1] - 1: all_ids.shape[1] + cand_len]   # [last, candidates...]
        if hasattr(cache, "reserve"):
            cache.reserve(cand_len + 2)
        t1 = time.time()
        self.draft_time.append(t1 - t0)
        v = self(input_ids=verify_in, past_key_values=cache, use_cache=True)
        logits = v.logits[0]
        picked = choose(logits)                                  # [cand_len + 1]
        if cand_len > 0:
            cand = verify_in[0, 1:]
            match = (picked[:cand_len] == cand).int().cumprod(dim=0)
            n_match = int(match.sum())
        else:
            n_match = 0
        accepted = picked[: n_match + 1]
        n_past = n_past + n_match + 1
        cache.crop(n_past)
        room = max_new_tokens - step
        accepted = accepted[:room]
        all_ids = torch.cat([all_ids, accepted.view(1, -1)], dim=1)
        step += accepted.shape[0]
        _sync(device)
        t2 = time.time()
        self.verify_time.append(t2 - t1)
        self.generate_time.append(t2 - t0)
        if streamer is not None:
            streamer.put(accepted.view(1, -1).cpu())
        # table and strategy updates
        for k in range(accepted.shape[0], 0, -1):
            gen.update_look_up_table(all_ids[:, : all_ids.shape[1] - k + 1])
        self.n_drafted += cand_len
        self.n_matched += n_match
        self.draft_num.append(cand_len)
        self.accept_num.append(n_match)
        n_verify += 1
        accept_rate = self.n_matched / self.n_drafted if self.n_drafted > 0 else 0.0
        gen.update_candidate_strategy(cand_len, n_match, accept_rate)
        if eos_ids:
            new = accepted.tolist()
            for e in eos_ids:
                if e in new:
                    cut = len(new) - new.index(e) - 1
                    if cut:
                        all_ids = all_ids[:, :-cut]
                        step -= cut
                    finished = True
                    break

    if streamer is not None:
        streamer.end()
    _sync(device)
    self.n_token_generated = step
    self.e2e_time_without_first = time.time() - e2e_tic
    return all_ids
