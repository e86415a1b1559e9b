"""Streamers for batched generation.

``BatchTextIteratorStreamer`` mirrors python/llm/src/ipex_llm/transformers/streamer.py:26-114 of the reference: the
``generate`` loop calls ``put`` with the new token of every sequence, and a consumer iterates over lists of text
pieces (one per sequence, ``""`` when a sequence produced nothing printable in that step).  Detokenization is
incremental per sequence: text is released up to the last position that cannot change any more (a complete word, or a
complete UTF-8 character), as HF's ``TextStreamer`` does for one sequence.
"""
from __future__ import annotations

from queue import Queue
from typing import List, Optional


class BatchTextIteratorStreamer:
    def __init__(self, batch_size: int, tokenizer, skip_prompt: bool = False, timeout: Optional[float] = None,
                 **decode_kwargs):
        self.batch_size = batch_size
        self.tokenizer = tokenizer
        self.skip_prompt = skip_prompt
        self.decode_kwargs = decode_kwargs
        self.timeout = timeout
        self.text_queue: Queue = Queue()
        self.stop_signal = None
        self.token_cache: List[List[int]] = [[] for _ in range(batch_size)]
        self.print_len = [0] * batch_size
        self.next_tokens_are_prompt = True
        self.generated_tokens = [0] * batch_size

    # -- producer side (called by generate) -------------------------------------------------------------
    def put(self, value):
        if hasattr(value, "tolist"):
            value = value.tolist()
        if value and not isinstance(value[0], list):
            value = [[v] for v in value] if len(value) == self.batch_size else [value]
        if len(value) != self.batch_size:
            raise ValueError(f"BatchTextIteratorStreamer was built for batch {self.batch_size}, got {len(value)}")
        if self.skip_prompt and self.next_tokens_are_prompt:
            self.next_tokens_are_prompt = False
            return
        self.next_tokens_are_prompt = False
        pieces = []
        for i, toks in enumerate(value):
            self.token_cache[i].extend(toks)
            self.generated_tokens[i] += len(toks)
            pieces.append(self._release(i, final=False))
        self.on_finalized_text(pieces)

    def _release(self, i: int, final: bool) -> str:
        text = self.tokenizer.decode(self.token_cache[i], **self.decode_kwargs)
        if final:
            out = text[self.print_len[i]:]
            self.token_cache[i] = []
            self.print_len[i] = 0
            return out
        if text.endswith("\n"):
            out = text[self.print_len[i]:]
            self.token_cache[i] = []
            self.print_len[i] = 0
            return out
        if len(text) > 0 and _is_cjk(ord(text[-1])):
            out = text[self.print_len[i]:]
            self.print_len[i] += len(out)
            return out
        if text.endswith("�"):          # incomplete multi-byte character: wait for the rest
            return ""
        cut = text.rfind(" ") + 1
        out = text[self.print_len[i]:cut] if cut > self.print_len[i] else ""
        self.print_len[i] += len(out)
        return out

    def end(self):
        pieces = [self._release(i, final=True) for i in range(self.batch_size)]
        self.next_tokens_are_prompt = True
        self.on_finalized_text(pieces, stream_end=True)

    def on_finalized_text(self, texts: List[str], stream_end: bool = False):
        if any(texts) or stream_end:
            self.text_queue.put(texts, timeout=self.timeout)
        if stream_end:
            self.text_queue.put(self.stop_signal, timeout=self.timeout)

    # -- consumer side ------------------------------------------------------------------------------------
    def __iter__(self):
        return self

    def __next__(self):
        value = self.text_queue.get(timeout=self.timeout)
        if value is self.stop_signal:
            raise StopIteration()
        return value


def _is_cjk(cp: int) -> bool:
    return (0x4E00 <= cp <= 0x9FFF) or (0x3400 <= cp <= 0x4DBF) or (0x20000 <= cp <= 0x2A6DF) or \
        (0x2A700 <= cp <= 0x2B73F) or (0x2B740 <= cp <= 0x2B81F) or (0x2B820 <= cp <= 0x2CEAF) or \
        (0xF900 <= cp <= 0xFAFF) or (0x2F800 <= cp <= 0x2FA1F)
