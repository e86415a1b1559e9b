"""JSON-constrained decoding.

The reference wraps the ``xgrammar`` package in a logits processor
(python/llm/src/ipex_llm/transformers/xgrammar.py:33-47: ``CustomLogitsProcessor`` +
``create_json_logits_processor(tokenizer, vocab_size, schema=None)``).  ``xgrammar`` is used here too when it is
installed; otherwise a built-in incremental JSON prefix checker constrains the candidates: at each step the
highest-scoring tokens are tried in order and the first ``max_candidates`` whose text keeps the output a valid JSON
prefix stay allowed (everything else is masked), and EOS is allowed only once the document is complete.
"""
from __future__ import annotations

from typing import Optional

import torch


class _JsonPrefix:
    """Incremental validity check of a JSON document prefix (RFC 8259 grammar, pushdown over characters)."""

    def __init__(self):
        self.stack = []          # '{' or '['
        self.state = "value"     # value | key_or_end | key | colon | comma_or_end | done
        self.tok = ""            # partial scalar (number / literal)
        self.in_str = False
        self.esc = 0             # >0: escape in progress (1 = after backslash, 2..5 = \uXXXX digits left + 1)
        self.str_is_key = False
        self.ok = True

    def clone(self):
        c = _JsonPrefix()
        c.stack, c.state, c.tok = list(self.stack), self.state, self.tok
        c.in_str, c.esc, c.str_is_key, c.ok = self.in_str, self.esc, self.str_is_key, self.ok
        return c

    @property
    def complete(self):
        return self.ok and not self.stack and not self.in_str and \
            (self.state == "done" or (self.state == "scalar" and self._scalar_done(self.tok)))

    @staticmethod
    def _scalar_prefix(t):
        for lit in ("true", "false", "null"):
            if lit.startswith(t):
                return True
        import re
        return re.fullmatch(r"-?(0|[1-9]\d*)?(\.\d*)?([eE][+-]?\d*)?", t) is not None and t not in ("",)

    @staticmethod
    def _scalar_done(t):
        import re
        return t in ("true", "false", "null") or re.fullmatch(r"-?(0|[1-9]\d*)(\.\d+)?([eE][+-]?\d+)?", t) is not None

    def _after_value(self):
        self.state = "comma_or_end" if self.stack else "done"

    def feed(self, text: str) -> bool:
        for ch in text:
            if not self.ok:
                return False
            self._ch(ch)
        return self.ok

    def _ch(self, ch):
        if self.in_str:
            if self.esc == 1:
                if ch == "u":
                    self.esc = 5
                elif ch in '"\\/bfnrt':
                    self.esc = 0
                else:
                    self.ok = False
            elif self.esc > 1:
                if ch in "0123456789abcdefABCDEF":
                    self.esc -= 1
                    if self.esc == 1:
                        self.esc = 0
                else:
                    self.ok = False
            elif ch == "\\":
                self.esc = 1
            elif ch == '"':
                self.in_str = False
                if self.str_is_key:
                    self.state = "colon"
                else:
                    self._after_value()
            elif ord(ch) < 0x20:
                self.ok = False
            return
        if self.state == "scalar":
            if self._scalar_prefix(self.tok + ch):
                self.tok += ch
                return
            if not self._scalar_done(self.tok):
                self.ok = False
                return
            self.tok = ""
            self._after_value()
        ws = ch in " \t\r\n"
        if ws:
            return
        s = self.state
        if s == "value" or s == "value_or_end":
            if s == "value_or_end" and ch == "]":
                self.stack.pop()
                self._after_value()
            elif ch == "{":
                self.stack.append("{")
                self.state = "key_or_end"
            elif ch == "[":
                self.stack.append("[")
                self.state = "value_or_end"
            elif ch == '"':
                self.in_str, self.str_is_key = True, False
            elif self._scalar_prefix(ch):
                self.tok, self.state = ch, "scalar"
            else:
                self.ok = False
        elif s in ("key_or_end", "key"):
            if ch == '"':
                self.in_str, self.str_is_key = True, True
            elif ch == "}" and s == "key_or_end":
                self.stack.pop()
                self._after_value()
            else:
                self.ok = False
        elif s == "colon":
            if ch == ":":
                self.state = "value"
            else:
                self.ok = False
        elif s == "comma_or_end":
            top = self.stack[-1]
            if ch == ",":
                self.state = "key" if top == "{" else "value"
            elif (ch == "}" and top == "{") or (ch == "]" and top == "["):
                self.stack.pop()
                self._after_value()
            else:
                self.ok = False
        else:   # done
            self.ok = False


class CustomLogitsProcessor:
    """``LogitsProcessor`` protocol: ``__call__(input_ids, scores) -> scores``."""

    def __init__(self, tokenizer, vocab_size: int, schema=None, max_candidates: int = 32, search: int = 512):
        self.tokenizer, self.vocab_size = tokenizer, vocab_size
        self.max_candidates, self.search = max_candidates, search
        self.prompt_len: Optional[int] = None
        self._xg = None
        try:                                               # pragma: no cover - optional dependency
            import xgrammar as xgr
            info = xgr.TokenizerInfo.from_huggingface(tokenizer, vocab_size=vocab_size)
            comp = xgr.GrammarCompiler(info)
            grammar = comp.compile_json_schema(schema) if schema is not None else comp.compile_builtin_json_grammar()
            self._xg = xgr.contrib.hf.LogitsProcessor(grammar)
        except Exception:  # noqa: BLE001
            self._xg = None

    def __call__(self, input_ids: torch.LongTensor, scores: torch.FloatTensor) -> torch.FloatTensor:
        if self._xg is not None:
            return self._xg(input_ids, scores)
        if self.prompt_len is None:
            self.prompt_len = input_ids.shape[1]
        eos = self.tokenizer.eos_token_id
        out = torch.full_like(scores, float("-inf"))
        for b in range(input_ids.shape[0]):
            st = _JsonPrefix()
            st.feed(self.tokenizer.decode(input_ids[b, self.prompt_len:], skip_special_tokens=True))
            order = torch.argsort(scores[b], descending=True)[: self.search].tolist()
            kept = 0
            for t in order:
                if t == eos:
                    if st.complete:
                        out[b, t] = scores[b, t]
                        kept += 1
                    continue
                piece = self.tokenizer.decode([t], skip_special_tokens=True)
                if piece and st.clone().feed(piece):
                    out[b, t] = scores[b, t]
                    kept += 1
                if kept >= self.max_candidates:
                    break
            if kept == 0 and eos is not None:
                out[b, eos] = 0.0
        return out


def create_json_logits_processor(tokenizer, vocab_size: int, schema=None):
    return CustomLogitsProcessor(tokenizer, vocab_size, schema)
