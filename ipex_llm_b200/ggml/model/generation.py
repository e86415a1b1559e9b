"""Hugging Face flavoured token API of the llama-cpp-style classes (reference:
python/llm/src/ipex_llm/ggml/model/generation/utils.py:28-180): ``tokenize`` / ``decode`` / ``batch_decode`` and a
``generate`` that takes one prompt or a batch of prompts as token lists (or a tensor) and returns, per prompt, the
list of NEW token ids (at most ``max_new_tokens``)."""
from __future__ import annotations

from typing import List, Optional, Sequence, Union


class GenerationMixin:
    def decode(self, tokens: List[int]) -> str:
        return self.detokenize(list(tokens)).decode("utf-8", errors="ignore")

    def batch_decode(self, tokens: Union[List[int], List[List[int]]]) -> Union[str, List[str]]:
        batched = len(tokens) > 0 and isinstance(tokens[0], Sequence)
        texts = [self.decode(t) for t in (tokens if batched else [tokens])]
        return texts if batched else texts[0]

    def generate(self, inputs=None, max_new_tokens: int = 128, top_k: int = 40, top_p: float = 0.95,
                 temperature: float = 0.80, repetition_penalty: float = 1.1, stop: Optional[Sequence[str]] = (),
                 **kwargs) -> Optional[List[List[int]]]:
        if hasattr(inputs, "tolist"):
            inputs = inputs.tolist()
        if not inputs:
            return None
        if not isinstance(inputs[0], Sequence):
            inputs = [inputs]
        # the llama-cpp spelling of the same knobs (``tokens``, ``temp``, ``repeat_penalty``, ``max_tokens``)
        temperature = kwargs.pop("temp", temperature)
        repetition_penalty = kwargs.pop("repeat_penalty", repetition_penalty)
        max_new_tokens = kwargs.pop("max_tokens", max_new_tokens)
        return [self._generate_ids(list(t), max_new_tokens, temperature, top_p, top_k, repetition_penalty)
                for t in inputs]
