"""Phi-3 / Phi-3.5 with LongRoPE: the switch from the short to the long rotary factors during generation.

LongRoPE models rotate with ``short_factor`` while the sequence fits ``original_max_position_embeddings`` and with
``long_factor`` beyond it, so the keys cached before the switch are rotated wrongly for everything after it.  The
reference decides the factor set per forward from the KV length (python/llm/src/ipex_llm/transformers/models/phi3.py:
62-86); transformers drops the cache at the switch but, in the releases that slice the step's input before the hook
runs, then feeds only the newest token, so the history is lost.  Here the hook empties the cache in place and asks for
the whole sequence once: one slower step, after which every cached key carries the long factors.
"""
from __future__ import annotations

from types import MethodType


def _switch_point(config):
    limit = getattr(config, "original_max_position_embeddings", None)
    rope = getattr(config, "rope_parameters", None) or getattr(config, "rope_scaling", None) or {}
    if isinstance(rope, dict):
        if rope.get("rope_type", rope.get("type")) not in ("longrope", "su", "yarn"):
            return None
        limit = limit or rope.get("original_max_position_embeddings")
    return int(limit) if limit else None


def prepare_inputs_for_generation(self, input_ids, past_key_values=None, **kwargs):
    from transformers.generation.utils import GenerationMixin
    limit = _switch_point(self.config)
    if past_key_values is not None and limit and input_ids.shape[1] >= limit + 1:
        held = past_key_values.get_seq_length()
        if 0 < held <= limit:
            past_key_values.crop(0)                 # same cache object: the generation loop keeps using it
            kwargs["next_sequence_length"] = None   # the step takes the whole sequence
    return GenerationMixin.prepare_inputs_for_generation(self, input_ids, past_key_values=past_key_values, **kwargs)


def install(model):
    """Family post-hook: bind the generation hook on the causal-LM wrapper when the model uses LongRoPE."""
    if hasattr(model, "prepare_inputs_for_generation") and _switch_point(getattr(model, "config", None)):
        model.prepare_inputs_for_generation = MethodType(prepare_inputs_for_generation, model)
    return model
