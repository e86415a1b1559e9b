"""One ``generate`` dispatcher.

The reference replaces ``GenerationMixin.generate`` three times at import and chains the saved originals
(lookup -> speculative -> pipeline-parallel -> HF; python/llm/src/ipex_llm/transformers/lookup.py:40-136,
speculative.py:65-138, pipeline_parallel.py:47-296).  Here one function, bound per converted model, picks the
strategy:

  pipeline-parallel model          -> ``pipeline_parallel_generate``
  ``lookahead=`` given / perf mode -> ``lookup_generate``
  model has a ``draft_model``      -> ``speculative_generate``
  CUDA model of a supported family -> the CUDA-graph decode engine
  otherwise                        -> Hugging Face ``generate`` (with the package's forwards and caches)
"""
from __future__ import annotations

import torch

from .. import config as cfg


def _engine_ok(model, inputs, kwargs) -> bool:
    if not cfg.use_native_engine():
        return False
    if inputs is None or not isinstance(inputs, torch.Tensor) or not inputs.is_cuda:
        return False
    from ..engine import supports
    return supports(model, kwargs)


@torch.no_grad()
def ipex_generate(self, inputs=None, generation_config=None, logits_processor=None, stopping_criteria=None,
                  prefix_allowed_tokens_fn=None, synced_gpus=None, assistant_model=None, streamer=None, **kwargs):
    if inputs is None and "input_ids" in kwargs:
        inputs = kwargs.pop("input_ids")
    if getattr(self, "pipeline_parallel_stages", 1) > 1:
        from ..parallel.pp import pipeline_parallel_generate
        return pipeline_parallel_generate(self, inputs=inputs, streamer=streamer, generation_config=generation_config,
                                          **kwargs)
    lookahead = kwargs.pop("lookahead", None)
    perf_mode = cfg.performance_mode()
    if lookahead is None and perf_mode and inputs is not None and inputs.shape[0] == 1 and inputs.shape[1] >= 100 \
            and getattr(self, "draft_model", None) is None:
        lookahead = 2
    if lookahead:
        from .lookup import lookup_generate
        kwargs.pop("max_matching_ngram_size", None)
        return lookup_generate(self, inputs=inputs, lookahead=lookahead, generation_config=generation_config,
                               streamer=streamer, **kwargs)
    if getattr(self, "draft_model", None) is not None:
        from .speculative import speculative_generate
        return speculative_generate(self, inputs=inputs, draft_model=self.draft_model,
                                    generation_config=generation_config, streamer=streamer, **kwargs)
    if logits_processor is None and stopping_criteria is None and prefix_allowed_tokens_fn is None \
            and assistant_model is None and _engine_ok(self, inputs, kwargs):
        from ..engine import engine_generate
        return engine_generate(self, inputs, generation_config=generation_config, streamer=streamer, **kwargs)
    # only what the caller actually gave: some generate() overrides (Whisper) test for the presence of a keyword
    optional = dict(generation_config=generation_config, logits_processor=logits_processor,
                    stopping_criteria=stopping_criteria, prefix_allowed_tokens_fn=prefix_allowed_tokens_fn,
                    synced_gpus=synced_gpus, assistant_model=assistant_model, streamer=streamer)
    kwargs.update({k: v for k, v in optional.items() if v is not None})
    if inputs is not None:
        kwargs["inputs"] = inputs
    return self._hf_generate(**kwargs)
