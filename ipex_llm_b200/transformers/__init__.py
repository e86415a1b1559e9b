"""Hugging Face ``transformers``-style API (reference: python/llm/src/ipex_llm/transformers/__init__.py)."""
from .convert import ggml_convert_low_bit  # noqa: F401
from .model import (AutoModel, AutoModelForCausalLM, AutoModelForMaskedLM, AutoModelForMultipleChoice,  # noqa: F401
                    AutoModelForNextSentencePrediction, AutoModelForQuestionAnswering,
                    AutoModelForSeq2SeqLM, AutoModelForSequenceClassification, AutoModelForSpeechSeq2Seq,
                    AutoModelForTokenClassification, AutoModelForVision2Seq,
                    Qwen2VLModelForConditionalGeneration)


def __getattr__(name):
    if name in ("init_pipeline_parallel", "PPModelWorker", "pipeline_parallel"):
        from . import pipeline_parallel as _pp
        return getattr(_pp, name)
    raise AttributeError(name)
