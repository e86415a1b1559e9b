"""Hugging Face ``transformers``-style API (reference: python/llm/src/ipex_llm/transformers/__init__.py)."""
from .convert import convert_model_hybrid, get_enable_ipex, ggml_convert_low_bit  # noqa: F401
from .model import (AutoModel, AutoModelForCausalLM, AutoModelForMaskedLM, AutoModelForMultipleChoice,  # noqa: F401
                    AutoModelForNextSentencePrediction, AutoModelForQuestionAnswering,
                    AutoModelForSeq2SeqLM, AutoModelForSequenceClassification, AutoModelForSpeechSeq2Seq,
                    AutoModelForTokenClassification, AutoModelForVision2Seq,
                    Qwen2VLModelForConditionalGeneration)
from .modelling_bigdl import (BigdlNativeForCausalLM, BloomForCausalLM, ChatGLMForCausalLM,  # noqa: F401
                              GptneoxForCausalLM, LlamaForCausalLM, StarcoderForCausalLM)

Qwen2VLForConditionalGeneration = Qwen2VLModelForConditionalGeneration   # the name the reference package exports


def __getattr__(name):
    if name in ("init_pipeline_parallel", "PPModelWorker", "pipeline_parallel"):
        import importlib
        _pp = importlib.import_module(__name__ + ".pipeline_parallel")
        # the submodule and the function share the name ``pipeline_parallel``: attribute access gives the
        # submodule once it is imported, as in the reference package
        return _pp if name == "pipeline_parallel" else getattr(_pp, name)
    raise AttributeError(name)
