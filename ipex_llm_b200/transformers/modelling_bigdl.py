"""Reference module path ``ipex_llm.transformers.modelling_bigdl`` (python/llm/src/ipex_llm/transformers/
modelling_bigdl.py:29-157): ``BigdlNativeForCausalLM`` and the per-family ``*ForCausalLM`` loaders of converted native
checkpoints (``from_pretrained(path, native=True / False)``)."""
from ..utils.common import invalidInputError


class _BaseAutoModelClass:
    GGML_Model = None

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path, native: bool = True, dtype: str = "int4", *args, **kwargs):
        """``native=True``: a checkpoint written by ``llm_convert`` (low-bit directory) -> the llama-cpp-style
        class of ``ipex_llm.models``; ``native=False``: a Hugging Face checkpoint quantized on load."""
        if native:
            from .. import models
            invalidInputError(cls.GGML_Model is not None, "use a family class such as LlamaForCausalLM")
            return getattr(models, cls.GGML_Model)(pretrained_model_name_or_path, *args, **kwargs)
        from . import AutoModelForCausalLM
        low_bit = {"int4": "sym_int4", "int8": "sym_int8"}.get(dtype, dtype)
        return AutoModelForCausalLM.from_pretrained(pretrained_model_name_or_path, load_in_low_bit=low_bit, **kwargs)


class LlamaForCausalLM(_BaseAutoModelClass):
    GGML_Model = "Llama"


class ChatGLMForCausalLM(_BaseAutoModelClass):
    GGML_Model = "ChatGLM"


class GptneoxForCausalLM(_BaseAutoModelClass):
    GGML_Model = "Gptneox"


class BloomForCausalLM(_BaseAutoModelClass):
    GGML_Model = "Bloom"


class StarcoderForCausalLM(_BaseAutoModelClass):
    GGML_Model = "Starcoder"


class BigdlNativeForCausalLM:
    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path, model_family: str = "llama", dtype: str = "int4",
                        **kwargs):
        fam = {"llama": LlamaForCausalLM, "chatglm": ChatGLMForCausalLM, "gptneox": GptneoxForCausalLM,
               "bloom": BloomForCausalLM, "starcoder": StarcoderForCausalLM}
        invalidInputError(model_family in fam, f"Unknown model family {model_family}; one of {sorted(fam)}")
        return fam[model_family].from_pretrained(pretrained_model_name_or_path, native=True, dtype=dtype, **kwargs)
