"""Reference module path ``ipex_llm.utils.convert_util`` (python/llm/src/ipex_llm/utils/convert_util.py: the
Hugging Face -> ggml fp16 file writers of the legacy native flow, ``_convert_llama`` / ``_convert_gptneox`` /
``_convert_bloom`` / ``_convert_starcoder`` / ``_convert_chatglm``).  This package has no ggml-file runtime: every
converter writes its low-bit checkpoint through ``ggml.quantize.quantize`` instead."""
from ..ggml.quantize import quantize


def _make(model_family):
    def convert(model_path, outfile_dir, outtype="q8_0"):
        return quantize(model_path, outfile_dir, model_family, outtype)
    convert.__name__ = f"_convert_{model_family}"
    return convert


_convert_llama = _make("llama")
_convert_gptneox = _make("gptneox")
_convert_bloom = _make("bloom")
_convert_starcoder = _make("starcoder")
_convert_chatglm = _make("chatglm")
