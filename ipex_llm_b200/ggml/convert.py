"""Reference module path ``ipex_llm.ggml.convert``: Hugging Face -> ggml fp16 file converters of the legacy native
flow (``_convert_to_ggml``).  This package has no ggml-file runtime; conversion goes straight to its low-bit
checkpoint through ``llm_convert`` / ``ggml.quantize.quantize``."""
from .quantize import quantize


def _convert_to_ggml(model_path: str, outfile_dir: str, model_family: str = "llama", outtype: str = "fp16"):
    return quantize(model_path, outfile_dir, model_family, "q8_0" if outtype == "fp16" else outtype)
