"""Reference module path ``ipex_llm.gptq.convert.convert_gptq_to_ggml``: GPTQ int4 checkpoints are re-packed
bit-exactly into ``asym_int4`` blocks by the loader (``transformers/convert.py::convert_gptq``); this entry point
runs that path and saves the result."""
from ...convert_model import llm_convert


def convert_gptq2ggml(model_path: str, output_path: str, tokenizer_path: str = None):
    return llm_convert(model_path, output_path, "llama", outtype="int4", model_format="gptq",
                       **({"tokenizer_path": tokenizer_path} if tokenizer_path else {}))
