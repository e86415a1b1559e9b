"""``ipex_llm.ggml.quantize``: the qtype table under its reference import path, and ``quantize``.

Reference: python/llm/src/ipex_llm/ggml/quantize.py:28-61 (``ggml_tensor_qtype``) and :87-142 (``quantize`` shells
out to a prebuilt ``quantize-<family>`` binary that rewrites a ggml fp16 file as a low-bit ggml file).  No such
family binaries exist here; ``quantize`` does the same job in process: it reads a Hugging Face checkpoint directory
(or a ``.gguf`` file), quantizes every linear with the host library and writes a low-bit checkpoint that
``load_low_bit`` (or ``llm_convert``'s consumers) read back.  File to file, ``quantize_gguf`` runs the package's native
``ipex-quantize`` executable (``native/tools/quantize_main.cpp``), which rewrites a GGUF file with k-quant tensors.
"""
from __future__ import annotations

import os

from ..quant.qtypes import ggml_tensor_qtype  # noqa: F401  (re-export under the reference's module path)
from ..utils.common import invalidInputError

# dtype spellings of the reference's CLI -> low_bit names
_quantize_type = {"q4_0": "sym_int4", "q4_1": "asym_int4", "q5_0": "sym_int5", "q5_1": "asym_int5", "q8_0": "sym_int8",
                  "int4": "sym_int4", "int5": "sym_int5", "int8": "sym_int8"}


def quantize_gguf(input_path: str, output_path: str, dtype: str = "q4_k", keep=(), output_type: str = None) -> str:
    """``input_path`` (f32 / f16 / bf16 GGUF) -> ``output_path`` with every large matrix packed to ``dtype`` (q2_k, q4_k,
    q5_k, q6_k) by the native executable.  ``keep``: name substrings of tensors to leave untouched."""
    import subprocess
    from ..native.build import build_tools
    invalidInputError(os.path.isfile(input_path), f"The file {input_path} is not found")
    cmd = [build_tools(), input_path, output_path, dtype.lower()]
    for k in keep:
        cmd += ["--keep", k]
    if output_type:
        cmd += ["--output-type", output_type.lower()]
    res = subprocess.run(cmd, capture_output=True, text=True)
    invalidInputError(res.returncode == 0, f"ipex-quantize failed: {res.stderr.strip() or res.stdout.strip()}")
    return output_path


def quantize(input_path: str, output_path: str = None, model_family: str = "llama", dtype: str = "q4_0") -> str:
    """Quantize ``input_path`` (checkpoint directory or ``.gguf`` file) to ``dtype`` and save it under
    ``output_path`` (default: next to the input).  Returns the output directory."""
    invalidInputError(model_family in ("llama", "bloom", "gptneox", "starcoder", "chatglm"),
                      f"{model_family} is not in the list: llama / bloom / gptneox / starcoder / chatglm")
    low_bit = _quantize_type.get(dtype.lower(), dtype.lower())
    invalidInputError(low_bit in ggml_tensor_qtype, f"{dtype} is not a supported quantization type")
    invalidInputError(os.path.exists(input_path), f"The file {input_path} is not found")
    from ..transformers import AutoModelForCausalLM
    if output_path is None:
        base = os.path.splitext(os.path.basename(input_path.rstrip("/")))[0]
        output_path = os.path.join(os.path.dirname(os.path.abspath(input_path.rstrip("/"))),
                                   f"bigdl_llm_{model_family}_{dtype.lower()}_{base}")
    if os.path.isfile(input_path) and input_path.endswith(".gguf") and output_path.endswith(".gguf") \
            and low_bit in ("q2_k", "q4_k", "q5_k", "q6_k"):
        return quantize_gguf(input_path, output_path, low_bit)
    if os.path.isfile(input_path) and input_path.endswith(".gguf"):
        model, _ = AutoModelForCausalLM.from_gguf(input_path, low_bit=low_bit)
    else:
        model = AutoModelForCausalLM.from_pretrained(input_path, load_in_low_bit=low_bit, trust_remote_code=True)
    model.save_low_bit(output_path)
    return output_path
