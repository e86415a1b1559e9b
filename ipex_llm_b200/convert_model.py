"""``llm_convert`` / ``llm-convert`` command: turn a Hugging Face checkpoint (plain or GPTQ) into a low-bit checkpoint.

Same call and flags as python/llm/src/ipex_llm/convert_model.py:30-140 of the reference.  The reference emits a
single GGML ``.bin`` for its llama.cpp-derived CPU runtimes; this package has one runtime for every architecture
(the transformers-style API), so the output is a ``save_low_bit`` directory
(``bigdl_llm_<family>_<outtype>/``) that ``AutoModelForCausalLM.load_low_bit`` opens without touching the original
weights again.  The returned string is the path of that directory.
"""
from __future__ import annotations

import argparse
import os

from .utils.common import invalidInputError

_OUTTYPE = {"int4": "sym_int4", "int8": "sym_int8", "int5": "sym_int5", "nf4": "nf4", "fp4": "fp4", "fp8": "fp8_e4m3",
            "sym_int4": "sym_int4", "asym_int4": "asym_int4", "sym_int8": "sym_int8", "fp8_e4m3": "fp8_e4m3",
            "fp8_e5m2": "fp8_e5m2", "fp6": "fp6", "nf3": "nf3", "sym_int5": "sym_int5", "asym_int5": "asym_int5"}
_FAMILIES = ("llama", "bloom", "gptneox", "starcoder", "chatglm", "mistral", "mixtral", "qwen2", "qwen", "gemma",
             "phi3", "baichuan", "internlm", "falcon", "mpt", "gpt2")


def _special_kwarg_check(kwargs, check_args):
    used = {}
    for arg in list(kwargs.keys()):
        if arg in check_args:
            used[arg] = kwargs[arg]
        else:
            invalidInputError(False, f"Invalid parameter: {arg}; valid ones here: {check_args}")
    return True, used


def llm_convert(model, outfile, model_family, outtype="int4", model_format="pth", **kwargs):
    """Quantize the checkpoint in directory ``model`` and save it under directory ``outfile``.

    ``model_format='pth'``: a Hugging Face checkpoint.  ``model_format='gptq'``: a GPTQ checkpoint (its int4 codes
    are re-packed without a round trip through floats where the formats allow it).  Returns the output path.
    """
    invalidInputError(model_family in _FAMILIES, f"Unsupported model family {model_family}; one of {_FAMILIES}")
    invalidInputError(outtype.lower() in _OUTTYPE, f"Unsupported outtype {outtype}; one of {sorted(_OUTTYPE)}")
    invalidInputError(os.path.isdir(model), f"The input path {model} is not a directory")
    os.makedirs(outfile, exist_ok=True)
    invalidInputError(os.path.isdir(outfile), f"The output_path {outfile} is not a directory")
    low_bit = _OUTTYPE[outtype.lower()]
    from .transformers import AutoModel, AutoModelForCausalLM
    if model_format == "pth":
        _special_kwarg_check(kwargs, ["tmp_path"])
    elif model_format == "gptq":
        invalidInputError(low_bit in ("sym_int4", "asym_int4"),
                          "Convert GPTQ models should always specify `--outtype int4` in the command line.")
        _special_kwarg_check(kwargs, ["tokenizer_path"])
        low_bit = "asym_int4"
    else:
        invalidInputError(False, f"Unsupported input model_type: {model_format}")
    cls = AutoModel if model_family == "chatglm" else AutoModelForCausalLM
    m = cls.from_pretrained(model, load_in_low_bit=low_bit, trust_remote_code=True)
    out = os.path.join(outfile, f"bigdl_llm_{model_family}_{outtype.lower()}" +
                       ("_from_gptq" if model_format == "gptq" else ""))
    m.save_low_bit(out)
    tok_src = kwargs.get("tokenizer_path") or model
    try:
        from transformers import AutoTokenizer
        AutoTokenizer.from_pretrained(tok_src, trust_remote_code=True).save_pretrained(out)
    except Exception:  # noqa: BLE001 - a checkpoint without tokenizer files is still a valid model checkpoint
        pass
    return out


def main(argv=None):
    p = argparse.ArgumentParser(description="Model Convert Parameters")
    p.add_argument("model", type=str, help="a path to a *directory* containing model weights")
    p.add_argument("-o", "--outfile", type=str, required=True, help="save path (directory) of the quantized model")
    p.add_argument("-x", "--model-family", type=str, required=True, help="model family of the input model")
    p.add_argument("-f", "--model-format", type=str, required=True, help="`pth` or `gptq`")
    p.add_argument("-t", "--outtype", type=str, default="int4", help="quantized precision")
    p.add_argument("-p", "--tmp-path", type=str, default=None, help="(pth) scratch directory; unused, kept for "
                                                                      "command-line compatibility")
    p.add_argument("-k", "--tokenizer-path", type=str, default=None, help="(gptq) where tokenizer.model lives")
    a = p.parse_args(argv)
    params = {k: v for k, v in vars(a).items() if v is not None}
    kw = {}
    if a.model_format == "pth" and a.tmp_path:
        kw["tmp_path"] = a.tmp_path
    if a.model_format == "gptq" and a.tokenizer_path:
        kw["tokenizer_path"] = a.tokenizer_path
    out = llm_convert(params["model"], params["outfile"], params["model_family"], params["outtype"],
                      params["model_format"], **kw)
    print(out)
    return out


if __name__ == "__main__":
    main()
