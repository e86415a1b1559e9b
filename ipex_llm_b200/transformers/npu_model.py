"""``ipex_llm.transformers.npu_model``: the reference's Intel-NPU entry point
(python/llm/src/ipex_llm/transformers/npu_model.py:57-770, which compiles per-layer OpenVINO blobs).  A B200 system
has no NPU; scripts written against that module keep working because the same class names load the model through the
CUDA path, and the NPU-only keyword arguments (``max_context_len``, ``max_prompt_len``, ``transpose_value_cache``,
``inter_pp``, ``intra_pp``, ``quantization_group_size``, ``mixed_precision``, ``save_directory``, ``pipeline``,
``compile_full_model`` ...) are accepted and ignored."""
from __future__ import annotations

from . import model as _m

_NPU_ONLY = ("max_context_len", "max_prompt_len", "transpose_value_cache", "inter_pp", "intra_pp",
             "quantization_group_size", "save_directory", "pipeline", "compile_full_model", "fuse_layers",
             "max_output_len", "convert_model", "compile_blob", "keep_ir", "imatrix_path")


def _strip(kwargs):
    for k in _NPU_ONLY:
        kwargs.pop(k, None)
    low_bit = kwargs.get("load_in_low_bit")
    if low_bit in ("sym_int4_rtn", "asym_int4_rtn", "sym_int8_rtn"):
        kwargs["load_in_low_bit"] = low_bit.replace("_rtn", "")
    kwargs.setdefault("optimize_model", True)
    return kwargs


class _NPUMixin:
    @classmethod
    def from_pretrained(cls, *args, **kwargs):
        return super().from_pretrained(*args, **_strip(kwargs))

    @classmethod
    def load_low_bit(cls, *args, **kwargs):
        return super().load_low_bit(*args, **_strip(kwargs))


class AutoModelForCausalLM(_NPUMixin, _m.AutoModelForCausalLM):
    pass


class AutoModel(_NPUMixin, _m.AutoModel):
    pass


class AutoModelForSpeechSeq2Seq(_NPUMixin, _m.AutoModelForSpeechSeq2Seq):
    pass


class AutoModelForSeq2SeqLM(_NPUMixin, _m.AutoModelForSeq2SeqLM):
    pass
