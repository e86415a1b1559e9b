"""Module paths of the reference library resolve (through both the ``ipex_llm`` and ``bigdl.llm`` aliases) to this
package's implementations."""
import importlib

import pytest
import torch

PATHS = [
    "transformers.low_bit_linear", "transformers.embedding", "transformers.kv", "transformers.utils",
    "transformers.convert", "transformers.models.utils", "transformers.models.common", "utils.common",
    "utils.common.log4Error", "transformers.modelling_bigdl", "transformers.training_patch", "transformers.qlora",
    "transformers.lookup", "transformers.speculative", "transformers.pipeline_parallel", "transformers.xpu_ops",
    "transformers.bmm", "transformers.lisa", "transformers.relora", "transformers.gguf.api", "transformers.awq.awq",
    "optimize", "llm_patching", "convert_model", "models", "serving.fastapi", "serving.fastchat.ipex_llm_worker",
    "vllm.xpu.model_convert", "vllm.cpu.model_convert", "langchain.llms", "langchain.embeddings", "llamaindex.llms",
    "utils.ipex_importer", "utils.lazy_load_torch", "transformers.npu_model", "transformers.patches",
    "transformers.streamer", "transformers.loader", "transformers.xgrammar", "ggml.quantize", "ggml.convert_model",
    "ggml.convert", "gptq.convert.convert_gptq_to_ggml", "transformers.convert_ipex",
]


@pytest.mark.parametrize("path", PATHS)
def test_reference_module_path(path):
    importlib.import_module("ipex_llm." + path)


def test_names_behind_the_paths():
    from ipex_llm.transformers.low_bit_linear import FP4Params, LowBitLinear, ggml_convert_qtype, ggml_tensor_qtype
    from ipex_llm.transformers.kv import DynamicCompressCache, DynamicFp8Cache, DynamicNormalCache  # noqa: F401
    from ipex_llm.transformers.embedding import CPUEmbedding, DiskEmbedding, LowBitEmbedding  # noqa: F401
    from ipex_llm.transformers.models.utils import should_use_compresskv, use_quantize_kv_cache  # noqa: F401
    from ipex_llm.transformers.models.common import merge_qkv_base, rms_norm_forward  # noqa: F401
    from ipex_llm.utils.common.log4Error import invalidInputError
    from ipex_llm.utils.lazy_load_torch import LazyLoadTensors
    from ipex_llm.ops.linear import LowBitLinear as impl
    assert LowBitLinear is impl and ggml_tensor_qtype["sym_int4"] == 2
    packed = ggml_convert_qtype(torch.randn(4, 64), ggml_tensor_qtype["sym_int8"])
    assert packed.dtype == torch.uint8
    assert issubclass(FP4Params, torch.nn.Parameter)
    with pytest.raises(RuntimeError):
        invalidInputError(False, "boom")
    with LazyLoadTensors():
        lin = torch.nn.Linear(8, 8)
    assert lin.weight.device.type == "meta"
    import bigdl.llm.transformers.low_bit_linear as legacy
    assert legacy.LowBitLinear is impl
