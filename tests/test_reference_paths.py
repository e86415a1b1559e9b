"""Module paths of the reference library resolve (through both the ``ipex_llm`` and ``bigdl.llm`` aliases) to this
package's implementations."""
import importlib

import pytest
import torch

PATHS = [
    "serving.fastapi.api_server", "serving.fastapi.model_worker",
    "serving.fastapi.openai_protocol", "serving.fastapi.tgi_protocol",
    "vllm.xpu.engine.engine", "vllm.cpu.engine.engine",
    "ggml.model.llama", "ggml.model.gptneox", "ggml.model.bloom",
    "ggml.model.starcoder", "ggml.model.generation", "utils.common.lazyimport",
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
    "transformers.models.sd", "utils.glibc_checker", "serving.fastchat.bigdl_llm_model", "serving.fastchat.model_worker",
    "serving.fastchat.vllm_worker", "serving.fastchat.tgi_api_server", "serving.fastchat.tgi_api_protocol",
    "llamaindex.llms.bigdlllm", "langchain.llms.bigdlllm", "langchain.llms.transformersllm",
    "langchain.llms.transformerspipelinellm", "langchain.embeddings.bigdlllm",
    "langchain.embeddings.transformersembeddings", "langchain.vllm.vllm", "vllm.xpu.engine", "vllm.cpu.engine",
    "vllm.xpu.entrypoints.openai.api_server", "vllm.cpu.entrypoints.openai.api_server",
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
    from ipex_llm.utils.lazy_load_torch import DisableTorchAllocTensor
    from ipex_llm.ops.linear import LowBitLinear as impl
    assert LowBitLinear is impl and ggml_tensor_qtype["sym_int4"] == 2
    packed = ggml_convert_qtype(torch.randn(4, 64), ggml_tensor_qtype["sym_int8"])
    assert packed.dtype == torch.uint8
    assert issubclass(FP4Params, torch.nn.Parameter)
    with pytest.raises(RuntimeError):
        invalidInputError(False, "boom")
    with DisableTorchAllocTensor():
        lin = torch.nn.Linear(8, 8)
    assert lin.weight.device.type == "meta"
    import bigdl.llm.transformers.low_bit_linear as legacy
    assert legacy.LowBitLinear is impl
    # everything the reference's ``ipex_llm.transformers`` package exports (transformers/__init__.py:17-32)
    import ipex_llm.transformers as pkg
    for name in ("ggml_convert_low_bit", "get_enable_ipex", "convert_model_hybrid", "AutoModelForCausalLM", "AutoModel",
                 "AutoModelForSeq2SeqLM", "AutoModelForSpeechSeq2Seq", "AutoModelForQuestionAnswering",
                 "AutoModelForSequenceClassification", "AutoModelForMaskedLM", "AutoModelForNextSentencePrediction",
                 "AutoModelForMultipleChoice", "AutoModelForTokenClassification", "Qwen2VLForConditionalGeneration",
                 "BigdlNativeForCausalLM", "LlamaForCausalLM", "ChatGLMForCausalLM", "GptneoxForCausalLM",
                 "BloomForCausalLM", "StarcoderForCausalLM", "init_pipeline_parallel", "PPModelWorker"):
        assert hasattr(pkg, name), name
    from ipex_llm.transformers.gguf import load_gguf_model  # noqa: F401
    from ipex_llm.utils.common import LazyImport
    from ipex_llm.vllm.xpu.engine import run_mp_engine  # noqa: F401
    lazy_fn = LazyImport("ipex_llm.transformers.low_bit_linear.ggml_convert_qtype")
    assert lazy_fn(torch.randn(2, 64), ggml_tensor_qtype["sym_int8"]).dtype == torch.uint8
    assert LazyImport("ipex_llm.ggml.quantize").ggml_tensor_qtype["sym_int4"] == 2


def test_torch_library_ops_have_fake_kernels_and_match_eager():
    """``torch.ops.ipex_llm.*`` exist with the reference's op names, trace with fake tensors (meta device) and
    compute the same numbers as the module path on CPU."""
    import torch
    import ipex_llm.transformers.xpu_ops  # noqa: F401  (registers the ops)
    from ipex_llm_b200.ops.linear import LowBitLinear
    from ipex_llm_b200.quant import qtypes as qt
    from ipex_llm_b200.quant.params import FP4Params
    torch.manual_seed(0)
    lin = torch.nn.Linear(128, 48, bias=False)
    w = FP4Params(lin.weight.data, quantized=False, qtype=qt.SYM_INT8).quantize("cpu")
    x = torch.randn(3, 128)
    y = torch.ops.ipex_llm.forward_new(x, w.data, qt.SYM_INT8, 48)
    ref = torch.nn.functional.linear(x, w.dequantize(torch.float32))
    assert torch.allclose(y, ref, atol=1e-4)
    g = torch.randn(3, 48)
    n = torch.ops.ipex_llm.rms_norm(torch.ones(48), g, 1e-6)
    assert torch.allclose(n, g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + 1e-6), atol=1e-5)
    # fake kernels: shapes without data
    with torch.device("meta"):
        xm, wm = torch.empty(5, 128), torch.empty(w.data.numel(), dtype=torch.uint8)
    ym = torch.ops.ipex_llm.forward_new(xm, wm, qt.SYM_INT8, 48)
    assert ym.shape == (5, 48) and ym.device.type == "meta"
    q = torch.empty(2, 4, 1, 64, device="meta")
    kv = torch.empty(2, 4, 9, 64, device="meta")
    assert torch.ops.ipex_llm.sdp(q, kv, kv).shape == (2, 4, 1, 64)
    # ... and through torch.compile's tracer (fake tensors), eager backend
    def f(a):
        return torch.ops.ipex_llm.rms_norm(torch.ones(48), a, 1e-6) * 2
    out = torch.compile(f, backend="eager")(g)
    assert torch.allclose(out, n * 2, atol=1e-5)


def test_lazy_tensor_loader(tmp_path):
    """``ipex_llm.utils.lazy_load_torch``: tensors of a zip checkpoint are file-backed until loaded, a stacked dtype
    conversion runs at load time, and inside ``LazyLoadTensors`` a plain ``torch.load`` is memory-mapped."""
    import torch
    from ipex_llm.utils.lazy_load_torch import LazyLoadTensors, LazyTensor, lazyload
    sd = {"a.weight": torch.randn(64, 32), "b": {"bias": torch.arange(8, dtype=torch.int32)}, "step": 7}
    path = str(tmp_path / "ckpt.bin")
    torch.save(sd, path)
    lazy = lazyload(path)
    assert isinstance(lazy["a.weight"], LazyTensor) and lazy["a.weight"].shape == [64, 32] and lazy["step"] == 7
    assert torch.equal(lazy["a.weight"].load(), sd["a.weight"])
    half = lazy["a.weight"].to(torch.float16)
    assert half.data_type == torch.float16 and half.load().dtype == torch.float16
    assert torch.equal(lazy["b"]["bias"].load(), sd["b"]["bias"])
    orig, seen = torch.load, []

    def recorder(f, *a, **kw):
        seen.append(kw.get("mmap"))
        return orig(f, *a, **kw)
    torch.load = recorder
    try:
        with LazyLoadTensors():
            mapped = torch.load(path, weights_only=True)
            assert torch.load is not recorder
        assert torch.load is recorder
    finally:
        torch.load = orig
    assert seen == [True]                                        # the archive was mapped, not read
    assert torch.equal(mapped["a.weight"], sd["a.weight"])


def test_glibc_checker():
    from ipex_llm.utils.glibc_checker import GlibcChecker, check_glibc_version
    check_glibc_version()                                   # the build machine satisfies its own requirement
    assert GlibcChecker.get_glibc_version()[0].isdigit()
    with pytest.raises(RuntimeError):
        GlibcChecker("999.0").check_requirements()
