"""Integration shims on CPU: LangChain / LlamaIndex wrappers, NPU-named entry point, JSON-constrained decoding,
llm_convert + CLI, BenchmarkWrapper."""
import json
import os

import pytest
import torch


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import LlamaConfig, LlamaForCausalLM, PreTrainedTokenizerFast
    d = tmp_path_factory.mktemp("tiny_ckpt")
    words = ["<pad>", "<s>", "</s>", "<unk>", "{", "}", "[", "]", ":", ",", '"a"', '"b"', "1", "2", "true", "null"] + \
        [f"w{i}" for i in range(48)]
    tk = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tk.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok = PreTrainedTokenizerFast(tokenizer_object=tk, pad_token="<pad>", bos_token="<s>", eos_token="</s>",
                                  unk_token="<unk>")
    cfg = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=64, max_position_embeddings=256, tie_word_embeddings=False,
                      eos_token_id=2, pad_token_id=0, bos_token_id=1)
    torch.manual_seed(0)
    LlamaForCausalLM(cfg).save_pretrained(d)
    tok.save_pretrained(d)
    return str(d)


def test_langchain_and_llamaindex(tiny):
    from ipex_llm.langchain.embeddings import TransformersEmbeddings
    from ipex_llm.langchain.llms import TransformersLLM
    from ipex_llm.llamaindex.llms import IpexLLM
    llm = TransformersLLM.from_model_id(tiny, model_kwargs={"torch_dtype": torch.float32}, device_map="cpu")
    out = llm.invoke("w1 w2 w3", max_new_tokens=5)
    assert isinstance(out, str)
    emb = TransformersEmbeddings.from_model_id(tiny, model_kwargs={"torch_dtype": torch.float32}, device_map="cpu")
    v = emb.embed_query("w1 w2")
    assert len(v) == 64 and len(emb.embed_documents(["w1", "w2 w3"])) == 2
    from ipex_llm.langchain.embeddings import TransformersBgeEmbeddings
    bge = TransformersBgeEmbeddings(model=emb.model, tokenizer=emb.tokenizer)
    b = torch.tensor(bge.embed_query("w1 w2"))
    assert b.shape == (64,) and abs(float(b.norm()) - 1.0) < 1e-4          # first token's state, unit length
    li = IpexLLM(model_name=tiny, device_map="cpu", max_new_tokens=4, model_kwargs={"torch_dtype": torch.float32})
    r = li.complete("w5 w6")
    assert isinstance(r.text, str)
    chunks = list(li.stream_complete("w5 w6"))
    assert chunks and chunks[-1].text == r.text


def test_npu_named_entry_point(tiny):
    from ipex_llm.transformers.npu_model import AutoModelForCausalLM
    m = AutoModelForCausalLM.from_pretrained(tiny, load_in_low_bit="sym_int4_rtn", max_context_len=1024,
                                             max_prompt_len=512, transpose_value_cache=True,
                                             torch_dtype=torch.float32)
    out = m.generate(torch.tensor([[5, 6, 7]]), max_new_tokens=3, do_sample=False)
    assert out.shape == (1, 6)


def test_json_prefix_checker_and_processor(tiny):
    from transformers import AutoTokenizer
    from ipex_llm.transformers.xgrammar import _JsonPrefix, create_json_logits_processor
    good = ['{"a": [1, 2.5e3, true, null], "b": {"c": "x\\n\\u00e9"}}', "[]", '"s"', "-0.5", "{}"]
    for g in good:
        s = _JsonPrefix()
        assert s.feed(g) and s.complete, g
        for cut in range(1, len(g)):
            assert _JsonPrefix().feed(g[:cut]), g[:cut]
    for bad in ['{"a" 1}', "[1,,2]", "{,}", "tru e", '{"a":}', "01", "[1 2]"]:
        assert not _JsonPrefix().feed(bad) or not _JsonPrefix().feed(bad + " "), bad
    tok = AutoTokenizer.from_pretrained(tiny)
    proc = create_json_logits_processor(tok, 64)
    ids = torch.tensor([[5, 6]])
    scores = torch.zeros(1, 64)
    out = proc(ids, scores)
    allowed = {tok.decode([i]) for i in torch.nonzero(torch.isfinite(out[0])).flatten().tolist()}
    assert "{" in allowed and "[" in allowed and "}" not in allowed and "," not in allowed


def test_llm_convert_cli_and_benchmark_wrapper(tiny, tmp_path, capsys):
    from ipex_llm import llm_convert
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm.utils import BenchmarkWrapper
    from ipex_llm_b200.cli.llm_cli import main as cli_main
    out = llm_convert(tiny, str(tmp_path / "out"), model_family="llama", outtype="int8")
    assert os.path.isdir(out) and "bigdl_transformers_low_bit" in json.load(open(os.path.join(out, "config.json")))
    m = AutoModelForCausalLM.load_low_bit(out)
    bw = BenchmarkWrapper(m, do_print=False)
    bw.generate(torch.tensor([[5, 6, 7, 8]]), max_new_tokens=6, do_sample=False)
    assert bw.first_cost > 0 and bw.rest_cost_mean > 0
    assert cli_main(["-m", out, "-p", "w1 w2", "-n", "4", "--device", "cpu"]) == 0


def test_native_style_classes_and_legacy_names(tiny):
    import bigdl.llm  # noqa: F401
    from bigdl.llm.transformers import AutoModelForCausalLM as Legacy
    from ipex_llm.models import Llama
    from ipex_llm.transformers import AutoModelForCausalLM
    assert Legacy is AutoModelForCausalLM
    llm = Llama(tiny, low_bit="sym_int8", device="cpu")
    res = llm("w1 w2 w3", max_tokens=5)
    assert res["object"] == "text_completion" and res["usage"]["completion_tokens"] <= 5
    toks = llm.tokenize("w1 w2")
    assert llm.detokenize(toks).decode().split() == ["w1", "w2"]
    pieces = list(llm("w1 w2", max_tokens=4, stream=True))
    assert pieces[-1]["choices"][0]["finish_reason"] in ("length", "stop")
    emb = llm.create_embedding("w3 w4")
    assert len(emb["data"][0]["embedding"]) == 64
    # the transformers-flavoured token API of the same classes (ggml/model/generation/utils.py:28-180)
    from ipex_llm.ggml.model.generation import GenerationMixin
    from ipex_llm.ggml.model.llama import Llama as ByPath
    assert ByPath is Llama and isinstance(llm, GenerationMixin)
    for fam in ("gptneox", "bloom", "starcoder", "chatglm"):
        __import__(f"ipex_llm.ggml.model.{fam}")
    new = llm.generate(toks, max_new_tokens=4, temperature=0.0)
    assert len(new) == 1 and 1 <= len(new[0]) <= 4
    assert new == llm.generate([toks], max_new_tokens=4, temperature=0.0)
    assert new[0] == list(llm._generate(toks, max_tokens=4))
    assert llm.batch_decode(new) == [llm.decode(new[0])] and isinstance(llm.batch_decode(new[0]), str)
    assert llm.generate([]) is None


def test_ggml_quantize_module(tiny_llama_dir, tmp_path):
    """The reference's ``ipex_llm.ggml.quantize`` import path: qtype table and in-process ``quantize``."""
    import torch
    from ipex_llm.ggml.quantize import ggml_tensor_qtype, quantize
    from ipex_llm.transformers import AutoModelForCausalLM
    assert ggml_tensor_qtype["sym_int4"] == 2 and ggml_tensor_qtype["nf4"] == 10
    out = quantize(tiny_llama_dir, str(tmp_path / "q"), model_family="llama", dtype="q8_0")
    model = AutoModelForCausalLM.load_low_bit(out)
    ids = torch.randint(0, 32000, (1, 8))
    assert model.generate(ids, max_new_tokens=2, do_sample=False).shape == (1, 10)


def test_ipex_llm_init_settings(capsys):
    from ipex_llm_b200.cli import ipex_llm_init
    env = ipex_llm_init.settings(gpu=True, tcmalloc=False, jemalloc=False, threads=6)
    assert env["OMP_NUM_THREADS"] == "6" and env["CUDA_DEVICE_MAX_CONNECTIONS"] == "1"
    assert env["MASTER_ADDR"] == "127.0.0.1" and "LD_PRELOAD" not in env
    assert "CUDA_DEVICE_MAX_CONNECTIONS" not in ipex_llm_init.settings(False, False, False)
    assert ipex_llm_init.main(["--gpu", "--threads", "3"]) == 0
    out = capsys.readouterr().out
    assert "export OMP_NUM_THREADS=3" in out and "export NCCL_NVLS_ENABLE=1" in out


def test_langchain_vllm_wrapper_builds_sampling_params():
    """``langchain.vllm.VLLM`` turns a generate call into sampling parameters + ``client.generate`` (a double stands in
    for the vLLM engine; nothing is loaded)."""
    from ipex_llm_b200.langchain.vllm import VLLM

    class _Out:
        def __init__(self, text):
            self.text = text
            self.outputs = [self]

    class _Client:
        def __init__(self):
            self.calls = []

        def generate(self, prompts, params):
            self.calls.append((list(prompts), params))
            return [_Out(p + "!") for p in prompts]

    client = _Client()
    llm = VLLM(client=client, model="unused", temperature=0.5, max_new_tokens=7)
    texts = llm.generate_texts(["a", "bc"], stop=["\n"], top_p=0.9)
    assert texts == ["a!", "bc!"]
    prompts, params = client.calls[0]
    get = (lambda k: params[k]) if isinstance(params, dict) else (lambda k: getattr(params, k))
    assert prompts == ["a", "bc"] and get("temperature") == 0.5 and get("max_tokens") == 7 and get("top_p") == 0.9
    assert list(get("stop")) == ["\n"]
    assert llm._llm_type == "vllm"


def test_vllm_adapter_against_the_installed_vllm():
    """The vLLM adapter on the installed vLLM, in a child process (vLLM keeps process-wide state and takes tens of
    seconds to import): vLLM's QKV / row / merged-column parallel linears and ``ParallelLMHead`` are built on the CPU,
    packed by ``convert_vllm_model`` and compared with the dense product; the loader / logits patches land on vLLM's
    classes; the ``IPEXLLM*`` engine classes subclass vLLM's and pass arguments through."""
    import importlib.util
    import os
    import socket
    import subprocess
    import sys
    import pytest
    if importlib.util.find_spec("vllm") is None:
        pytest.skip("vllm is not installed")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    worker = os.path.join(os.path.dirname(__file__), "dist_workers", "vllm_layers_worker.py")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", CUDA_VISIBLE_DEVICES="")
    res = subprocess.run([sys.executable, worker, str(port)], capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0 and res.stdout.strip().endswith("OK"), res.stderr[-3000:]


def test_langchain_native_class_wrappers(tiny):
    """``LlamaLLM`` / ``BigdlNativeLLM`` / ``LlamaEmbeddings`` over the llama-cpp-python style classes (reference
    langchain/llms/bigdlllm.py, langchain/embeddings/bigdlllm.py): blocking and streaming calls agree, stop words cut
    the text, the family table rejects unknown names."""
    from ipex_llm.langchain.embeddings import BigdlNativeEmbeddings, LlamaEmbeddings
    from ipex_llm.langchain.llms import BigdlNativeLLM, LlamaLLM, type_to_cls_dict
    from ipex_llm.langchain.llms.transformerspipelinellm import TransformersPipelineLLM  # noqa: F401
    llm = LlamaLLM(model_path=tiny, max_tokens=6, temperature=0.0, streaming=False, low_bit="sym_int8", device="cpu")
    assert llm._llm_type == "BigDL" and llm._identifying_params["model_family"] == "llama"
    text = llm._call("w1 w2 w3")
    assert isinstance(text, str) and llm.get_num_tokens("w1 w2 w3") >= 3
    pieces = list(llm.stream("w1 w2 w3"))
    assert "".join(pieces).strip() == text.strip()
    words = text.split()
    if len(words) >= 2:                                     # a stop word cuts the completion before it
        cut = llm._call("w1 w2 w3", stop=[words[-1]])
        assert words[-1] not in cut and cut.strip() == text[:text.find(words[-1])].strip()
    with pytest.raises(ValueError):
        LlamaLLM(client=llm.client, stop=["a"])._get_parameters(stop=["b"])
    same = BigdlNativeLLM(model_family="llama", client=llm.client, max_tokens=6, temperature=0.0, streaming=True)
    assert same._call("w1 w2 w3").strip() == text.strip()
    with pytest.raises(ValueError):
        BigdlNativeLLM(model_family="mamba", model_path=tiny)
    assert type_to_cls_dict["LlamaLLM"] is LlamaLLM
    emb = LlamaEmbeddings(client=llm.client)
    v = emb.embed_query("w1 w2")
    assert len(v) == 64 and len(emb.embed_documents(["w1", "w2 w3"])) == 2
    assert BigdlNativeEmbeddings(model_family="llama", client=llm.client).embed_query("w1 w2") == v
