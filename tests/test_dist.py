"""Multi-process tests: tensor parallel (gloo ranks on CPU, NCCL + peer-memory kernels on GPUs), pipeline
parallel and the host-side failure paths.  Workers live in tests/dist_workers/ and are launched with torchrun."""
import os
import socket
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKERS = os.path.join(ROOT, "tests", "dist_workers")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_workers(script, nproc, extra_args, env=None, timeout=600):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(WORKERS, script), *extra_args]
    e = dict(os.environ)
    e.setdefault("OMP_NUM_THREADS", "2")
    e["NCCL_NVLS_ENABLE"] = "0"
    if env:
        e.update(env)
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e)
    return res


@pytest.fixture(scope="module")
def tp_llama_dir(tmp_path_factory):
    """Tiny Llama whose per-rank shards stay multiples of 64 for 2 and 4 ranks."""
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=256, intermediate_size=768, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=4, vocab_size=32000, max_position_embeddings=512, tie_word_embeddings=False)
    torch.manual_seed(0)
    m = LlamaForCausalLM(cfg)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() > 1:
                p.normal_(0.0, 0.02)
    d = tmp_path_factory.mktemp("tp_llama")
    m.save_pretrained(d)
    return str(d)


def test_tensor_parallel_cpu_gloo(tp_llama_dir):
    res = run_workers("tp_worker.py", 2, ["--device", "cpu", "--model-dir", tp_llama_dir])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count(": ok") == 2


def test_pipeline_parallel_across_families_cpu_gloo():
    """Wrappers that scale / divide / soft-cap their logits, MoE blocks, latent attention, fused qkv: see the worker."""
    res = run_workers("pp_families_worker.py", 2, [], timeout=900)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count(": ok") == 2


def test_pipeline_parallel_serving_cpu_gloo(tmp_path):
    """``PPModelWorker`` end to end on two gloo stages (reference Pipeline-Parallel-Serving/pipeline_serving.py)."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import LlamaConfig, LlamaForCausalLM, PreTrainedTokenizerFast
    words = ["<pad>", "<s>", "</s>", "<unk>"] + [f"w{i}" for i in range(60)]
    tk = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tk.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok = PreTrainedTokenizerFast(tokenizer_object=tk, pad_token="<pad>", bos_token="<s>", eos_token="</s>",
                                  unk_token="<unk>")
    cfg = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=64, max_position_embeddings=256, tie_word_embeddings=False,
                      eos_token_id=2, pad_token_id=0, bos_token_id=1)
    torch.manual_seed(0)
    LlamaForCausalLM(cfg).save_pretrained(tmp_path)
    tok.save_pretrained(tmp_path)
    res = run_workers("pp_serving_worker.py", 2, [str(tmp_path)], timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count(": ok") == 2


def test_tensor_parallel_across_families_cpu_gloo():
    """Fused qkv / gate_up, expert banks, shared experts, replicated attention: see the worker's docstring."""
    res = run_workers("tp_families_worker.py", 2, [], timeout=900)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count(": ok") == 2


@pytest.mark.gpu
def test_tensor_parallel_gpu(tp_llama_dir):
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    res = run_workers("tp_worker.py", 2, ["--device", "cuda", "--model-dir", tp_llama_dir])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.fixture(scope="module")
def pp_llama_dir(tmp_path_factory):
    """Tiny Llama with 5 layers, so that 2 stages get 3 + 2 layers."""
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=128, intermediate_size=256, num_hidden_layers=5, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=32000, max_position_embeddings=512, tie_word_embeddings=False)
    torch.manual_seed(1)
    m = LlamaForCausalLM(cfg)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() > 1:
                p.normal_(0.0, 0.05)
    d = tmp_path_factory.mktemp("pp_llama")
    m.save_pretrained(d)
    return str(d)


def test_pipeline_parallel_cpu_gloo(pp_llama_dir):
    res = run_workers("pp_worker.py", 2, ["--device", "cpu", "--model-dir", pp_llama_dir])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count(": ok") == 2


@pytest.mark.gpu
def test_pipeline_parallel_gpu(pp_llama_dir):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    res = run_workers("pp_worker.py", 2, ["--device", "cuda", "--model-dir", pp_llama_dir])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]


def test_dp_fused_optimizer_cpu_gloo():
    res = run_workers("dp_worker.py", 2, ["--device", "cpu"])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count(": ok") == 2


@pytest.mark.gpu
def test_dp_fused_optimizer_gpu():
    """reduce-scatter + AdamW + all-gather in one kernel over peer memory."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    res = run_workers("dp_worker.py", 2, ["--device", "cuda"])
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.gpu
def test_device_wait_times_out_cleanly():
    """A bounded device-side wait that nothing satisfies returns an error status and leaves the context usable."""
    from ipex_llm_b200.native.lib import cuda_lib, current_stream, ptr
    from ipex_llm_b200.ops import cuda_ops
    dev = torch.device("cuda", 0)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    err = cuda_ops.error_flag(dev)
    rc = cuda_lib().ipex_wait_timeout_probe(ptr(counter), 1, 2000, ptr(err), current_stream())
    assert rc == 0
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="wait expired"):
        cuda_ops.check_error_flag(dev)
    # the flag was cleared and the context still works
    cuda_ops.check_error_flag(dev)
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0
