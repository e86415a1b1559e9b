"""Tracing hooks: NVTX ranges are free without a GPU / without the flag; the profiler wrapper returns a table."""
import torch


def test_nvtx_range_is_a_noop_without_cuda(monkeypatch):
    from ipex_llm_b200.utils.tracing import nvtx_range
    monkeypatch.setenv("IPEX_LLM_NVTX", "1")
    with nvtx_range("anything"):
        x = torch.ones(2) + 1
    assert x.sum().item() == 4


def test_profile_generate_on_cpu(tiny_llama_dir):
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.utils.tracing import profile_generate
    model = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_low_bit="sym_int8")
    ids = torch.randint(0, 32000, (1, 8))
    out, table = profile_generate(model, ids, max_new_tokens=3, do_sample=False, row_limit=5)
    assert out.shape == (1, 11)
    assert "Name" in table and "CPU total" in table
