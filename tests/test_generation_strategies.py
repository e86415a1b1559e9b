"""Self-speculative and prompt-lookup decoding: greedy output must equal plain greedy decoding of the target."""
import pytest
import torch


@pytest.fixture(scope="module")
def target_and_draft(tiny_llama_dir):
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.transformers.speculative import attach_draft_model
    target = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_low_bit="sym_int8")
    draft = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_low_bit="sym_int4")
    return target, draft, attach_draft_model


def _plain_greedy(model, ids, n):
    return model._hf_generate(ids, max_new_tokens=n, do_sample=False)


def test_speculative_greedy_equals_target(target_and_draft):
    target, draft, attach = target_and_draft
    torch.manual_seed(0)
    ids = torch.randint(0, 32000, (1, 24))
    ref = _plain_greedy(target, ids, 24)
    attach(target, draft)
    try:
        out = target.generate(ids, max_new_tokens=24, do_sample=False)
        assert torch.equal(out, ref)
        assert target.n_drafted > 0 and 0 <= target.n_matched <= target.n_drafted
        assert len(target.draft_time) == len(target.verify_time) > 0
        assert target.n_token_generated == 24
        # the draft of a random-weight model rarely agrees; a draft identical to the target always does
        attach(target, target)
        out2 = target.speculative_generate(ids, draft_model=target, max_new_tokens=24, do_sample=False,
                                           max_step_draft=4, th_stop_draft=0.0, auto_th_stop_draft=False)
        assert torch.equal(out2, ref)
        assert target.n_matched == target.n_drafted
    finally:
        target.draft_model = None


def test_speculative_sampling_runs(target_and_draft):
    target, draft, attach = target_and_draft
    attach(target, draft)
    try:
        torch.manual_seed(1)
        ids = torch.randint(0, 32000, (1, 16))
        out = target.generate(ids, max_new_tokens=12, do_sample=True, temperature=0.8, top_k=50, top_p=0.95)
        assert out.shape == (1, 28)
    finally:
        target.draft_model = None


def test_lookup_greedy_equals_target(target_and_draft):
    target, _, _ = target_and_draft
    torch.manual_seed(2)
    # a repetitive prompt gives the n-gram table something to find
    piece = torch.randint(0, 32000, (1, 8))
    ids = piece.repeat(1, 4)
    ref = _plain_greedy(target, ids, 20)
    out = target.generate(ids, max_new_tokens=20, do_sample=False, lookahead=3)
    assert torch.equal(out, ref)
    assert target.n_token_generated == 20


def test_lookup_candidate_generator():
    from ipex_llm_b200.transformers.lookup import PromptLookupCandidateGenerator
    g = PromptLookupCandidateGenerator(num_output_tokens=3, max_matching_ngram_size=2)
    ids = torch.tensor([[5, 6, 7, 8, 9, 5, 6]])
    g.init_look_up_table(ids)
    cand, _ = g.get_candidates(ids)
    assert cand[0, 7:].tolist() == [7, 8, 9]
    g.update_candidate_strategy(3, 3, 1.0)
    assert g.num_output_tokens == 4
    g2 = PromptLookupCandidateGenerator(num_output_tokens=2)
    no_match = torch.tensor([[1, 2, 3, 4]])
    g2.init_look_up_table(no_match)
    same, _ = g2.get_candidates(no_match)
    assert same.shape[1] in (4, 5)


def test_performance_mode_enables_lookup(target_and_draft, monkeypatch):
    target, _, _ = target_and_draft
    monkeypatch.setenv("IPEX_LLM_PERFORMANCE_MODE", "1")
    ids = torch.randint(0, 32000, (1, 20)).repeat(1, 6)   # >= 100 tokens
    target.n_token_generated = -1
    out = target.generate(ids, max_new_tokens=6, do_sample=False)
    assert out.shape[1] == 126 and target.n_token_generated == 6


@pytest.mark.parametrize("family", ["qwen3", "gemma2", "mixtral", "deepseek_v3", "gptj"])
def test_speculative_and_lookup_equal_greedy_across_families(family):
    """Self-speculative and prompt-lookup decoding are exact for greedy search whatever the family's cache and
    attention path (package cache, soft-capped / sliding-window attention, MoE blocks, latent attention, a family
    with its own eager attention)."""
    import transformers
    from ipex_llm.transformers import AutoModelForCausalLM
    from test_cpu_model import FAMILY_CONFIGS
    cls_name, extra = FAMILY_CONFIGS[family]
    kw = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, vocab_size=1000, max_position_embeddings=256)
    kw.update(extra)
    cfg = getattr(transformers, cls_name)(**kw)
    torch.manual_seed(0)
    m = AutoModelForCausalLM.from_config(cfg, load_in_low_bit="bf16", device="cpu", torch_dtype=torch.float32,
                                         speculative=True)
    ids = torch.randint(0, 900, (1, 20))
    greedy = m._hf_generate(inputs=ids, max_new_tokens=12, do_sample=False)
    spec = m.generate(ids, max_new_tokens=12, do_sample=False)
    assert torch.equal(spec[:, :greedy.shape[1]], greedy[:, :spec.shape[1]])
    m.draft_model = None
    look = m.generate(ids, max_new_tokens=12, do_sample=False, lookahead=3, max_matching_ngram_size=2)
    assert torch.equal(look[:, :greedy.shape[1]], greedy[:, :look.shape[1]])
