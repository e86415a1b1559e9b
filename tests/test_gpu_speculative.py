"""Self-speculative decoding on the two graph engines: multi-token verification against token-by-token decode,
and the generate loop against plain greedy decoding of the target."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _load(tiny_llama_dir, low_bit, dtype=torch.float16):
    from ipex_llm.transformers import AutoModelForCausalLM
    m = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_low_bit=low_bit, torch_dtype=dtype)
    return m.to(dtype).to("cuda")


@pytest.mark.parametrize("low_bit", ["sym_int4", "fp16"])
@pytest.mark.parametrize("kv", ["0", "1"])
def test_verify_step_equals_sequential_decode(tiny_llama_dir, monkeypatch, low_bit, kv):
    """Scoring S tokens in one pass gives the logits that S single-token steps give."""
    from ipex_llm_b200.engine import DecoderEngine
    from ipex_llm_b200.ops import cuda_ops
    monkeypatch.setenv("IPEX_LLM_QUANTIZE_KV_CACHE", kv)
    m = _load(tiny_llama_dir, low_bit)
    eng = DecoderEngine(m, max_batch=8, max_len=256)
    torch.manual_seed(3)
    ids = torch.randint(0, 32000, (1, 21), device="cuda")
    S = 6
    # token by token
    first = int(torch.argmax(eng.prefill(ids)[0]))
    eng.tokens[:1].fill_(first)
    seq_tokens, seq_logits = [first], []
    for _ in range(S):
        eng.decode_step(1)
        seq_logits.append(eng.logits[0].float().clone())
        seq_tokens.append(int(eng.tokens[0]))
    k_seq = eng.cache.layers[1]._k[:, :, 21:21 + S].clone()
    # in one pass (fresh prompt pass: the cache pool hands back the same storage, rows past the prompt are stale)
    eng.prefill(ids)
    eng.vtokens[:S].copy_(torch.tensor(seq_tokens[:S]))
    for use_graph in (False, True, True):
        eng.logits.zero_()
        eng.verify_step(S, use_graph=use_graph)
        torch.cuda.synchronize()
        cuda_ops.check_error_flag(ids.device)
        assert int(eng.past_len[0]) == 21
        for i in range(S):
            cos = torch.nn.functional.cosine_similarity(eng.logits[i].float(), seq_logits[i], dim=0).item()
            assert cos > 0.999, (use_graph, i, cos)
        assert eng.vout[:S].tolist() == [int(torch.argmax(eng.logits[i])) for i in range(S)]
        k_ver = eng.cache.layers[1]._k[:, :, 21:21 + S]
        if k_ver.dtype == torch.uint8:
            assert (k_ver != k_seq).float().mean().item() < 0.02
        else:
            assert torch.allclose(k_ver.float(), k_seq.float(), atol=2e-2)


def test_speculative_engine_greedy(tiny_llama_dir, monkeypatch):
    from ipex_llm_b200.transformers.speculative import attach_draft_model
    target = _load(tiny_llama_dir, "fp16")
    draft = _load(tiny_llama_dir, "sym_int4")
    torch.manual_seed(0)
    ids = torch.randint(0, 32000, (1, 24), device="cuda")
    ref = target.generate(ids, max_new_tokens=24, do_sample=False)
    attach_draft_model(target, draft)
    try:
        out = target.speculative_generate(ids, draft_model=draft, max_new_tokens=24, do_sample=False)
        assert getattr(draft, "_ipex_engine", None) is not None
        assert any(isinstance(k, tuple) and k[0] == "verify" for k in target._ipex_engine._graphs)
        assert out.shape == ref.shape
        # greedy decoding of a random model is chaotic after the first divergence; the first tokens must agree
        assert (out[0, 24:28] == ref[0, 24:28]).float().mean().item() >= 0.75, (out[0, 24:], ref[0, 24:])
        assert target.n_token_generated == 24 and target.n_drafted > 0
        assert len(target.draft_time) == len(target.verify_time) > 0
        # a draft identical to the target is always accepted, and the result is the target's own greedy decode
        twin = _load(tiny_llama_dir, "fp16")
        out2 = target.speculative_generate(ids, draft_model=twin, max_new_tokens=24, do_sample=False,
                                           max_step_draft=4, th_stop_draft=0.0, auto_th_stop_draft=False)
        assert target.n_matched >= target.n_drafted - 1, (target.n_matched, target.n_drafted)
        assert (out2[0, 24:30] == ref[0, 24:30]).float().mean().item() >= 0.8
        # the module-tree loop still runs when the engines are switched off
        monkeypatch.setenv("IPEX_LLM_SPEC_ENGINE", "0")
        out3 = target.speculative_generate(ids, draft_model=draft, max_new_tokens=8, do_sample=False)
        assert out3.shape == (1, 32)
    finally:
        target.draft_model = None


def test_speculative_engine_sampling_and_stream(tiny_llama_dir):
    from ipex_llm_b200.transformers.speculative import attach_draft_model
    target = _load(tiny_llama_dir, "fp16")
    draft = _load(tiny_llama_dir, "sym_int4")
    attach_draft_model(target, draft)

    class _Collect:
        def __init__(self):
            self.n, self.ended = 0, False

        def put(self, t):
            self.n += t.numel()

        def end(self):
            self.ended = True

    torch.manual_seed(1)
    ids = torch.randint(0, 32000, (1, 16), device="cuda")
    st = _Collect()
    out = target.speculative_generate(ids, draft_model=draft, max_new_tokens=12, do_sample=True, temperature=0.8,
                                      top_k=50, top_p=0.95, streamer=st)
    assert out.shape == (1, 28)
    assert st.ended and st.n == 28
