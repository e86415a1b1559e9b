"""Whole-step decode kernel (native/cuda/decode_mega.cu) against the per-kernel decode path of the same engine:
logits, chosen tokens and appended KV rows, for symmetric int4 and fp8 weights, plain and e5m2 KV caches,
multi-head / grouped-query / 16-way grouped heads, 1-4 sequences, eager launches and graph replay."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _force_fused_step(monkeypatch):
    # on one GPU the engine prefers the separate kernels; these tests are about the fused step
    monkeypatch.setenv("IPEX_LLM_DECODE_MEGA", "1")


def _model(hidden, inter, heads, kv_heads, layers, low_bit, dtype, head_dim=None):
    from transformers import LlamaConfig
    from ipex_llm.transformers import AutoModelForCausalLM
    kw = {} if head_dim is None else {"head_dim": head_dim}
    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers,
                      num_attention_heads=heads, num_key_value_heads=kv_heads, vocab_size=32000,
                      max_position_embeddings=2048, tie_word_embeddings=False, **kw)
    torch.manual_seed(0)
    return AutoModelForCausalLM.from_config(cfg, load_in_low_bit=low_bit, device="cuda", torch_dtype=dtype)


def _run(eng, ids, steps, mega, graph=False):
    B = ids.shape[0]
    logits = eng.prefill(ids)
    eng.tokens[:B] = logits.argmax(-1)
    eng._mega = None if mega else False
    eng._graphs = {}
    rec = []
    for _ in range(steps):
        eng.decode_step(B, use_graph=graph)
        rec.append((eng.logits[:B].float().clone(), eng.tokens[:B].clone()))
    torch.cuda.synchronize()
    from ipex_llm_b200.ops import cuda_ops
    cuda_ops.check_error_flag(ids.device)
    S = ids.shape[1]
    kv = [(lay._k[:B, :, S:S + steps].clone(), lay._v[:B, :, S:S + steps].clone()) for lay in eng.cache.layers]
    return rec, kv, int(eng.past_len[0].item())


CASES = [
    # hidden, inter, heads, kv, layers, low_bit, dtype, kv_fp8, B, prompt
    (512, 1408, 8, 2, 2, "sym_int4", torch.float16, True, 1, 40),
    (512, 1408, 8, 2, 2, "sym_int4", torch.float16, False, 2, 33),
    (1024, 2816, 8, 8, 2, "sym_int4", torch.float16, True, 1, 300),       # head_dim 128, multi-head, several splits
    (1024, 2816, 8, 8, 1, "sym_int4", torch.bfloat16, False, 3, 70),
    (1024, 2816, 16, 1, 2, "sym_int4", torch.float16, True, 1, 700),      # 16 query heads per kv head
    (1024, 2816, 8, 1, 2, "fp8_e4m3", torch.bfloat16, True, 1, 130),      # head_dim 128, 8 per kv head, fp8 weights
    (512, 1408, 8, 2, 2, "fp8_e4m3", torch.bfloat16, False, 4, 20),
]


@pytest.mark.parametrize("case", CASES)
def test_fused_step_matches_per_kernel_path(case, monkeypatch):
    hidden, inter, heads, kvh, layers, low_bit, dtype, kv_fp8, B, prompt = case
    monkeypatch.setenv("IPEX_LLM_QUANTIZE_KV_CACHE", "1" if kv_fp8 else "0")
    from ipex_llm_b200.engine import get_engine
    from ipex_llm_b200.engine.mega import MegaStep
    m = _model(hidden, inter, heads, kvh, layers, low_bit, dtype)
    eng = get_engine(m, B, 1024)
    assert MegaStep.supported(eng) is None, MegaStep.supported(eng)
    g = torch.Generator(device="cpu").manual_seed(prompt)
    ids = torch.randint(0, 32000, (B, prompt), generator=g).cuda()
    steps = 5
    ref, kv_ref, len_ref = _run(eng, ids, steps, mega=False)
    out, kv_out, len_out = _run(eng, ids, steps, mega=True)
    assert eng._mega not in (None, False)
    assert len_ref == len_out == prompt + steps
    # the first step sees identical inputs: logits must agree closely and the KV rows it appends must match
    l0, l1 = ref[0][0], out[0][0]
    cos = torch.nn.functional.cosine_similarity(l0.flatten(), l1.flatten(), dim=0).item()
    assert cos > 0.9995, cos
    scale = l0.abs().max().item()
    assert (l0 - l1).abs().max().item() < 0.03 * scale + 1e-3
    for (k0, v0), (k1, v1) in zip(kv_ref, kv_out):
        if k0.dtype == torch.uint8:
            # e5m2 codes: a rotated value may round to the neighbouring code; compare the decoded values
            from ipex_llm_b200.ops.kv_cache import fp8_e5m2_dequantize
            for x0, x1 in ((k0, k1), (v0, v1)):
                f0 = fp8_e5m2_dequantize(x0[:, :, 0].contiguous(), torch.float32)
                f1 = fp8_e5m2_dequantize(x1[:, :, 0].contiguous(), torch.float32)
                assert torch.allclose(f0, f1, atol=2e-2, rtol=0.26)
        else:
            assert torch.allclose(k0[:, :, 0].float(), k1[:, :, 0].float(), atol=2e-2, rtol=2e-2)
            assert torch.allclose(v0[:, :, 0].float(), v1[:, :, 0].float(), atol=2e-2, rtol=2e-2)
    # later steps: same tokens as long as neither path has diverged, logits stay close while they agree
    agree = True
    for (la, ta), (lb, tb) in zip(ref, out):
        if not agree:
            break
        c = torch.nn.functional.cosine_similarity(la.flatten(), lb.flatten(), dim=0).item()
        assert c > 0.999, c
        agree = bool((ta == tb).all())
    # the arg-max the kernel reports is the arg-max of the logits it wrote
    for lg, tk in out:
        top = lg.max(dim=-1).values
        assert torch.equal(lg.gather(1, tk.view(-1, 1)).view(-1), top)


def test_fused_step_graph_replay_matches_eager(monkeypatch):
    monkeypatch.setenv("IPEX_LLM_QUANTIZE_KV_CACHE", "1")
    from ipex_llm_b200.engine import get_engine
    m = _model(512, 1408, 8, 2, 2, "sym_int4", torch.float16)
    eng = get_engine(m, 1, 512)
    ids = torch.randint(0, 32000, (1, 48), device="cuda")
    eager, _, _ = _run(eng, ids, 6, mega=True, graph=False)
    replay, _, _ = _run(eng, ids, 6, mega=True, graph=True)
    for (la, ta), (lb, tb) in zip(eager, replay):
        assert torch.equal(ta, tb)
        assert torch.allclose(la, lb, atol=2e-3, rtol=1e-3)


def test_generate_uses_fused_step():
    m = _model(512, 1408, 8, 2, 2, "sym_int4", torch.float16)
    ids = torch.randint(0, 32000, (1, 24), device="cuda")
    out = m.generate(ids, max_new_tokens=8, do_sample=False)
    assert out.shape == (1, 32)
    eng = m._ipex_engine
    assert eng._mega not in (None, False) and eng.kernel_launches_per_step == 1
