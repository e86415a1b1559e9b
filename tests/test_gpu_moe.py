"""Mixture-of-experts kernels: device-side routing, per-slot expert GEMVs, grouped prompt path, tiny Mixtral."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("E,k", [(8, 2), (60, 4), (128, 8), (256, 6)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_router_softmax_topk(E, k, dtype):
    from ipex_llm_b200.ops import cuda_ops
    torch.manual_seed(E + k)
    logits = torch.randn(37, E, device="cuda").to(dtype)
    probs, w, idx = cuda_ops.moe_softmax_topk(logits, k, True)
    ref_p = torch.softmax(logits.float(), dim=-1)
    ref_w, ref_i = torch.topk(ref_p, k, dim=-1)
    ref_w = ref_w / ref_w.sum(-1, keepdim=True)
    assert torch.allclose(probs, ref_p, atol=1e-5)
    assert torch.equal(idx, ref_i)
    assert torch.allclose(w, ref_w, atol=1e-5)
    _, w2, _ = cuda_ops.moe_softmax_topk(logits, k, False)
    assert torch.allclose(w2, torch.topk(ref_p, k, dim=-1).values, atol=1e-5)


@pytest.mark.parametrize("cfg", [(256, 8, 4, 8), (64, 8, 3, 6), (160, 8, 3, 6), (16, 4, 2, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_group_topk_kernel(cfg, dtype):
    """DeepSeek-V3 grouped routing kernel against the tensor-op formulation."""
    from ipex_llm_b200.ops import cuda_ops
    from ipex_llm_b200.ops.moe import _group_topk_impl
    E, n_group, topk_group, k = cfg
    torch.manual_seed(E + k)
    scores = (torch.randn(37, E, device="cuda") * 2).to(dtype)
    bias = torch.randn(E, device="cuda") * 0.3
    assert hasattr(cuda_ops.cuda_lib(), "ipex_moe_group_topk")
    for renorm in (True, False):
        idx, w = cuda_ops.moe_group_topk(scores, bias, n_group, topk_group, k, renorm, 2.5)
        ref_idx, ref_w = _group_topk_impl(scores, bias, n_group, topk_group, k, renorm, 2.5)
        assert torch.equal(idx, ref_idx)
        assert torch.allclose(w, ref_w.float(), atol=1e-5, rtol=1e-4)


def _bank(E, H, I, qname, dtype):
    from ipex_llm_b200.ops.moe import LowBitExperts
    from ipex_llm_b200.quant import qtypes as qt
    from ipex_llm_b200.quant.params import FP4Params
    q = qt.qtype_from_name(qname)
    bank = LowBitExperts(E, H, I, q)
    torch.manual_seed(1)
    for e in range(E):
        for name, shape in (("w1", (I, H)), ("w3", (I, H)), ("w2", (H, I))):
            w = torch.randn(*shape) * 0.05
            getattr(bank[e], name)._parameters["weight"] = FP4Params(w, requires_grad=False, quantized=False,
                                                                     qtype=q).to("cuda")
    return bank.to("cuda")


@pytest.mark.parametrize("qname", ["sym_int4", "fp8_e4m3", "nf4"])
@pytest.mark.parametrize("T", [1, 5, 8, 19, 32, 40])
def test_moe_forward_matches_expert_loop(qname, T):
    """T = 1 takes the per-slot GEMV launch, 2 <= T <= 32 the expert-grouped GEMV (one to four groups of eight rows
    per expert), T = 40 the grouped tensor-core path; all against a plain loop over the dequantized experts."""
    from ipex_llm_b200.ops import cuda_ops
    E, H, I, k = 8, 256, 512, 2
    bank = _bank(E, H, I, qname, torch.float16)
    assert cuda_ops.moe_supported(bank)
    torch.manual_seed(T)
    x = (torch.randn(T, H, device="cuda") * 0.5).half()
    logits = torch.randn(T, E, device="cuda")
    logits[:, 2] += 2.0                # a popular expert: more than eight rows in one group for the larger T
    _, w, idx = cuda_ops.moe_softmax_topk(logits, k, True)
    out = bank(x, idx, w)
    ref = torch.zeros(T, H, device="cuda")
    for t in range(T):
        for r in range(k):
            e = bank[int(idx[t, r])]
            w1 = e.w1.weight.dequantize(torch.float32)
            w3 = e.w3.weight.dequantize(torch.float32)
            w2 = e.w2.weight.dequantize(torch.float32)
            h = torch.nn.functional.silu(x[t].float() @ w1.t()) * (x[t].float() @ w3.t())
            ref[t] += float(w[t, r]) * (h.half().float() @ w2.t())
    torch.cuda.synchronize()
    err = (out.float() - ref).abs().max().item() / ref.abs().max().item()
    assert err < 1e-2, err


def test_moe_grouped_gemv_long_contraction():
    """A down projection whose staged rows do not fit eight at a time (K = 8192 -> six rows per CTA): one expert gets
    all eight tokens, so its rows span two row groups."""
    from ipex_llm_b200.ops import cuda_ops
    E, H, I, k, T = 4, 128, 8192, 2, 8
    bank = _bank(E, H, I, "sym_int4", torch.float16)
    torch.manual_seed(3)
    x = (torch.randn(T, H, device="cuda") * 0.5).half()
    logits = torch.randn(T, E, device="cuda")
    logits[:, 1] += 10.0
    _, w, idx = cuda_ops.moe_softmax_topk(logits, k, True)
    out = cuda_ops.moe_forward(bank, x, idx, w)
    ref = cuda_ops._moe_forward_per_expert(bank, x, idx, w)
    torch.cuda.synchronize()
    err = (out.float() - ref.float()).abs().max().item() / ref.float().abs().max().item()
    assert err < 1e-2, err


@pytest.mark.parametrize("qname", ["sym_int4", "fp8_e4m3"])
@pytest.mark.parametrize("T", [300, 1100])
def test_moe_grouped_prompt_device_ranges(qname, T):
    """Prompt-sized routing with a skew (one expert gets most tokens, one gets none): the grouped GEMMs read their
    row ranges on the device and must agree with the per-expert loop that synchronises with the host."""
    from ipex_llm_b200.ops import cuda_ops
    E, H, I, k = 8, 256, 512, 2
    bank = _bank(E, H, I, qname, torch.float16)
    torch.manual_seed(T)
    x = (torch.randn(T, H, device="cuda") * 0.5).half()
    logits = torch.randn(T, E, device="cuda")
    logits[:, 3] += 3.0            # most tokens pick expert 3
    logits[:, 5] = -1e4            # nobody picks expert 5
    _, w, idx = cuda_ops.moe_softmax_topk(logits, k, True)
    assert hasattr(cuda_ops.cuda_lib(), "ipex_gemm_lowbit_tcgen05_grouped")
    out = cuda_ops._moe_forward_grouped(bank, x, idx, w)
    ref = cuda_ops._moe_forward_per_expert(bank, x, idx, w)
    torch.cuda.synchronize()
    cuda_ops.check_error_flag(x.device)
    err = (out.float() - ref.float()).abs().max().item() / ref.float().abs().max().item()
    assert err < 1e-2, err


def test_tiny_mixtral_decode_gpu():
    from transformers import MixtralConfig
    from ipex_llm.transformers import AutoModelForCausalLM
    cfg = MixtralConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, vocab_size=1000, max_position_embeddings=256, num_local_experts=4,
                        num_experts_per_tok=2, tie_word_embeddings=False)
    m = AutoModelForCausalLM.from_config(cfg, load_in_low_bit="sym_int4", torch_dtype=torch.float16, device="cuda")
    ids = torch.randint(0, 1000, (1, 12), device="cuda")
    out = m.generate(ids, max_new_tokens=6, do_sample=False)
    assert out.shape == (1, 18)
    # incremental decoding agrees with a full forward over the generated prefix
    with torch.no_grad():
        full = m(out[:, :-1]).logits[:, -1].argmax(-1)
    assert torch.equal(full, out[:, -1])


def test_mixtral_runs_on_the_graph_engine():
    """Mixtral's sparse layers are part of the flattened engine: graph-captured decode steps (router, expert GEMVs
    through the device pointer table) and the flat prompt pass (expert-sorted grouped GEMMs) agree with the module
    tree, for batch 1 and for a batch of 8."""
    from transformers import MixtralConfig
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200 import engine
    cfg = MixtralConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, vocab_size=1000, max_position_embeddings=512, num_local_experts=8,
                        num_experts_per_tok=2, tie_word_embeddings=False, sliding_window=None)
    m = AutoModelForCausalLM.from_config(cfg, load_in_low_bit="sym_int4", torch_dtype=torch.float16, device="cuda")
    assert engine.supports(m, {})

    def close(a, b):
        # random routers have near-ties: a rounding difference may send a token to another expert, so rows are
        # compared by direction (every row close, almost all rows very close) instead of element by element
        cos = torch.nn.functional.cosine_similarity(a, b, dim=-1)
        return bool(cos.min() > 0.9) and bool(cos.median() > 0.99)

    for B, S in ((1, 12), (8, 40)):
        ids = torch.randint(0, 1000, (B, S), device="cuda", generator=torch.Generator("cuda").manual_seed(B))
        eng = engine.get_engine(m, B, S + 8)
        assert eng.has_moe
        logits = eng.prefill(ids).float()
        with torch.no_grad():
            ref = m(ids).logits[:, -1].float()
        assert close(logits, ref), torch.nn.functional.cosine_similarity(logits, ref, dim=-1)
        # two graph-captured decode steps against full forwards over the extended sequences
        seq = ids
        for _ in range(2):
            nxt = ref.argmax(-1)
            seq = torch.cat([seq, nxt[:, None]], dim=1)
            eng.tokens[:B] = nxt
            eng.decode_step(B, use_graph=True)
            torch.cuda.synchronize()
            step = eng.logits[:B].float()
            with torch.no_grad():
                ref = m(seq).logits[:, -1].float()
            assert close(step, ref), torch.nn.functional.cosine_similarity(step, ref, dim=-1)
        assert len(eng._graphs) > 0, "decode steps were not graph-captured"
    out = m.generate(ids, max_new_tokens=6, do_sample=False)
    assert out.shape == (8, 46)
