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
@pytest.mark.parametrize("T", [1, 5, 40])
def test_moe_forward_matches_expert_loop(qname, T):
    """T*k <= 64 takes the per-slot GEMV launch, T = 40 the grouped tensor-core path; both against a plain loop
    over the dequantized experts."""
    from ipex_llm_b200.ops import cuda_ops
    E, H, I, k = 8, 256, 512, 2
    bank = _bank(E, H, I, qname, torch.float16)
    assert cuda_ops.moe_supported(bank)
    torch.manual_seed(T)
    x = (torch.randn(T, H, device="cuda") * 0.5).half()
    logits = torch.randn(T, E, device="cuda")
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
