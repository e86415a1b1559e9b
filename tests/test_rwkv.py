"""RWKV: reference loops of the three operators, the patched RWKV-4 forwards against transformers' own, and the
CUDA kernels against the loops."""
import pytest
import torch


def _tiny_rwkv(seed=0):
    from transformers import RwkvConfig, RwkvForCausalLM
    torch.manual_seed(seed)
    cfg = RwkvConfig(vocab_size=500, context_length=64, hidden_size=128, num_hidden_layers=3,
                     attention_hidden_size=128, intermediate_size=256, rescale_every=2)
    model = RwkvForCausalLM(cfg).eval()
    with torch.no_grad():
        for blk in model.rwkv.blocks:
            blk.attention.time_decay.uniform_(-2.0, 0.5)
            blk.attention.time_first.uniform_(-1.0, 1.0)
            for n in ("time_mix_key", "time_mix_value", "time_mix_receptance"):
                getattr(blk.attention, n).uniform_(0.1, 0.9)
            for n in ("time_mix_key", "time_mix_receptance"):
                getattr(blk.feed_forward, n).uniform_(0.1, 0.9)
    return model


def test_wkv_v4_loop_matches_transformers():
    from transformers.models.rwkv.modeling_rwkv import rwkv_linear_attention_cpu
    from ipex_llm_b200.ops.rwkv import rwkv_linear_attention_v4
    torch.manual_seed(0)
    B, T, C = 2, 9, 48
    decay, first = torch.randn(C), torch.randn(C)
    k, v = torch.randn(B, T, C), torch.randn(B, T, C)
    ref, ref_state = rwkv_linear_attention_cpu(decay, first, k, v, state=None, return_state=True)
    num, den = torch.zeros(B, C), torch.zeros(B, C)
    mx = torch.full((B, C), -1e38)
    out = rwkv_linear_attention_v4(-torch.exp(decay), first, k, v, num, den, mx)
    assert torch.allclose(out, ref, atol=1e-5)
    for a, b in zip((num, den, mx), ref_state):
        assert torch.allclose(a, b, atol=1e-5)


def test_time_shift_loop():
    from ipex_llm_b200.ops.rwkv import rwkv_time_shift
    torch.manual_seed(1)
    h, prev, mix = torch.randn(2, 5, 16), torch.randn(2, 16), torch.rand(3, 1, 16)
    out = rwkv_time_shift(h, prev, mix)
    sh = torch.cat([prev.unsqueeze(1), h[:, :-1]], dim=1)
    for n in range(3):
        assert torch.allclose(out[n], h * mix[n] + sh * (1 - mix[n]), atol=1e-6)
    out0 = rwkv_time_shift(h, None, mix)
    assert torch.allclose(out0[0][:, 0], h[:, 0] * mix[0, 0])


def test_rwkv4_patched_forward_equals_transformers():
    """optimize_model on RWKV-4: fused shift/recurrence forwards and low-bit linears; with a half-precision
    "low bit" the logits equal the stock model's, across a prompt pass and state-carrying single-token steps."""
    from ipex_llm import optimize_model
    ref = _tiny_rwkv()
    # batch 1: the stock single-token step broadcasts its carried row [B, C] against hidden [B, 1, C], which is
    # only right for one sequence
    ids = torch.randint(0, 500, (1, 12))
    with torch.no_grad():
        r1 = ref(ids[:, :8], use_cache=True)
        r2 = ref(ids[:, 8:9], state=r1.state, use_cache=True)
        r3 = ref(ids[:, 9:], state=r2.state, use_cache=True)
    model = optimize_model(_tiny_rwkv(), low_bit="bf16").float()
    assert model.rwkv.blocks[0].attention.forward.__func__.__name__ == "rwkv4_attention_forward"
    with torch.no_grad():
        o1 = model(ids[:, :8], use_cache=True)
        o2 = model(ids[:, 8:9], state=o1.state, use_cache=True)
        o3 = model(ids[:, 9:], state=o2.state, use_cache=True)
    for a, b in ((o1, r1), (o2, r2), (o3, r3)):
        cos = torch.nn.functional.cosine_similarity(a.logits[:, -1].flatten(), b.logits[:, -1].flatten(), dim=0).item()
        assert cos > 0.999, cos
    # low-bit: rescale happened on dense weights before quantization, so the quantized model still tracks the stock one
    q = optimize_model(_tiny_rwkv(), low_bit="sym_int8")
    with torch.no_grad():
        oq = q(ids[:, :8], use_cache=True)
    cos = torch.nn.functional.cosine_similarity(oq.logits[:, -1].flatten().float(), r1.logits[:, -1].flatten(),
                                                dim=0).item()
    assert cos > 0.99, cos


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_wkv_v4_kernel(dtype):
    from ipex_llm_b200.ops.rwkv import rwkv_linear_attention_v4
    torch.manual_seed(2)
    B, T, C = 3, 37, 200
    w, u = -torch.exp(torch.randn(C)), torch.randn(C)
    k, v = torch.randn(B, T, C).to(dtype), torch.randn(B, T, C).to(dtype)
    st = [torch.zeros(B, C), torch.zeros(B, C), torch.full((B, C), -1e38)]
    ref = rwkv_linear_attention_v4(w, u, k.float(), v.float(), *st)
    st_g = [torch.zeros(B, C).cuda(), torch.zeros(B, C).cuda(), torch.full((B, C), -1e38).cuda()]
    # two calls that carry the state must equal one call over the whole sequence
    o1 = rwkv_linear_attention_v4(w.cuda(), u.cuda(), k[:, :20].cuda(), v[:, :20].cuda(), *st_g)
    o2 = rwkv_linear_attention_v4(w.cuda(), u.cuda(), k[:, 20:].cuda(), v[:, 20:].cuda(), *st_g)
    out = torch.cat([o1, o2], dim=1).float().cpu()
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert (out - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item())
    for a, b in zip(st_g, st):
        assert torch.allclose(a.cpu(), b, atol=1e-3, rtol=1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("S", [32, 64])
def test_rwkv5_kernel(S):
    from ipex_llm_b200.ops.rwkv import rwkv_linear_attention_v5
    torch.manual_seed(3)
    B, H, T = 2, 3, 21
    w = torch.exp(-torch.exp(torch.randn(H, S)))
    u = torch.randn(H, S)
    r, k, v = (torch.randn(B, H, T, S) * 0.5 for _ in range(3))
    st = torch.randn(B, H, S, S) * 0.1
    st_g = st.clone().cuda()
    ref = rwkv_linear_attention_v5(w, u, r, k, v, st)
    out = rwkv_linear_attention_v5(w.cuda(), u.cuda(), r.cuda(), k.cuda(), v.cuda(), st_g)
    assert out.shape == (B, T, H, S)
    assert torch.allclose(out.cpu(), ref, atol=1e-3, rtol=1e-3)
    assert torch.allclose(st_g.cpu(), st, atol=1e-3, rtol=1e-3)


@pytest.mark.gpu
def test_time_shift_kernel_and_model_on_gpu():
    from ipex_llm import optimize_model
    from ipex_llm_b200.ops.rwkv import rwkv_time_shift
    torch.manual_seed(4)
    h, prev, mix = torch.randn(2, 7, 136).half(), torch.randn(2, 136).half(), torch.rand(3, 1, 136).half()
    ref = rwkv_time_shift(h.float(), prev.float(), mix.float())
    out = rwkv_time_shift(h.cuda(), prev.cuda(), mix.cuda())
    assert torch.allclose(out.float().cpu(), ref, atol=1e-2)
    ref_m = _tiny_rwkv()
    ids = torch.randint(0, 500, (1, 10))
    with torch.no_grad():
        r1 = ref_m(ids[:, :9], use_cache=True)
        r2 = ref_m(ids[:, 9:], state=r1.state, use_cache=True)
    m = optimize_model(_tiny_rwkv(), low_bit="sym_int8").half().cuda()
    with torch.no_grad():
        o1 = m(ids[:, :9].cuda(), use_cache=True)
        o2 = m(ids[:, 9:].cuda(), state=o1.state, use_cache=True)
    for a, b in ((o1, r1), (o2, r2)):
        cos = torch.nn.functional.cosine_similarity(a.logits[:, -1].flatten().float().cpu(), b.logits[:, -1].flatten(),
                                                    dim=0)
        assert cos.item() > 0.99, cos.item()
