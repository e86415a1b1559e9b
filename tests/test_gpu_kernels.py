"""GPU numerics: every sm_100a kernel against a plain PyTorch fp32 reference (and the C++ host oracle)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

TILED = ["sym_int4", "asym_int4", "nf4", "fp4", "fp8_e4m3", "fp8_e5m2", "sym_int8"]


def _qt(name):
    from ipex_llm_b200.quant import qtypes as qt
    return qt.qtype_from_name(name)


def _quantize_cpu(w, name):
    """canonical blocks, dequantized fp32 weight, device-layout bytes (via the host library)."""
    from ipex_llm_b200.quant.params import ggml_convert_fp32, ggml_convert_qtype, ggml_q_format_convet_cpu2xpu
    q = _qt(name)
    packed = ggml_convert_qtype(w.float().contiguous(), q)
    raw = packed.view(torch.uint8)
    deq = ggml_convert_fp32(raw, w.shape, w.numel(), q)
    dev = ggml_q_format_convet_cpu2xpu(raw, w.shape, q)
    return packed, deq, dev


@pytest.mark.parametrize("name", TILED)
def test_gpu_quantizer_matches_host(name):
    from ipex_llm_b200.ops.cuda_quant import quantize_to_device_layout
    torch.manual_seed(0)
    N, K = 80, 384
    w = (torch.randn(N, K) * 0.02)
    _, deq, dev_host = _quantize_cpu(w, name)
    dev_gpu = quantize_to_device_layout(w.cuda(), _qt(name)).cpu()
    assert dev_gpu.numel() == dev_host.numel()
    mism = (dev_gpu != dev_host).float().mean().item()
    if name.startswith("fp8"):
        assert mism < 2e-3, mism   # ties round differently (nearest-lower vs nearest-even)
    else:
        assert mism == 0.0, mism


@pytest.mark.parametrize("name", TILED)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dequantize_tiles(name, dtype):
    from ipex_llm_b200.ops.cuda_ops import dequantize_device
    torch.manual_seed(1)
    N, K = 48, 256
    w = torch.randn(N, K) * 0.05
    _, deq, dev = _quantize_cpu(w, name)
    out = dequantize_device(dev.cuda(), (N, K), _qt(name), dtype).float().cpu()
    tol = 2e-3 if dtype == torch.float16 else 1e-2
    assert torch.allclose(out, deq, rtol=tol, atol=tol * deq.abs().max().item())


@pytest.mark.parametrize("name", ["sym_int5", "asym_int5", "nf3", "fp6", "q4_k", "q5_k", "q6_k", "q2_k"])
def test_dequantize_blocks(name):
    from ipex_llm_b200.ops.cuda_ops import dequantize_device
    from ipex_llm_b200.quant.params import ggml_convert_fp32, ggml_convert_qtype
    torch.manual_seed(2)
    N, K = 16, 512
    w = torch.randn(N, K) * 0.05
    q = _qt(name)
    packed = ggml_convert_qtype(w, q)
    deq = ggml_convert_fp32(packed, w.shape, w.numel(), q)
    out = dequantize_device(packed.cuda(), (N, K), q, torch.float32).cpu()
    assert torch.allclose(out, deq, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("name", TILED)
@pytest.mark.parametrize("M", [1, 2, 7, 8])
@pytest.mark.parametrize("shape", [(48, 256), (4096 + 16, 1024), (688, 4096)])
def test_gemv_lowbit_vs_oracle(name, M, shape):
    from ipex_llm_b200.ops.cuda_ops import gemv_lowbit
    torch.manual_seed(3)
    N, K = shape
    w = torch.randn(N, K) * 0.02
    _, deq, dev = _quantize_cpu(w, name)
    x = torch.randn(M, K)
    for dtype in (torch.float16, torch.bfloat16):
        xd = x.to(dtype).cuda()
        ref = xd.float().cpu() @ deq.t()
        y = gemv_lowbit(xd, dev.cuda(), _qt(name), N, K).float().cpu()
        tol = 4e-3 if dtype == torch.float16 else 2e-2
        err = (y - ref).abs().max().item() / ref.abs().max().item()
        assert err < tol, (name, M, shape, dtype, err)


def test_gemv_fused_norm_bias_residual_act():
    from ipex_llm_b200.ops.cuda_ops import gemv_lowbit
    from ipex_llm_b200.engine.decoder_engine import _W, _interleave_row_tiles
    from ipex_llm_b200.native import cuda_api as api
    torch.manual_seed(4)
    K, I, M = 512, 704, 3
    x = torch.randn(M, K)
    gamma = 1.0 + 0.1 * torch.randn(K)
    wg, wu = torch.randn(I, K) * 0.03, torch.randn(I, K) * 0.03
    _, dg, devg = _quantize_cpu(wg, "sym_int4")
    _, du, devu = _quantize_cpu(wu, "sym_int4")
    q = _qt("sym_int4")
    xd = x.half().cuda()
    xn = xd.float().cpu()
    xn = xn * torch.rsqrt(xn.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma.half().float()
    # norm + bias + residual
    bias, res = torch.randn(I) * 0.1, torch.randn(M, I)
    ref = xn @ dg.t() + bias.half().float() + res.half().float()
    y = gemv_lowbit(xd, devg.cuda(), q, I, K, norm_weight=gamma.half().cuda(), eps=1e-6, bias=bias.half().cuda(),
                    residual=res.half().cuda()).float().cpu()
    assert (y - ref).abs().max().item() < 2e-2 * ref.abs().max().item()
    # fused SwiGLU on interleaved gate/up tiles
    a = _W(devg.cuda(), api.WF_SYM_INT4, q, I, K)
    b = _W(devu.cuda(), api.WF_SYM_INT4, q, I, K)
    gu = _interleave_row_tiles(a, b)
    g, u = xn @ dg.t(), xn @ du.t()
    ref2 = torch.nn.functional.silu(g) * u
    y2 = gemv_lowbit(xd, gu.data, q, 2 * I, K, norm_weight=gamma.half().cuda(), eps=1e-6, act=1).float().cpu()
    assert y2.shape == (M, I)
    assert (y2 - ref2).abs().max().item() < 2e-2 * ref2.abs().max().item() + 1e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemv_dense(dtype):
    from ipex_llm_b200.ops.cuda_ops import dense_linear
    torch.manual_seed(5)
    for (M, N, K) in [(1, 100, 688), (5, 4096, 1024)]:
        x = torch.randn(M, K).to(dtype).cuda()
        w = (torch.randn(N, K) * 0.05).to(dtype).cuda()
        ref = x.float() @ w.float().t()
        y = dense_linear(x, w).float()
        assert (y - ref).abs().max().item() < 1e-2 * ref.abs().max().item()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M", [1, 7])
def test_gemv_dense_norm_residual_act(dtype, M):
    """Dense half weights with the fused RMSNorm prologue (vector and scalar staging), residual and SwiGLU."""
    from ipex_llm_b200.engine.decoder_engine import _W, _interleave_row_tiles
    from ipex_llm_b200.native import cuda_api as api
    from ipex_llm_b200.ops.cuda_ops import gemv_lowbit
    torch.manual_seed(8)
    K, I = 1040, 608
    wf = api.WF_F16 if dtype == torch.float16 else api.WF_BF16
    xb = torch.randn(M, K + 3).to(dtype).cuda()
    gamma = (1.0 + 0.1 * torch.randn(K)).to(dtype).cuda()
    wg = (torch.randn(I, K) * 0.03).to(dtype).cuda()
    wu = (torch.randn(I, K) * 0.03).to(dtype).cuda()
    res = torch.randn(M, I).to(dtype).cuda()
    tol = 6e-3 if dtype == torch.float16 else 3e-2
    for x in (xb[:, :K].contiguous(), xb[:, :K]):          # aligned rows, then a row stride of K + 3 elements
        xf = x.float()
        xn = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float()
        xn = xn.to(dtype).float()
        ref = xn @ wg.float().t() + res.float()
        y = gemv_lowbit(x, wg, None, I, K, norm_weight=gamma, eps=1e-5, residual=res, wf=wf).float()
        assert (y - ref).abs().max().item() < tol * ref.abs().max().item()
        gu = _interleave_row_tiles(_W(wg, wf, None, I, K), _W(wu, wf, None, I, K))
        ref2 = torch.nn.functional.silu(xn @ wg.float().t()) * (xn @ wu.float().t())
        y2 = gemv_lowbit(x, gu.data, None, 2 * I, K, norm_weight=gamma, eps=1e-5, act=1, wf=wf).float()
        assert y2.shape == (M, I)
        assert (y2 - ref2).abs().max().item() < tol * ref2.abs().max().item() + 1e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_norms_act_softmax(dtype):
    from ipex_llm_b200.ops import cuda_ops
    torch.manual_seed(6)
    x = torch.randn(5, 4096).to(dtype).cuda()
    w = (1 + 0.1 * torch.randn(4096)).to(dtype).cuda()
    b = (0.1 * torch.randn(4096)).to(dtype).cuda()
    xf = x.float()
    ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).to(dtype).float() * w.float()
    assert torch.allclose(cuda_ops.rms_norm(x, w, 1e-5).float(), ref, atol=2e-2, rtol=2e-2)
    ref_ln = torch.nn.functional.layer_norm(xf, (4096,), w.float(), b.float(), 1e-5)
    assert torch.allclose(cuda_ops.layer_norm(x, w, b, 1e-5).float(), ref_ln, atol=3e-2, rtol=3e-2)
    g, u = torch.randn(3, 1000).to(dtype).cuda(), torch.randn(3, 1000).to(dtype).cuda()
    assert torch.allclose(cuda_ops.act_mul(g, u, 0).float(), torch.nn.functional.silu(g.float()) * u.float(),
                          atol=2e-2, rtol=2e-2)
    assert torch.allclose(cuda_ops.act_mul(g, u, 1).float(),
                          torch.nn.functional.gelu(g.float(), approximate="tanh") * u.float(), atol=2e-2, rtol=2e-2)
    s = torch.randn(2, 4, 7, 333).to(dtype).cuda()
    ref_s = torch.softmax(s.float(), -1)
    assert torch.allclose(cuda_ops.softmax_inplace(s.clone()).float(), ref_s, atol=1e-2)


@pytest.mark.parametrize("interleaved", [False, True])
def test_rope_inplace(interleaved):
    from ipex_llm_b200.models.common import apply_rotary_pos_emb
    torch.manual_seed(7)
    B, Hq, Hk, S, D = 2, 8, 2, 5, 128
    qkv = torch.randn(B, S, (Hq + 2 * Hk) * D).half().cuda()
    q = qkv[..., : Hq * D].view(B, S, Hq, D).transpose(1, 2)
    k = qkv[..., Hq * D: (Hq + Hk) * D].view(B, S, Hk, D).transpose(1, 2)
    pos = torch.arange(S).float()
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D))
    fr = torch.outer(pos, inv)
    if interleaved:
        emb = fr.repeat_interleave(2, dim=-1)
    else:
        emb = torch.cat([fr, fr], dim=-1)
    cos, sin = emb.cos()[None].expand(B, S, D).cuda(), emb.sin()[None].expand(B, S, D).cuda()
    q_ref, k_ref = apply_rotary_pos_emb(q.float().cpu(), k.float().cpu(), cos.cpu(), sin.cpu(),
                                        interleaved=interleaved)
    q2, k2 = apply_rotary_pos_emb(q, k, cos, sin, interleaved=interleaved)
    assert torch.allclose(q2.float().cpu(), q_ref, atol=1e-2)
    assert torch.allclose(k2.float().cpu(), k_ref, atol=1e-2)


def test_kv_e5m2_roundtrip():
    from ipex_llm_b200.ops import cuda_ops
    torch.manual_seed(8)
    x = (torch.randn(2, 4, 9, 128) * 3).half()
    ref = x.clamp(-57344, 57344).to(torch.float8_e5m2)
    got = cuda_ops.quantize_kv_e5m2(x.cuda()).cpu()
    assert (got != ref.view(torch.uint8)).float().mean().item() == 0.0
    back = cuda_ops.dequantize_kv_e5m2(got.cuda(), torch.float16).cpu()
    assert torch.equal(back, ref.to(torch.float16))


def _ref_attention(q, k, v, scale, causal, softcap=None, window=None):
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    k = k.repeat_interleave(Hq // Hkv, dim=1)
    v = v.repeat_interleave(Hq // Hkv, dim=1)
    w = (q.float() @ k.float().transpose(2, 3)) * scale
    if softcap:
        w = torch.tanh(w / softcap) * softcap
    qi = torch.arange(Skv - Sq, Skv).view(-1, 1)
    ki = torch.arange(Skv).view(1, -1)
    allowed = torch.ones(Sq, Skv, dtype=torch.bool)
    if causal:
        allowed = ki <= qi
    if window:
        allowed = allowed & (ki > qi - window)
    w = w.masked_fill(~allowed.to(w.device), float("-inf"))
    return torch.softmax(w, -1) @ v.float()


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("cfg", [(1, 4, 4, 1, 128, 300), (2, 32, 8, 1, 128, 1100), (1, 8, 8, 9, 64, 77),
                                 (2, 16, 2, 4, 128, 513), (1, 64, 8, 1, 128, 2050), (1, 4, 1, 3, 256, 129)])
def test_attn_decode_module_path(fp8, cfg):
    from ipex_llm_b200.ops import cuda_ops
    torch.manual_seed(9)
    B, Hq, Hkv, Sq, D, Skv = cfg
    for dtype in (torch.float16, torch.bfloat16):
        q = torch.randn(B, Hq, Sq, D).to(dtype).cuda()
        k = torch.randn(B, Hkv, Skv, D).to(dtype).cuda()
        v = torch.randn(B, Hkv, Skv, D).to(dtype).cuda()
        if fp8:
            k8, v8 = cuda_ops.quantize_kv_e5m2(k), cuda_ops.quantize_kv_e5m2(v)
            kr, vr = cuda_ops.dequantize_kv_e5m2(k8, dtype), cuda_ops.dequantize_kv_e5m2(v8, dtype)
            out = cuda_ops.sdpa_decode(q, k8, v8, None, 1 / math.sqrt(D), None, None, causal=True)
        else:
            kr, vr = k, v
            out = cuda_ops.sdpa_decode(q, k, v, None, 1 / math.sqrt(D), None, None, causal=True)
        ref = _ref_attention(q.cpu(), kr.cpu(), vr.cpu(), 1 / math.sqrt(D), True)
        tol = 5e-3 if dtype == torch.float16 else 2e-2
        assert (out.float().cpu() - ref).abs().max().item() < tol, (cfg, dtype, fp8)


def test_attn_decode_softcap_window():
    from ipex_llm_b200.ops import cuda_ops
    torch.manual_seed(10)
    B, Hq, Hkv, Sq, D, Skv = 1, 8, 4, 2, 128, 700
    q = torch.randn(B, Hq, Sq, D).half().cuda()
    k = torch.randn(B, Hkv, Skv, D).half().cuda()
    v = torch.randn(B, Hkv, Skv, D).half().cuda()
    out = cuda_ops.sdpa_decode(q, k, v, None, 0.1, 30.0, 256, causal=True)
    ref = _ref_attention(q.cpu(), k.cpu(), v.cpu(), 0.1, True, softcap=30.0, window=256)
    assert (out.float().cpu() - ref).abs().max().item() < 5e-3


def test_embedding_rows_and_argmax_and_penalty():
    from ipex_llm_b200.ops import cuda_ops
    from ipex_llm_b200.ops.embedding import LowBitEmbedding
    torch.manual_seed(11)
    emb = torch.nn.Embedding(300, 512)
    ids = torch.randint(0, 300, (2, 7))
    for name in ("q4_k", "q2_k", "sym_int4"):
        low = LowBitEmbedding.from_embedding(emb, _qt(name))
        ref = low(ids)
        got = low.to("cuda")(ids.cuda()).cpu()
        assert torch.allclose(got.float(), ref.float(), atol=1e-3), name
    logits = torch.randn(3, 1000).half().cuda()
    ids = torch.randint(0, 1000, (3, 5)).cuda()
    ref = logits.clone().float()
    for b in range(3):
        for t in set(ids[b].tolist()):
            ref[b, t] = ref[b, t] * 1.3 if ref[b, t] < 0 else ref[b, t] / 1.3
    got = cuda_ops.repetition_penalty_inplace(logits.clone(), ids, 1.3)
    assert torch.allclose(got.float(), ref, atol=2e-3, rtol=2e-3)


def test_gemv_non_pipelined_variant_and_wait_flags(monkeypatch):
    """The register-path GEMV stays available (it serves shapes whose x does not fit beside the TMA ring) and no
    bounded wait of the pipelined kernel has expired during the tests above."""
    from ipex_llm_b200.ops import cuda_ops
    torch.manual_seed(12)
    N, K, M = 1040, 2048, 4
    w = torch.randn(N, K) * 0.02
    _, deq, dev = _quantize_cpu(w, "sym_int4")
    x = torch.randn(M, K).half().cuda()
    ref = x.float().cpu() @ deq.t()
    y_tma = cuda_ops.gemv_lowbit(x, dev.cuda(), _qt("sym_int4"), N, K).float().cpu()
    monkeypatch.setattr(cuda_ops, "_GEMV_IMPL", "v1")
    y_v1 = cuda_ops.gemv_lowbit(x, dev.cuda(), _qt("sym_int4"), N, K).float().cpu()
    assert (y_v1 - ref).abs().max().item() < 4e-3 * ref.abs().max().item()
    assert (y_tma - y_v1).abs().max().item() < 2e-3 * ref.abs().max().item()
    torch.cuda.synchronize()
    cuda_ops.check_error_flag(x.device)
