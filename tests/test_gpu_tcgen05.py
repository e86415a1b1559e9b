"""tcgen05 GEMM kernels against fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel_err(a, b):
    return (a.float() - b.float()).abs().max().item() / max(1e-6, b.float().abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [
    # M, N, K
    (17, 128, 64),          # one tile, one k block, ragged tokens
    (32, 256, 512),
    (100, 384, 1024),       # token tile 128 with a ragged edge
    (300, 1000, 4096),      # N not a multiple of 128, two token tiles
    (1024, 4096, 4096),     # many tiles per CTA: both accumulators and every stage wrap
    (2048, 512, 72),        # K with a ragged last block (K % 64 != 0)
])
def test_gemm_dense(dtype, shape):
    from ipex_llm_b200.ops import cuda_ops, tcgen05_gemm
    M, N, K = shape
    torch.manual_seed(M + N + K)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dtype)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(dtype)
    ref = x.float() @ w.float().t()
    out = tcgen05_gemm.gemm_dense(x, w)
    torch.cuda.synchronize()
    cuda_ops.check_error_flag(x.device)
    tol = 2e-3 if dtype == torch.float16 else 1e-2
    assert _rel_err(out, ref) < tol
    # twice in a row on the same buffers: barriers and TMEM are per-launch state
    out2 = tcgen05_gemm.gemm_dense(x, w)
    assert torch.equal(out, out2)


def test_gemm_dense_bias_residual_strided():
    from ipex_llm_b200.ops import cuda_ops, tcgen05_gemm
    torch.manual_seed(3)
    M, N, K = 200, 640, 1536
    xb = (torch.randn(M, K + 64, device="cuda") * 0.5).half()
    x = xb[:, :K]                                   # row stride K + 64
    w = (torch.randn(N, K, device="cuda") * 0.05).half()
    bias = torch.randn(N, device="cuda").half()
    res = torch.randn(M, N, device="cuda").half()
    ref = x.float() @ w.float().t() + bias.float() + res.float()
    out = tcgen05_gemm.gemm_dense(x, w, bias=bias, residual=res)
    torch.cuda.synchronize()
    cuda_ops.check_error_flag(x.device)
    assert _rel_err(out, ref) < 3e-3


TILED = ["sym_int4", "asym_int4", "nf4", "fp4", "fp8_e4m3", "fp8_e5m2", "sym_int8"]


@pytest.mark.parametrize("name", TILED)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(40, 144, 256), (300, 1008, 1024), (1024, 4096, 4096)])
def test_gemm_lowbit_vs_dequantized(name, dtype, shape):
    """In-kernel dequantization: compare with fp32 matmul over the weights the tile dequantizer produces."""
    from ipex_llm_b200.ops import cuda_ops, tcgen05_gemm
    from ipex_llm_b200.ops.cuda_quant import quantize_to_device_layout
    from ipex_llm_b200.quant import qtypes as qt
    M, N, K = shape
    if shape[0] == 1024 and name not in ("sym_int4", "fp8_e4m3", "nf4"):
        pytest.skip("large shape covered by three families")
    q = qt.qtype_from_name(name)
    torch.manual_seed(N + K)
    w = torch.randn(N, K, device="cuda") * 0.05
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dtype)
    packed = quantize_to_device_layout(w.half(), q)
    deq = cuda_ops.dequantize_device(packed, (N, K), q, torch.float32)
    assert tcgen05_gemm.supported(M, N, K, q)
    out = tcgen05_gemm.gemm_lowbit(x, packed, q, N, K)
    torch.cuda.synchronize()
    cuda_ops.check_error_flag(x.device)
    ref = x.float() @ deq.t()
    # the kernel rounds each dequantized weight (and its scale) to the activation dtype before the MMA
    tol = 4e-3 if dtype == torch.float16 else 1.5e-2
    assert _rel_err(out, ref) < tol, (name, dtype, _rel_err(out, ref))
    out2 = tcgen05_gemm.gemm_lowbit(x, packed, q, N, K)
    assert torch.equal(out, out2)


def test_gemm_lowbit_bias_residual_and_gate_up_act():
    from ipex_llm_b200.engine.decoder_engine import _W, _interleave_row_tiles
    from ipex_llm_b200.ops import cuda_ops, tcgen05_gemm
    from ipex_llm_b200.ops.cuda_quant import quantize_to_device_layout
    from ipex_llm_b200.quant import qtypes as qt
    torch.manual_seed(5)
    M, N, K = 150, 512, 768
    q = qt.qtype_from_name("sym_int4")
    x = (torch.randn(M, K, device="cuda") * 0.5).half()
    wg, wu = torch.randn(N, K, device="cuda") * 0.05, torch.randn(N, K, device="cuda") * 0.05
    pg, pu = quantize_to_device_layout(wg.half(), q), quantize_to_device_layout(wu.half(), q)
    dg = cuda_ops.dequantize_device(pg, (N, K), q, torch.float32)
    du = cuda_ops.dequantize_device(pu, (N, K), q, torch.float32)
    # bias + residual
    bias, res = torch.randn(N, device="cuda").half(), torch.randn(M, N, device="cuda").half()
    out = tcgen05_gemm.gemm_lowbit(x, pg, q, N, K, bias=bias, residual=res)
    assert _rel_err(out, x.float() @ dg.t() + bias.float() + res.float()) < 4e-3
    # silu(gate) * up over 16-row-interleaved tiles
    wf = cuda_ops.QTYPE_TO_WF[q]
    merged = _interleave_row_tiles(_W(pg, wf, q, N, K), _W(pu, wf, q, N, K))
    out = tcgen05_gemm.gemm_lowbit(x, merged.data, q, 2 * N, K, act=1)
    g = x.float() @ dg.t()
    ref = torch.nn.functional.silu(g) * (x.float() @ du.t())
    assert out.shape == (M, N)
    assert _rel_err(out, ref) < 6e-3
    cuda_ops.check_error_flag(x.device)


def test_dense_linear_routes_to_tcgen05():
    from ipex_llm_b200.ops import cuda_ops
    torch.manual_seed(4)
    x = torch.randn(64, 1024, device="cuda").half()
    w = (torch.randn(768, 1024, device="cuda") * 0.05).half()
    out = cuda_ops.dense_linear(x, w)
    assert _rel_err(out, x.float() @ w.float().t()) < 2e-3


@pytest.mark.parametrize("dequant_min_tokens", ["100000", "1"])
@pytest.mark.parametrize("low_bit", ["sym_int4", "fp8_e4m3"])
def test_flat_prefill_matches_module_path(low_bit, dequant_min_tokens, monkeypatch):
    """The engine's flattened prompt pass (tcgen05 GEMMs with fused residual / act) against the module-tree pass,
    with the dequantizer warps in the GEMM and with the weight expanded once in front of the dense kernel."""
    monkeypatch.setenv("IPEX_LLM_PREFILL_DEQUANT_MIN_TOKENS", dequant_min_tokens)
    from transformers import LlamaConfig
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.engine import get_engine
    cfg = LlamaConfig(hidden_size=512, intermediate_size=1408 if low_bit == "sym_int4" else 1536, num_hidden_layers=2,
                      num_attention_heads=8, num_key_value_heads=2, vocab_size=2000, max_position_embeddings=512,
                      tie_word_embeddings=False)
    # unquantized KV cache: the module path attends over what the cache returns (e5m2-rounded when quantized), the
    # flat path over the exact K/V of the prompt, so only with a half-precision cache are the two comparable
    monkeypatch.setenv("IPEX_LLM_QUANTIZE_KV_CACHE", "0")
    model = AutoModelForCausalLM.from_config(cfg, load_in_low_bit=low_bit, device="cuda", torch_dtype=torch.float16)
    ids = torch.randint(0, 2000, (2, 37), device="cuda")
    eng = get_engine(model, 2, 128)
    if not eng._flat_prefill_ok():
        pytest.skip("shapes outside the flat path")
    flat = eng.prefill(ids).float()
    k_flat = eng.cache.layers[1].keys.clone()
    monkeypatch.setenv("IPEX_LLM_FLAT_PREFILL", "0")
    eng._flat_ok = None
    ref = eng.prefill(ids).float()
    k_ref = eng.cache.layers[1].keys
    cos = torch.nn.functional.cosine_similarity(flat.flatten(), ref.flatten(), dim=0).item()
    assert cos > 0.9995, cos
    assert k_flat.shape == k_ref.shape
    if k_flat.dtype == torch.uint8:
        assert (k_flat != k_ref).float().mean().item() < 0.02      # e5m2 codes may differ by rounding ties
    else:
        assert torch.allclose(k_flat.float(), k_ref.float(), atol=2e-2)
    # decoding continues from the flat pass
    eng._flat_ok = None
    monkeypatch.delenv("IPEX_LLM_FLAT_PREFILL")
    out = model.generate(ids, max_new_tokens=5, do_sample=False)
    assert out.shape == (2, 42)
