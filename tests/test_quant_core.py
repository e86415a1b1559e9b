"""Host quantization core: golden formulas, block geometry, layout round trips, CPU matmul oracle."""
import pytest
import torch

from ipex_llm_b200.quant import qtypes as qt
from ipex_llm_b200.quant.params import (FP4Params, device_nbytes, get_block_size, get_type_size,
                                         ggml_convert_fp32, ggml_convert_qtype, ggml_matmul_src1_x_src0_t,
                                         ggml_q_format_convet_cpu2xpu, ggml_q_format_convet_xpu2cpu)

ALL = ["sym_int4", "asym_int4", "sym_int5", "asym_int5", "sym_int8", "nf4", "nf3", "fp4", "fp6", "fp8_e4m3",
       "fp8_e5m2", "q2_k", "q4_k", "q5_k", "q6_k"]
EXPECTED_GEOMETRY = {"sym_int4": (64, 34), "asym_int4": (64, 36), "sym_int5": (32, 22), "asym_int5": (32, 24),
                     "sym_int8": (64, 66), "nf4": (64, 34), "fp8_e4m3": (128, 132), "q4_k": (256, 144),
                     "q6_k": (256, 210)}
MAX_REL_ERR = {"sym_int4": 0.12, "asym_int4": 0.11, "sym_int5": 0.06, "asym_int5": 0.05, "sym_int8": 0.01,
               "nf4": 0.11, "nf3": 0.23, "fp4": 0.13, "fp6": 0.07, "fp8_e4m3": 0.04, "fp8_e5m2": 0.07,
               "q2_k": 0.40, "q4_k": 0.10, "q5_k": 0.05, "q6_k": 0.03}


def test_qtype_ids_match_reference_table():
    assert qt.ggml_tensor_qtype["sym_int4"] == 2 and qt.ggml_tensor_qtype["asym_int4"] == 3
    assert qt.ggml_tensor_qtype["nf4"] == 10 and qt.ggml_tensor_qtype["fp8_e4m3"] == 15
    assert qt.ggml_tensor_qtype["fp8"] == qt.ggml_tensor_qtype["fp8_e5m2"] == 19
    assert qt.ggml_tensor_qtype["fp6"] == 29 and qt.ggml_tensor_qtype["woq_int4"] == 34
    assert qt.gguf_mixed_qtype == {"gguf_q4k_s": 101, "gguf_q4k_m": 102}
    assert len(qt.ggml_tensor_qtype) == 29 and len(set(qt.ggml_tensor_qtype.values())) == 28


@pytest.mark.parametrize("name", list(EXPECTED_GEOMETRY))
def test_block_geometry(name):
    q = qt.qtype_from_name(name)
    assert (get_block_size(q), get_type_size(q)) == EXPECTED_GEOMETRY[name]


def _torch_q4_0(t):
    """ggml q4_0 with QK=64, the formula the reference documents in utils/convert_chatglm.py."""
    t = t.view(-1, 64)
    idx = t.abs().max(dim=-1, keepdim=True).indices
    mx = torch.take_along_dim(t, idx, dim=-1)
    scale = mx / -8
    q = (t / scale + 8).round().clamp(0, 15).to(torch.uint8)
    packed = q[:, :32] | (q[:, 32:] << 4)
    return torch.cat((scale.half().view(torch.uint8), packed), dim=-1)


def _torch_q4_1(t):
    t = t.view(-1, 64)
    mn, mx = t.min(dim=-1, keepdim=True).values, t.max(dim=-1, keepdim=True).values
    scale = (mx - mn) / 15
    q = ((t - mn) / scale).round().clamp(0, 15).to(torch.uint8)
    packed = q[:, :32] | (q[:, 32:] << 4)
    return torch.cat((scale.half().view(torch.uint8), mn.half().view(torch.uint8), packed), dim=-1)


def _torch_q8_0(t):
    t = t.view(-1, 64)
    scale = t.abs().max(dim=-1, keepdim=True).values / 127
    q = (t / scale).round().clamp(-128, 127).to(torch.int8)
    return torch.cat((scale.half().view(torch.uint8), q.view(torch.uint8)), dim=-1)


@pytest.mark.parametrize("name,fn", [("sym_int4", _torch_q4_0), ("asym_int4", _torch_q4_1), ("sym_int8", _torch_q8_0)])
def test_golden_vs_torch_formula(name, fn):
    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.02
    ours = ggml_convert_qtype(w, qt.qtype_from_name(name)).view(-1, get_type_size(qt.qtype_from_name(name)))
    gold = fn(w.clone())
    hdr = 4 if name == "asym_int4" else 2
    assert torch.equal(ours[:, :hdr], gold[:, :hdr])          # scales (and mins) bit exact
    # codes: x*(1/d)+8.5 truncation (ggml) vs round(x/d+8) (torch) may differ by one step on exact ties only
    if name == "sym_int8":
        diff = (ours[:, hdr:].view(torch.int8).int() - gold[:, hdr:].view(torch.int8).int()).abs()
        assert diff.max() <= 1 and (diff != 0).float().mean() < 1e-3
    else:
        lo = (ours[:, hdr:] & 0xF).int() - (gold[:, hdr:] & 0xF).int()
        hi = (ours[:, hdr:] >> 4).int() - (gold[:, hdr:] >> 4).int()
        assert lo.abs().max() <= 1 and hi.abs().max() <= 1
        assert ((lo != 0) | (hi != 0)).float().mean() < 2e-3


@pytest.mark.parametrize("name", ALL)
def test_quantize_dequantize_error(name):
    torch.manual_seed(1)
    q = qt.qtype_from_name(name)
    w = torch.randn(32, 512) * 0.02
    packed = ggml_convert_qtype(w, q)
    assert packed.numel() * packed.element_size() == w.numel() // get_block_size(q) * get_type_size(q)
    deq = ggml_convert_fp32(packed.view(torch.uint8), w.shape, w.numel(), q)
    rel = ((deq - w).norm() / w.norm()).item()
    assert rel < MAX_REL_ERR[name], (name, rel)


def test_nf4_is_exposed_as_bf16():
    w = torch.randn(8, 128)
    p = ggml_convert_qtype(w, qt.NF4)
    assert p.dtype == torch.bfloat16 and p.numel() * 2 == 8 * 128 // 64 * 34


@pytest.mark.parametrize("name", ["sym_int4", "asym_int4", "nf4", "fp4", "fp8_e4m3", "fp8_e5m2", "sym_int8", "fp6"])
@pytest.mark.parametrize("shape", [(16, 128), (40, 192), (7, 320), (33, 1024)])
def test_device_layout_roundtrip(name, shape):
    torch.manual_seed(2)
    q = qt.qtype_from_name(name)
    if shape[1] % get_block_size(q):
        pytest.skip("K not a multiple of the block")
    w = torch.randn(*shape)
    packed = ggml_convert_qtype(w, q).view(torch.uint8)
    dev = ggml_q_format_convet_cpu2xpu(packed, shape, q)
    assert dev.numel() == device_nbytes(shape[0], shape[1], q)
    back = ggml_q_format_convet_xpu2cpu(dev, shape, q).view(torch.uint8)
    assert torch.equal(back, packed)


@pytest.mark.parametrize("name", ALL)
def test_cpu_matmul_oracle(name):
    torch.manual_seed(3)
    q = qt.qtype_from_name(name)
    w = torch.randn(24, 512) * 0.05
    x = torch.randn(5, 512)
    packed = ggml_convert_qtype(w, q)
    deq = ggml_convert_fp32(packed.view(torch.uint8), w.shape, w.numel(), q)
    y = ggml_matmul_src1_x_src0_t(packed.view(torch.uint8), x, w.shape, q)
    assert torch.allclose(y, x @ deq.t(), atol=1e-4, rtol=1e-4)


def test_mixed_fp4_picks_by_mse():
    torch.manual_seed(4)
    w = torch.randn(16, 128)
    p = FP4Params(w.clone(), qtype=qt.MOFQ4).quantize("cpu")
    assert p.qtype in (qt.SYM_INT4, qt.FP4) and p.quantized
    p8 = FP4Params(w.clone(), qtype=qt.MOFQ8).quantize("cpu")
    assert p8.qtype in (qt.SYM_INT8, qt.FP8E4)


def test_scale_search_and_imatrix_do_not_hurt():
    torch.manual_seed(5)
    w = torch.randn(16, 256) * 0.02
    for name in ("fp8_e4m3", "fp6", "sym_int4"):
        q = qt.qtype_from_name(name)
        base = ggml_convert_fp32(ggml_convert_qtype(w, q).view(torch.uint8), w.shape, w.numel(), q)
        srch = ggml_convert_fp32(ggml_convert_qtype(w, q, enable_scale_search=True).view(torch.uint8), w.shape,
                                 w.numel(), q)
        assert (srch - w).norm() <= (base - w).norm() * 1.001
    im = torch.rand(256) + 0.1
    q = qt.SYM_INT4
    wq = ggml_convert_fp32(ggml_convert_qtype(w, q, imatrix=im, in_features=256).view(torch.uint8), w.shape,
                           w.numel(), q)
    base = ggml_convert_fp32(ggml_convert_qtype(w, q).view(torch.uint8), w.shape, w.numel(), q)
    werr = lambda a: (((a - w) ** 2) * im).sum()  # noqa: E731
    assert werr(wq) <= werr(base) * 1.001


def test_rtn_formats():
    w = torch.randn(8, 64)
    codes, scale = ggml_convert_qtype(w, qt.SYM_INT8_RTN)
    assert codes.shape == (8, 64) and codes.dtype == torch.int8 and scale.shape == (8,)
    assert torch.allclose(codes.float() * scale.float()[:, None], w, atol=w.abs().max().item() / 100)
    codes4, scale4 = ggml_convert_qtype(w, qt.ASYM_INT4_RTN)
    assert codes4.shape == (8, 32) and scale4.shape == (16,)


IQ_CASES = [("gguf_iq2_xxs", 66, 0.36), ("gguf_iq2_xs", 74, 0.32), ("gguf_iq1_s", 50, 0.48), ("gguf_iq1_m", 56, 0.45)]


@pytest.mark.parametrize("name,type_size,max_rel", IQ_CASES)
def test_codebook_formats_round_trip_and_read_like_gguf(name, type_size, max_rel):
    """The four code-book formats: bytes per super-block, error of our quantizer on Gaussian weights, and the packed
    bytes decode to the same values through the `gguf` package's own reader (format compatibility)."""
    gq = pytest.importorskip("gguf.quants")
    from gguf.constants import GGMLQuantizationType as T
    from ipex_llm_b200.quant import iq_codebooks as iq
    from ipex_llm_b200.quant.params import get_block_size, get_type_size
    q = qt.qtype_from_name(name)
    assert get_block_size(q) == 256 and get_type_size(q) == type_size == iq.TYPE_SIZE[q]
    torch.manual_seed(3)
    w = torch.randn(24, 512)
    w[5] = 0                                                    # an all-zero row must survive
    packed = ggml_convert_qtype(w, q)
    assert packed.dtype == torch.uint8 and packed.numel() == 24 * 2 * type_size
    back = ggml_convert_fp32(packed, w.shape, w.numel(), q)
    assert torch.isfinite(back).all() and back[5].abs().max() == 0
    assert ((back - w).norm() / w.norm()).item() < max_rel
    theirs = gq.dequantize(packed.numpy().reshape(24, -1), getattr(T, name[5:].upper()))
    assert torch.equal(back, torch.from_numpy(theirs))


def test_codebook_importance_weights_lower_the_weighted_error():
    pytest.importorskip("gguf.quants")
    torch.manual_seed(4)
    w = torch.randn(16, 512)
    im = torch.rand(512) ** 4 + 1e-3                            # a few columns matter much more than the rest
    for name in ("gguf_iq2_xxs", "gguf_iq1_s"):
        q = qt.qtype_from_name(name)
        plain = ggml_convert_fp32(ggml_convert_qtype(w, q), w.shape, w.numel(), q)
        weighted = ggml_convert_fp32(ggml_convert_qtype(w, q, imatrix=im, in_features=512), w.shape, w.numel(), q)

        def werr(x):
            return float((im * (x - w) ** 2).sum())
        assert werr(weighted) < werr(plain)


def test_codebook_linear_on_cpu():
    """LowBitLinear over a code-book weight: same numbers as the dense product with the dequantized weight, and the
    packed bytes survive a state-dict round trip."""
    pytest.importorskip("gguf.quants")
    from ipex_llm_b200.ops.linear import LowBitLinear
    from ipex_llm_b200.quant.params import FP4Params
    torch.manual_seed(5)
    lin = torch.nn.Linear(256, 48, bias=True)
    q = qt.qtype_from_name("gguf_iq2_xs")
    low = LowBitLinear(256, 48, q, bias=True)
    low._parameters["weight"] = FP4Params(lin.weight.data.clone(), qtype=q, in_features=256).to("cpu")
    low._parameters["bias"] = lin.bias
    x = torch.randn(3, 256)
    want = torch.nn.functional.linear(x, low.weight.dequantize(), lin.bias)
    assert torch.allclose(low(x), want, atol=1e-4)
    many = torch.randn(600, 256)                                # the dequantize-then-dense branch
    assert torch.allclose(low(many), torch.nn.functional.linear(many, low.weight.dequantize(), lin.bias), atol=1e-3)
    assert torch.nn.functional.cosine_similarity(low(x).flatten(), lin(x).flatten(), dim=0) > 0.93
    sd = low.state_dict()
    assert sd["weight"].dtype == torch.uint8 and sd["weight"].numel() == 48 * 74


ALL_BLOCK_FORMATS = ["sym_int4", "asym_int4", "sym_int5", "asym_int5", "sym_int8", "nf4", "nf3", "fp4", "fp6", "fp8_e4m3",
                     "fp8_e5m2", "q2_k", "q4_k", "q5_k", "q6_k", "gguf_iq2_xxs", "gguf_iq2_xs", "gguf_iq1_s",
                     "gguf_iq1_m"]


@pytest.mark.parametrize("name", ALL_BLOCK_FORMATS)
def test_quantizers_survive_degenerate_and_extreme_blocks(name):
    """All-zero, constant, one-hot, denormal, beyond-fp16 and wildly mixed-magnitude rows: every format decodes to
    finite values, zeros stay zeros, and no element is off by more than the largest magnitude of the input (a scale
    beyond the fp16 range saturates, so such a block clips instead of decoding to inf)."""
    if name.startswith("gguf_iq"):
        pytest.importorskip("gguf.quants")
    q = qt.qtype_from_name(name)
    k = 512
    g = torch.Generator().manual_seed(7)
    rnd = torch.randn(2, k, generator=g)
    cases = {
        "zeros": torch.zeros(2, k), "const": torch.full((2, k), 3.0), "negconst": torch.full((2, k), -7.5),
        "one_hot": torch.nn.functional.one_hot(torch.tensor([5, 300]), k).float(),
        "tiny": rnd * 1e-30, "denormal": rnd * 1e-42, "beyond_fp16": rnd * 6e4, "huge": rnd * 1e30,
        "mixed": rnd * torch.exp(torch.rand(2, k, generator=g) * 40 - 20),
        "outlier": torch.cat([rnd[:, :-1], torch.full((2, 1), 1e4)], 1),
    }
    for cname, x in cases.items():
        p = ggml_convert_qtype(x.contiguous(), q)
        y = ggml_convert_fp32(p.view(torch.uint8) if p.dtype != torch.uint8 else p, x.shape, x.numel(), q)
        assert torch.isfinite(y).all(), cname
        amax = x.abs().max().item()
        if amax == 0:
            assert y.abs().max().item() == 0, cname
        else:
            assert (y - x).abs().max().item() <= 1.01 * amax + 1e-38, cname      # (denormal scales lose bits)


@pytest.mark.parametrize("name,type_size,tail_scale", [("gguf_iq2_xxs", 66, False), ("gguf_iq2_xs", 74, False),
                                                        ("gguf_iq1_s", 50, False), ("gguf_iq1_m", 56, None)])
def test_codebook_decoders_on_arbitrary_bytes(name, type_size, tail_scale):
    """Random super-blocks (every bit pattern of indices, signs, scales and shift bits, not only those the quantizer
    emits) decode to exactly what the ``gguf`` package's decoder gives."""
    gq = pytest.importorskip("gguf.quants")
    from gguf.constants import GGMLQuantizationType as T
    from ipex_llm_b200.quant import iq_codebooks as iq
    import numpy as np
    rng = np.random.default_rng(11)
    raw = rng.integers(0, 256, size=(64, type_size), dtype=np.uint8)
    d = np.array([0.0173], dtype=np.float16).view(np.uint8)
    if tail_scale is None:
        # iq1_m spreads its fp16 scale over the top nibbles of four 16-bit words: keep it a small finite number
        words = raw[:, 48:56].copy().view(np.uint16)
        bits = int(np.array([0.0173], dtype=np.float16).view(np.uint16)[0])
        for u in range(4):
            words[:, u] = (words[:, u] & 0x0FFF) | (((bits >> (4 * u)) & 0xF) << 12)
        raw[:, 48:56] = words.view(np.uint8)
    else:
        raw[:, :2] = d
    q = qt.qtype_from_name(name)
    ours = iq.dequantize(torch.from_numpy(raw.reshape(-1)), (64, 256), q)
    theirs = torch.from_numpy(gq.dequantize(raw, getattr(T, name[5:].upper())))
    assert torch.equal(ours, theirs)


@pytest.mark.parametrize("name,type_size,scale_at", [("q2_k", 84, (80, 82)), ("q4_k", 144, (0, 2)), ("q5_k", 176, (0, 2)),
                                                      ("q6_k", 210, (208,))])
def test_kquant_decoders_on_arbitrary_bytes(name, type_size, scale_at):
    """The host library's k-quant decoders against the ``gguf`` package on random super-blocks (all scale / minimum /
    high-bit patterns), i.e. the byte layouts are ggml's."""
    gq = pytest.importorskip("gguf.quants")
    from gguf.constants import GGMLQuantizationType as T
    import numpy as np
    rng = np.random.default_rng(5)
    raw = rng.integers(0, 256, size=(48, type_size), dtype=np.uint8)
    for off, val in zip(scale_at, (0.0131, 0.0077)):
        raw[:, off:off + 2] = np.array([val], dtype=np.float16).view(np.uint8)
    q = qt.qtype_from_name(name)
    ours = ggml_convert_fp32(torch.from_numpy(raw.reshape(-1)), (48, 256), 48 * 256, q)
    theirs = torch.from_numpy(gq.dequantize(raw, getattr(T, name.upper())))
    assert torch.allclose(ours, theirs, atol=1e-6, rtol=1e-6)
