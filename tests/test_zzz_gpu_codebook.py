"""Code-book weights on the GPU: the search and the look-up are tensor code that runs where the weight is; the
product then goes through the dense kernels.  Compared against the CPU codec and an fp32 PyTorch product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["gguf_iq2_xxs", "gguf_iq2_xs", "gguf_iq1_s", "gguf_iq1_m"])
def test_codebook_linear_on_gpu(name):
    pytest.importorskip("gguf.quants")
    from ipex_llm_b200.ops.linear import LowBitLinear
    from ipex_llm_b200.quant import iq_codebooks as iq, qtypes as qt
    from ipex_llm_b200.quant.params import FP4Params
    q = qt.qtype_from_name(name)
    torch.manual_seed(0)
    w = torch.randn(96, 512)
    # the search gives the same quality wherever it runs (near-ties between grid entries may fall differently between
    # the two matmul implementations, so bytes are not compared)
    on_cpu = iq.quantize(w, q)
    on_gpu = iq.quantize(w.cuda(), q)
    assert on_gpu.is_cuda and on_gpu.numel() == on_cpu.numel()
    err_cpu = ((iq.dequantize(on_cpu, w.shape, q) - w).norm() / w.norm()).item()
    err_gpu = ((iq.dequantize(on_gpu, w.shape, q).cpu() - w).norm() / w.norm()).item()
    assert abs(err_gpu - err_cpu) < 0.02 and err_gpu < 0.5, (err_cpu, err_gpu)
    # the decoder itself is exact: the same bytes decode to the same values on both devices
    assert torch.allclose(iq.dequantize(on_cpu.cuda(), w.shape, q).cpu(), iq.dequantize(on_cpu, w.shape, q), atol=1e-6)
    low = LowBitLinear(512, 96, q, bias=False)
    low._parameters["weight"] = FP4Params(w.clone(), qtype=q, in_features=512).to("cuda")
    assert low.weight.data.is_cuda and low.weight.data.numel() == 96 * 2 * iq.TYPE_SIZE[q]
    for rows in (1, 40):
        x = torch.randn(rows, 512, device="cuda", dtype=torch.float16)
        want = x.float() @ low.weight.dequantize(torch.float32).t()
        got = low(x).float()
        assert torch.allclose(got, want, atol=0.05 * want.abs().max().item()), rows
    back = low.weight.to("cpu")
    assert torch.equal(back.data.view(torch.uint8), low.weight.data.cpu().view(torch.uint8))
