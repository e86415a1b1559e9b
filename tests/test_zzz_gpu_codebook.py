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
    # the same bytes whether the search ran on the CPU or on the GPU
    on_cpu = iq.quantize(w, q)
    on_gpu = iq.quantize(w.cuda(), q)
    same = (on_cpu == on_gpu.cpu()).float().mean().item()
    assert same > 0.9, same                            # ties in the arg-min may fall differently; the values agree
    deq = iq.dequantize(on_gpu, w.shape, q)
    assert ((deq.cpu() - iq.dequantize(on_cpu, w.shape, q)).norm() / w.norm()).item() < 0.05
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
