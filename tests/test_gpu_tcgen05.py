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


def test_dense_linear_routes_to_tcgen05():
    from ipex_llm_b200.ops import cuda_ops
    torch.manual_seed(4)
    x = torch.randn(64, 1024, device="cuda").half()
    w = (torch.randn(768, 1024, device="cuda") * 0.05).half()
    out = cuda_ops.dense_linear(x, w)
    assert _rel_err(out, x.float() @ w.float().t()) < 2e-3
