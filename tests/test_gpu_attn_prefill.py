"""tcgen05 prompt attention against an fp32 PyTorch reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(q, k, v, scale, causal):
    B, Hq, S, D = q.shape
    n_rep = Hq // k.shape[1]
    kk = k.float().repeat_interleave(n_rep, dim=1)
    vv = v.float().repeat_interleave(n_rep, dim=1)
    w = torch.matmul(q.float(), kk.transpose(2, 3)) * scale
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        w = w.masked_fill(~mask, float("-inf"))
    return torch.matmul(torch.softmax(w, dim=-1), vv)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cfg", [
    # B, Hq, Hkv, S, D, causal
    (1, 4, 4, 128, 128, True),       # one block
    (1, 2, 2, 64, 64, True),         # half a block, head dim 64
    (2, 8, 2, 300, 128, True),       # ragged blocks that run into the next sequence, grouped-query heads
    (1, 4, 4, 1024, 64, True),       # many key blocks: every barrier wraps, both K/V stages reused
    (2, 4, 2, 259, 128, False),      # bidirectional, length not a multiple of 8 (padded V^T)
    (1, 32, 32, 1024, 128, True),    # the 7B prompt shape
])
def test_attn_prefill_tcgen05(dtype, cfg):
    from ipex_llm_b200.ops import cuda_ops
    B, Hq, Hkv, S, D, causal = cfg
    torch.manual_seed(S + D + Hq)
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device="cuda").to(dtype)
    q = qkv[:, :, :Hq].transpose(1, 2)
    k = qkv[:, :, Hq:Hq + Hkv].transpose(1, 2)
    v = qkv[:, :, Hq + Hkv:].transpose(1, 2)
    scale = 1.0 / math.sqrt(D)
    assert cuda_ops._token_major(q) and cuda_ops._token_major(k)
    out = cuda_ops.attn_prefill_tcgen05(q, k, v, scale, causal)
    torch.cuda.synchronize()
    cuda_ops.check_error_flag(q.device)
    ref = _reference(q, k, v, scale, causal)
    assert out.shape == ref.shape
    tol = 4e-3 if dtype == torch.float16 else 2e-2
    err = (out.float() - ref).abs().max().item()
    assert err < tol, (cfg, err)
    out2 = cuda_ops.attn_prefill_tcgen05(q, k, v, scale, causal)
    assert torch.equal(out, out2)


def test_sdpa_prefill_routes_to_tcgen05(monkeypatch):
    from ipex_llm_b200.ops import cuda_ops
    monkeypatch.setenv("IPEX_LLM_TCGEN05_ATTN", "1")
    torch.manual_seed(0)
    qkv = torch.randn(1, 200, 12, 128, device="cuda").half()
    q, k, v = qkv[:, :, :8].transpose(1, 2), qkv[:, :, 8:10].transpose(1, 2), qkv[:, :, 10:].transpose(1, 2)
    assert cuda_ops.attn_prefill_tcgen05_ok(q, k, v)
    out = cuda_ops.sdpa_prefill(q, k, v, None, 0.1, None, None, causal=True)
    assert out.transpose(1, 2).is_contiguous()          # the [B, S, Hq, D] buffer of the kernel
    ref = _reference(q, k, v, 0.1, True)
    assert (out.float() - ref).abs().max().item() < 4e-3
    # contiguous [B, H, S, D] inputs are not token-major: library path
    assert not cuda_ops.attn_prefill_tcgen05_ok(q.contiguous(), k.contiguous(), v)
