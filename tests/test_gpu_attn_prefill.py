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


def _reference_ext(q, k, v, scale, causal, softcap, window, lo):
    B, Hq, S, D = q.shape
    n_rep = Hq // k.shape[1]
    kk = k.float().repeat_interleave(n_rep, dim=1)
    vv = v.float().repeat_interleave(n_rep, dim=1)
    w = torch.matmul(q.float(), kk.transpose(2, 3)) * scale
    if softcap:
        w = torch.tanh(w / softcap) * softcap
    qi = torch.arange(S, device=q.device).view(1, 1, S, 1)
    ki = torch.arange(S, device=q.device).view(1, 1, 1, S)
    ok = torch.ones(B, 1, S, S, dtype=torch.bool, device=q.device)
    if causal:
        ok = ok & (ki <= qi)
    if window:
        ok = ok & (ki > qi - window)
    if lo is not None:
        ok = ok & (ki >= lo.view(B, 1, 1, 1))
    w = w.masked_fill(~ok, float("-inf"))
    p = torch.softmax(w, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)        # rows that see nothing (padding queries)
    return torch.matmul(p, vv), ok


@pytest.mark.parametrize("cfg", [
    # B, Hq, Hkv, S, D, causal, softcap, window, left padding per row
    (1, 4, 2, 300, 128, True, 50.0, 0, None),            # Gemma-2 soft-cap
    (2, 4, 4, 700, 64, True, 0.0, 256, None),            # sliding window shorter than the prompt: key blocks skipped
    (1, 8, 2, 512, 128, True, 30.0, 128, None),          # both
    (3, 4, 2, 400, 128, True, 0.0, 0, (0, 37, 290)),     # left-padded batch (a whole key block of padding in row 2)
    (2, 4, 2, 333, 64, True, 20.0, 100, (5, 200)),       # everything at once
    (2, 2, 2, 260, 128, False, 0.0, 0, (0, 131)),        # bidirectional with padding
])
def test_attn_prefill_softcap_window_padding(cfg):
    """Soft-capped, sliding-window and left-padded prompts on the tcgen05 kernel against an fp32 reference."""
    from ipex_llm_b200.ops import cuda_ops
    B, Hq, Hkv, S, D, causal, softcap, window, pad = cfg
    torch.manual_seed(S + D)
    qkv = torch.randn(B, S, Hq + 2 * Hkv, D, device="cuda").half()
    q = qkv[:, :, :Hq].transpose(1, 2)
    k = qkv[:, :, Hq:Hq + Hkv].transpose(1, 2)
    v = qkv[:, :, Hq + Hkv:].transpose(1, 2)
    scale = 1.0 / math.sqrt(D)
    lo = torch.tensor(pad, dtype=torch.int32, device="cuda") if pad is not None else None
    out = cuda_ops.attn_prefill_tcgen05(q, k, v, scale, causal, softcap, window, lo)
    torch.cuda.synchronize()
    cuda_ops.check_error_flag(q.device)
    ref, ok = _reference_ext(q, k, v, scale, causal, softcap, window, lo)
    real = torch.ones(B, 1, S, 1, dtype=torch.bool, device="cuda")
    if lo is not None:
        real = torch.arange(S, device="cuda").view(1, 1, S, 1) >= lo.view(B, 1, 1, 1)
    err = ((out.float() - ref) * real).abs().max().item()
    assert err < 6e-3, (cfg, err)
    assert (out.float() * ~real).abs().max().item() == 0.0          # padding queries produce zeros

    # the dispatcher recognises the same cases from a model-style call (4-D mask for the padded batch)
    mask = None
    if lo is not None:
        mask = torch.zeros(B, 1, S, S, device="cuda", dtype=torch.float16).masked_fill(~ok, torch.finfo(torch.float16).min)
        found = cuda_ops.left_pad_mask_bounds(mask, S, window)
        assert found is not None and torch.equal(found[0], lo) and found[1] == causal
    out2 = cuda_ops.sdpa_prefill(q, k, v, mask, scale, softcap or None, window or None, causal=causal)
    assert ((out2.float() - ref) * real).abs().max().item() < 6e-3
    assert out2.transpose(1, 2).is_contiguous()                      # came from the kernel, not the eager path


def test_irregular_mask_is_not_taken_for_padding():
    from ipex_llm_b200.ops import cuda_ops
    S = 130
    m = torch.ones(1, 1, S, S, dtype=torch.bool, device="cuda").tril()
    m[0, 0, 100, 50] = False                    # a hole: not a left-padding mask
    assert cuda_ops.left_pad_mask_bounds(m, S) is None


@pytest.mark.parametrize("D", [80, 96])
def test_head_dims_between_kernel_sizes_are_padded(D):
    """Head dims 80 / 96 (Phi-2, StableLM-3B, Phi-3-mini) run on the tcgen05 kernel through a zero-padded copy."""
    from ipex_llm_b200.ops import cuda_ops
    B, Hq, Hkv, S = 2, 8, 4, 200
    torch.manual_seed(D)
    q = torch.randn(B, Hq, S, D, device="cuda").half()
    k = torch.randn(B, Hkv, S, D, device="cuda").half()
    v = torch.randn(B, Hkv, S, D, device="cuda").half()
    scale = 1.0 / math.sqrt(D)
    out = cuda_ops.sdpa_prefill(q, k, v, None, scale, None, None, causal=True)
    torch.cuda.synchronize()
    cuda_ops.check_error_flag(q.device)
    ref = _reference(q, k, v, scale, True)
    assert out.shape == ref.shape
    assert (out.float() - ref).abs().max().item() < 4e-3
