"""Chained-GEMV persistent kernel: o_proj -> gate/up(+act) -> down -> next projection in one launch, against the same
ops computed in fp32 from the dequantized weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(N, K, seed):
    from ipex_llm_b200.ops import cuda_ops
    from ipex_llm_b200.ops.cuda_quant import quantize_to_device_layout
    from ipex_llm_b200.quant import qtypes as qt
    q = qt.qtype_from_name("sym_int4")
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.03
    packed = quantize_to_device_layout(w.half(), q)
    return packed, cuda_ops.dequantize_device(packed, (N, K), q, torch.float32)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M", [1, 3])
@pytest.mark.parametrize("dims", [(512, 1408, 768), (4096, 11008, 12288)])
def test_chain_matches_reference(dtype, M, dims):
    from ipex_llm_b200.engine.decoder_engine import _W, _interleave_row_tiles
    from ipex_llm_b200.native import cuda_api as api
    from ipex_llm_b200.ops import cuda_ops
    from ipex_llm_b200.quant import qtypes as qt
    H, I, NQ = dims
    q = qt.qtype_from_name("sym_int4")
    po, do = _mk(H, H, 1)
    pg, dg = _mk(I, H, 2)
    pu, du = _mk(I, H, 3)
    pd, dd = _mk(H, I, 4)
    pq, dq = _mk(NQ, H, 5)
    gate_up = _interleave_row_tiles(_W(pg, api.WF_SYM_INT4, q, I, H), _W(pu, api.WF_SYM_INT4, q, I, H))
    torch.manual_seed(0)
    attn = torch.randn(M, H, device="cuda").to(dtype)
    h0 = torch.randn(M, H, device="cuda").to(dtype)
    ln2 = (1 + 0.1 * torch.randn(H, device="cuda")).to(dtype)
    ln1 = (1 + 0.1 * torch.randn(H, device="cuda")).to(dtype)
    eps = 1e-5
    h1 = torch.zeros(M, H, device="cuda", dtype=dtype)
    act = torch.zeros(M, I, device="cuda", dtype=dtype)
    h0_out = h0.clone()
    qkv = torch.zeros(M, NQ, device="cuda", dtype=dtype)
    ops = [dict(w=po, x=attn, y=h1, N=H, K=H, residual=h0_out),
           dict(w=gate_up.data, x=h1, y=act, N=2 * I, K=H, norm_w=ln2, act=1, eps=eps),
           dict(w=pd, x=act, y=h0_out, N=H, K=I, residual=h1),
           dict(w=pq, x=h0_out, y=qkv, N=NQ, K=H, norm_w=ln1, eps=eps)]

    def rms(x, w):
        xf = x.float()
        return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()

    # reference follows the same rounding points (every op output is stored in `dtype`)
    r1 = (attn.float() @ do.t() + h0.float()).to(dtype)
    n1 = rms(r1, ln2)
    ra = (torch.nn.functional.silu(n1 @ dg.t()) * (n1 @ du.t())).to(dtype)
    r0 = (ra.float() @ dd.t() + r1.float()).to(dtype)
    rq = (rms(r0, ln1) @ dq.t()).to(dtype)

    for rep in range(3):                      # repeated launches: barrier counters and rings are per-launch state
        h0_out.copy_(h0)
        cuda_ops.gemv_chain(ops, M, dtype, attn.device)
    torch.cuda.synchronize()
    cuda_ops.check_error_flag(attn.device)
    assert int(cuda_ops.chain_barrier(attn.device).abs().sum()) == 0

    def rel(a, b):
        return (a.float() - b.float()).abs().max().item() / max(1e-6, b.float().abs().max().item())
    tol = 6e-3 if dtype == torch.float16 else 3e-2
    assert rel(h1, r1) < tol and rel(act, ra) < tol and rel(h0_out, r0) < tol and rel(qkv, rq) < tol, \
        (rel(h1, r1), rel(act, ra), rel(h0_out, r0), rel(qkv, rq))
