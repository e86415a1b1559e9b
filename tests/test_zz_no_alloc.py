"""Decode attention through the library-owned scratch array (``ipex_attn_decode_noalloc``), called by its exported
C symbol, against the regular entry point (``ipex_attn_decode``) that takes caller-provided work buffers and a
plain fp32 PyTorch restatement.  Collected last on purpose: it must pass alone and after every other GPU test has
used the device."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

c_void_p, c_int, c_float, c_int64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_int64


def _lib():
    from ipex_llm_b200.native.lib import cuda_lib
    lib = cuda_lib()
    f = lib.ipex_attn_decode_noalloc
    f.argtypes = [c_void_p] * 10 + [ctypes.POINTER(c_int64)] + [c_int] * 10 + [c_float, c_float, c_int, c_int, c_int,
                                                                              c_void_p]
    f.restype = c_int
    lib.ipex_attn_decode_noalloc_setup.argtypes = []
    lib.ipex_attn_decode_noalloc_setup.restype = c_int
    lib.ipex_attn_decode_noalloc_strerror.argtypes = [c_int]
    lib.ipex_attn_decode_noalloc_strerror.restype = ctypes.c_char_p
    lib.ipex_attn_decode_noalloc_max_floats.restype = c_int64
    lib.ipex_attn_decode_noalloc_max_counters.restype = c_int64
    return lib


def _case(B, Hq, Hkv, Sq, Skv, D, fp8, dtype, seed):
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, Hq, Sq, D, device=dev, generator=g).to(dtype)
    k = torch.randn(B, Hkv, Skv, D, device=dev, generator=g).to(dtype)
    v = torch.randn(B, Hkv, Skv, D, device=dev, generator=g).to(dtype)
    if fp8:
        from ipex_llm_b200.ops.kv_cache import fp8_e5m2_dequantize, fp8_e5m2_quantize
        k8, v8 = fp8_e5m2_quantize(k), fp8_e5m2_quantize(v)
        return q, k8, v8, fp8_e5m2_dequantize(k8, torch.float32), fp8_e5m2_dequantize(v8, torch.float32)
    return q, k, v, k.float(), v.float()


def _torch_ref(q, kf, vf, scale):
    B, Hq, Sq, D = q.shape
    Hkv, Skv = kf.shape[1], kf.shape[2]
    rep = Hq // Hkv
    kk = kf.repeat_interleave(rep, dim=1)
    vv = vf.repeat_interleave(rep, dim=1)
    w = torch.matmul(q.float(), kk.transpose(2, 3)) * scale
    qi = torch.arange(Skv - Sq, Skv, device=q.device).view(-1, 1)
    ki = torch.arange(Skv, device=q.device).view(1, -1)
    w = w.masked_fill(~(ki <= qi), float("-inf"))
    return torch.matmul(torch.softmax(w, dim=-1), vv)       # [B, Hq, Sq, D]


def _run_both(lib, q, k, v, nsplit, scale):
    from ipex_llm_b200.native.lib import current_stream, ptr
    from ipex_llm_b200.ops import cuda_ops
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    G = Hq // Hkv
    fp8 = k.dtype == torch.uint8
    dt = cuda_ops._dt(q)
    strides = (c_int64 * 12)(q.stride(0), q.stride(2), q.stride(1), 0, 0, 0, k.stride(0), k.stride(1), k.stride(2),
                             Sq * Hq * D, Hq * D, D)
    # existing entry point, caller-provided buffers
    out_a = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    floats = lib.ipex_attn_decode_scratch_floats(B, Hkv, G, Sq, D, nsplit)
    ints = lib.ipex_attn_decode_counter_ints(B, Hkv, G, Sq)
    scratch = torch.empty(floats, dtype=torch.float32, device=q.device)
    counters = torch.zeros(ints, dtype=torch.int32, device=q.device)
    rc = lib.ipex_attn_decode(ptr(q), None, None, ptr(k), ptr(v), ptr(out_a), None, Skv, None, None, ptr(scratch),
                              ptr(counters), strides, B, Sq, Hq, Hkv, D, nsplit, 0, 0, 1, 0, float(scale), 0.0,
                              int(fp8), dt, 0, current_stream())
    assert rc == 0
    # library-owned scratch
    out_b = torch.full((B, Sq, Hq, D), float("nan"), dtype=q.dtype, device=q.device)
    rc = lib.ipex_attn_decode_noalloc(ptr(q), None, None, ptr(k), ptr(v), ptr(out_b), None, Skv, None, None, strides,
                                      B, Sq, Hq, Hkv, D, nsplit, 0, 0, 1, 0, float(scale), 0.0, int(fp8), dt, 0,
                                      current_stream())
    assert rc == 0, lib.ipex_attn_decode_noalloc_strerror(rc)
    torch.cuda.synchronize()
    return out_a, out_b


@pytest.mark.parametrize("shape", [
    # B, Hq, Hkv, Sq, Skv, D, fp8, nsplit
    (1, 32, 32, 1, 1024, 128, False, 8),
    (2, 16, 4, 1, 777, 128, True, 5),
    (1, 8, 2, 3, 300, 64, False, 3),
])
def test_noalloc_matches_regular_entry_point_twice(shape):
    B, Hq, Hkv, Sq, Skv, D, fp8, nsplit = shape
    lib = _lib()
    torch.cuda.set_device(0)
    assert lib.ipex_attn_decode_noalloc_setup() == 0      # set-up, outside any capture
    scale = D ** -0.5
    for call in range(2):                                   # two calls in a row share the array
        q, k, v, kf, vf = _case(B, Hq, Hkv, Sq, Skv, D, fp8, torch.float16, seed=10 * call + Skv)
        out_a, out_b = _run_both(lib, q, k, v, nsplit, scale)
        assert torch.isfinite(out_b.float()).all()
        assert torch.equal(out_a, out_b) or (out_a.float() - out_b.float()).abs().max().item() < 2e-3
        ref = _torch_ref(q, kf, vf, scale).transpose(1, 2)  # [B, Sq, Hq, D]
        assert (out_b.float() - ref).abs().max().item() < 2e-2


def test_noalloc_rejects_oversized_requests():
    lib = _lib()
    torch.cuda.set_device(0)
    from ipex_llm_b200.native.lib import current_stream, ptr
    max_f = lib.ipex_attn_decode_noalloc_max_floats()
    max_c = lib.ipex_attn_decode_noalloc_max_counters()
    assert max_f == 2 * 1024 * 1024 and max_c == 4096
    B, Hq, Hkv, Sq, D, nsplit = 8, 64, 64, 1, 128, 64     # partials far beyond the array
    assert lib.ipex_attn_decode_scratch_floats(B, Hkv, 1, Sq, D, nsplit) > max_f
    q = torch.zeros(B, Hq, Sq, D, dtype=torch.float16, device="cuda")
    k = torch.zeros(B, Hkv, 64, D, dtype=torch.float16, device="cuda")
    out = torch.zeros(B, Sq, Hq, D, dtype=torch.float16, device="cuda")
    strides = (c_int64 * 12)(q.stride(0), q.stride(2), q.stride(1), 0, 0, 0, k.stride(0), k.stride(1), k.stride(2),
                             Sq * Hq * D, Hq * D, D)
    rc = lib.ipex_attn_decode_noalloc(ptr(q), None, None, ptr(k), ptr(k), ptr(out), None, 64, None, None, strides,
                                      B, Sq, Hq, Hkv, D, nsplit, 0, 0, 1, 0, 1.0, 0.0, 0, 0, 0, current_stream())
    assert rc == -1
    assert b"exceed" in lib.ipex_attn_decode_noalloc_strerror(rc)
    # too many tickets: batch x kv heads beyond 4096 with two splits.  The ticket limit is checked first, so the
    # code is the ticket one although the partials of such a launch do not fit either.
    B2 = 128
    assert lib.ipex_attn_decode_counter_ints(B2, 64, 1, 1) > max_c
    rc = lib.ipex_attn_decode_noalloc(ptr(q), None, None, ptr(k), ptr(k), ptr(out), None, 64, None, None, strides,
                                      B2, 1, 64, 64, 64, 2, 0, 0, 1, 0, 1.0, 0.0, 0, 0, 0, current_stream())
    assert rc == -2
    assert b"tickets" in lib.ipex_attn_decode_noalloc_strerror(rc)
    torch.cuda.synchronize()


def test_noalloc_single_split_needs_no_work_buffer():
    """One split writes straight to the output: the array is not used, so a batch whose split partials would be
    far over the limit is accepted and matches the regular entry point."""
    lib = _lib()
    torch.cuda.set_device(0)
    B, Hq, Hkv, Sq, Skv, D = 32, 32, 32, 1, 96, 128
    assert lib.ipex_attn_decode_scratch_floats(B, Hkv, 1, Sq, D, 1) > lib.ipex_attn_decode_noalloc_max_floats()
    q, k, v, kf, vf = _case(B, Hq, Hkv, Sq, Skv, D, False, torch.float16, seed=7)
    out_a, out_b = _run_both(lib, q, k, v, 1, D ** -0.5)
    assert torch.isfinite(out_b.float()).all()
    assert torch.equal(out_a, out_b) or (out_a.float() - out_b.float()).abs().max().item() < 2e-3
