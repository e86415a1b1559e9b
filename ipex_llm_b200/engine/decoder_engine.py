"""CUDA-graph decode engine for llama-architecture decoders (llama / mistral / qwen2 / yi ...).

The reference decodes through the Hugging Face module tree, one Python call and several device kernels per
sub-module, synchronising every token (python/llm/src/ipex_llm/utils/benchmark_util_4_47.py:3297-3378,
models/llama.py:56-206).  Decode at batch 1 on a B200 moves only ~3.6 GB per token for a 7B int4 model, so the
step is bounded by how tightly the weight stream is kept busy, not by arithmetic.  This engine therefore

* flattens the converted model into five fused kernels per layer
    1. RMSNorm + qkv GEMV (+bias)
    2. RoPE + KV-cache append (+e5m2 quantization) + split-KV attention
    3. o_proj GEMV + residual
    4. RMSNorm + gate/up GEMV + SiLU*mul
    5. down_proj GEMV + residual
  plus embedding gather, final-norm + lm_head GEMV and argmax;
* chains them with programmatic dependent launch (each kernel prefetches its weights into L2 while its
  predecessor drains) and captures the whole step in one CUDA graph;
* keeps the position in device memory so the same graph replays for every token;
* shares KV storage with the module path (prefill, speculative verification) through the package's cache
  classes, whose pre-allocated tensors it reads and appends to in place.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import List, Optional

import torch

from ..native import cuda_api as api
from ..native.lib import cuda_lib, current_stream, ptr
from ..ops import cuda_ops
from ..ops.kv_cache import DynamicFp8Cache, DynamicNormalCache
from ..ops.linear import LowBitLinear
from ..quant import qtypes as qt


class _W:
    """One linear of the flattened model: tiled low-bit bytes or a dense half matrix."""

    def __init__(self, data, wf, qtype, N, K, bias=None, tp=None):
        self.data, self.wf, self.qtype, self.N, self.K, self.bias = data, wf, qtype, N, K, bias
        self.tp = tp   # TPGroup of a row-parallel layer (its output is summed over the group), else None

    @staticmethod
    def from_module(mod, dtype):
        bias = mod.bias.data.to(dtype) if getattr(mod, "bias", None) is not None else None
        tp = getattr(mod, "mp_group", None)
        if tp is not None and getattr(tp, "world_size", 1) <= 1:
            tp = None
        if isinstance(mod, LowBitLinear):
            w = mod.weight
            if not cuda_ops.is_tiled(w.qtype):
                raise NotImplementedError(f"decode engine needs a tiled qtype, got {qt.qtype_name(w.qtype)}")
            return _W(w.data, cuda_ops.QTYPE_TO_WF[w.qtype], w.qtype, int(w._shape[0]), int(w._shape[1]), bias, tp)
        w = mod.weight.data.to(dtype).contiguous()
        wf = api.WF_F16 if dtype == torch.float16 else api.WF_BF16
        return _W(w, wf, None, w.shape[0], w.shape[1], bias, tp)


def _interleave_row_tiles(a: _W, b: _W) -> _W:
    """Merge two tiled weights of equal shape so that row tile 2i comes from ``a`` and 2i+1 from ``b``
    (gate / up), which lets one CTA produce act(gate) * up for 16 output features."""
    assert a.wf == b.wf and a.N == b.N and a.K == b.K and a.N % 16 == 0
    if a.wf in (api.WF_F16, api.WF_BF16):
        t = a.N // 16
        w = torch.stack([a.data.view(t, 16, a.K), b.data.view(t, 16, a.K)], dim=1).reshape(2 * a.N, a.K).contiguous()
        return _W(w, a.wf, None, 2 * a.N, a.K)
    Np, Kp = a.N, (a.K + 127) // 128 * 128
    T = Np // 16
    four_bit = a.wf in (api.WF_SYM_INT4, api.WF_ASYM_INT4, api.WF_LUT4)
    code_bytes = Np * Kp // 2 if four_bit else Np * Kp
    if four_bit:
        plane_sizes = [code_bytes] + [Np * (Kp // 64) * 2] * (2 if a.wf == api.WF_ASYM_INT4 else 1)
    elif a.wf == api.WF_INT8:
        plane_sizes = [code_bytes, Np * (Kp // 64) * 2]
    else:
        plane_sizes = [code_bytes, Np * (Kp // 128) * 4]
    out_planes = []
    off = 0
    for sz in plane_sizes:
        pa = a.data[off:off + sz].view(T, -1)
        pb = b.data[off:off + sz].view(T, -1)
        out_planes.append(torch.stack([pa, pb], dim=1).reshape(-1))
        off += sz
    return _W(torch.cat(out_planes).contiguous(), a.wf, a.qtype, 2 * a.N, a.K)


class _Layer:
    pass


class DecoderEngine:
    """Flattened llama-architecture decoder with graph-captured decode steps."""

    def __init__(self, model, max_batch: int = 1, max_len: int = 2048, kv_fp8: Optional[bool] = None):
        cfg = model.config
        self.model = model
        self.cfg = cfg
        base = model.model
        # a pipeline stage holds a slice of the layers; only the first stage has the embedding table and only the
        # last one the final norm and lm_head (parallel/pp.py replaces the rest by parameter-free stand-ins)
        real = [blk for blk in base.layers if hasattr(blk, "self_attn")]
        self.first_stage = getattr(base.embed_tokens, "weight", None) is not None
        self.last_stage = getattr(base.norm, "weight", None) is not None and \
            getattr(model.lm_head, "weight", None) is not None
        self.device = next(model.parameters()).device
        ndt = base.norm.weight.dtype if self.last_stage else real[0].input_layernorm.weight.dtype
        self.dtype = ndt if ndt in (torch.float16, torch.bfloat16) else torch.float16
        self.H = cfg.hidden_size
        self.n_heads_cfg = cfg.num_attention_heads
        self.n_kv_cfg = getattr(cfg, "num_key_value_heads", None) or cfg.num_attention_heads
        self.hd = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        self.eps = float(getattr(cfg, "rms_norm_eps", 1e-6))
        self.vocab = cfg.vocab_size
        self.max_batch = max_batch
        self.max_len = max_len
        if kv_fp8 is None:
            from ..models.utils import use_quantize_kv_cache
            kv_fp8 = use_quantize_kv_cache(None, torch.empty(max_batch, 1, device=self.device), 1, 1)
        self.kv_fp8 = bool(kv_fp8)
        self.use_pdl = os.environ.get("IPEX_LLM_PDL", "1") != "0"
        dt = self.dtype

        self.embed = None
        if self.first_stage:
            self.embed = base.embed_tokens.weight.data
            if self.embed.dtype != dt:
                self.embed = self.embed.to(dt)
        self.final_norm = base.norm.weight.data.to(dt) if self.last_stage else None
        self.lm_head = _W.from_module(model.lm_head, dt) if self.last_stage else None
        # vocabulary-parallel lm_head: this rank scores rows [vocab_offset, vocab_offset + lm_head.N) of the vocabulary
        self.lm_gather = getattr(model.lm_head, "tp_gather", None)
        if self.lm_gather is not None and getattr(self.lm_gather, "world_size", 1) <= 1:
            self.lm_gather = None
        self.vocab_offset = self.lm_gather.rank * self.lm_head.N if self.lm_gather is not None else 0
        self.layers: List[_Layer] = []
        for blk in real:
            L = _Layer()
            attn, mlp = blk.self_attn, blk.mlp
            if not hasattr(attn, "qkv_proj"):
                raise NotImplementedError("decode engine expects merged qkv_proj (optimize_model=True)")
            L.qkv = _W.from_module(attn.qkv_proj, dt)
            L.o = _W.from_module(attn.o_proj, dt)
            L.moe = None
            if hasattr(mlp, "experts"):
                # sparse mixture-of-experts block: router matrix + expert bank (kernels of ops/cuda_ops.moe_forward)
                if not cuda_ops.moe_supported(mlp.experts) or getattr(mlp.experts, "_tp_group", None) is not None \
                        or getattr(mlp, "shared_expert", None) is not None:
                    raise NotImplementedError("decode engine: this mixture-of-experts block needs the module tree")
                L.moe = mlp.experts
                L.router = mlp.gate.weight.data.to(dt).contiguous()
                L.top_k = int(getattr(mlp.gate, "top_k", None) or getattr(mlp, "top_k", 2))
                L.renorm = bool(getattr(mlp.gate, "norm_topk_prob", True))
                L.gate_up = L.down = None
            else:
                g, u = _W.from_module(mlp.gate_proj, dt), _W.from_module(mlp.up_proj, dt)
                L.gate_up = _interleave_row_tiles(g, u)
                L.down = _W.from_module(mlp.down_proj, dt)
            L.ln1 = blk.input_layernorm.weight.data.to(dt)
            L.ln2 = blk.post_attention_layernorm.weight.data.to(dt)
            L.layer_idx = attn.layer_idx
            self.layers.append(L)
        # local (possibly tensor-parallel) head counts follow the fused qkv shape
        groups = self.n_heads_cfg // self.n_kv_cfg
        total_heads = self.layers[0].qkv.N // self.hd
        self.n_kv = total_heads // (groups + 2)
        self.n_heads = total_heads - 2 * self.n_kv
        self.has_moe = any(L.moe is not None for L in self.layers)
        dense = [L for L in self.layers if L.moe is None]
        self.inter = dense[0].gate_up.N // 2 if dense else self.layers[0].moe.intermediate_dim
        self.tp_group = getattr(self.layers[0], "tp", None)

        # rotary table (fp32) from the model's own rotary module, so every rope-scaling flavour is honoured
        pos = torch.arange(max_len, device=self.device).unsqueeze(0)
        dummy = torch.zeros(1, max_len, self.H, device=self.device, dtype=torch.float32)
        cos, sin = base.rotary_emb(dummy, position_ids=pos)
        R = cos.shape[-1]
        self.rot_dim = R
        self.cos = cos[0, :, : R // 2].float().contiguous()
        self.sin = sin[0, :, : R // 2].float().contiguous()

        B = max_batch
        dev = self.device
        self.tokens = torch.zeros(B, dtype=torch.int64, device=dev)
        self.vtokens = torch.zeros(8, dtype=torch.int64, device=dev)      # verify_step: tokens in, arg-max out
        self.vout = torch.zeros(8, dtype=torch.int64, device=dev)
        self.past_len = torch.zeros(B, dtype=torch.int32, device=dev)
        self.h = [torch.zeros(B, self.H, dtype=dt, device=dev) for _ in range(2)]
        self.qkv_buf = torch.zeros(B, self.layers[0].qkv.N, dtype=dt, device=dev)
        self.attn_buf = torch.zeros(B, self.n_heads * self.hd, dtype=dt, device=dev)
        self.act_buf = torch.zeros(B, self.inter, dtype=dt, device=dev)
        self.logits = torch.zeros(B, self.vocab, dtype=dt, device=dev) if self.last_stage else None
        self.cache = None
        self._graphs = {}
        self._lib = cuda_lib()
        self._nsplit = None
        self._kv_hint = None       # prompt length of the current generation (sizes the attention splits)
        self._mega = None          # whole-step kernel launcher, created on first use (False = not applicable)

    # ------------------------------------------------------------------------------------------------
    def new_cache(self, batch: int):
        """A cache of the package's own class whose storage is pre-allocated to ``max_len`` tokens."""
        pool = self.__dict__.setdefault("_cache_pool", {})
        if batch in pool:
            cache = pool[batch]
            for layer in cache.layers:
                layer.set_length(0)
            return cache
        cls = DynamicFp8Cache if self.kv_fp8 else DynamicNormalCache
        cache = cls(self.cfg)
        pool[batch] = cache
        for _ in self.layers:
            layer = cache.layer_class_to_replicate()
            layer.preallocate(batch, self.n_kv, self.max_len, self.hd, self.hd, self.dtype, self.device)
            cache.layers.append(layer)
        return cache

    def bind_cache(self, cache, batch: int):
        self.cache = cache
        self.batch = batch
        self._graphs = {k: v for k, v in self._graphs.items() if v[1] is cache}

    # ------------------------------------------------------------------------------------------------
    def _gemv(self, w: _W, x, out, norm_w=None, bias=None, residual=None, act=0):
        M = x.shape[0]
        for s in range(0, M, 8):
            e = min(M, s + 8)
            if w.tp is not None and norm_w is None and act == 0 and w.wf not in (api.WF_F16, api.WF_BF16) and \
                    os.environ.get("IPEX_LLM_TP_FUSED_AR", "0") == "1":
                # row-parallel layer, opt-in: the GEMV kernel exchanges its partial tiles with the peers itself.
                # Measured on a 70B-shaped model at TP=2, the GEMV followed by the one-shot peer-memory all-reduce
                # kernel is faster (2.69 vs 3.15 ms for 8 layers), so that is the default below.
                cuda_ops.gemv_lowbit_ar(x[s:e], w.data, w.qtype, w.N, w.K, out[s:e], w.tp.symm(),
                                        bias=bias if bias is not None else w.bias,
                                        residual=residual[s:e] if residual is not None else None,
                                        pdl=self.use_pdl, wf=w.wf)
                continue
            if w.tp is not None and norm_w is None and act == 0 and out[s:e].is_contiguous() and \
                    (residual is None or residual[s:e].is_contiguous()) and w.tp.symm() is not None and \
                    (e - s) * w.N * out.element_size() <= w.tp.symm().ar_bytes and \
                    os.environ.get("IPEX_LLM_TP_STAGED_AR", "1") != "0":
                # row-parallel layer, default: the GEMV writes its partial product straight into this rank's
                # symmetric staging buffer and ONE kernel does the peer-memory all-reduce + bias + residual
                # (two launches per layer half instead of GEMV, copy, all-reduce, bias add, residual add)
                comm = w.tp.symm()
                stage, token = comm.ar_stage((e - s) * w.N, out.dtype)
                cuda_ops.gemv_lowbit(x[s:e], w.data, w.qtype, w.N, w.K, out=stage.view(e - s, w.N),
                                     pdl=self.use_pdl, wf=w.wf)
                comm.all_reduce_staged(token, out[s:e], residual=residual[s:e] if residual is not None else None,
                                       bias=bias if bias is not None else w.bias,
                                       pdl=self.use_pdl and os.environ.get("IPEX_LLM_TP_AR_PDL", "1") != "0")
                continue
            if w.tp is not None:
                # row-parallel layer, stand-alone steps: plain GEMV, all-reduce, then bias and residual
                cuda_ops.gemv_lowbit(x[s:e], w.data, w.qtype, w.N, w.K, out=out[s:e], pdl=False, wf=w.wf)
                w.tp.all_reduce(out[s:e])
                b_ = bias if bias is not None else w.bias
                if b_ is not None:
                    out[s:e].add_(b_)
                if residual is not None:
                    out[s:e].add_(residual[s:e])
                continue
            cuda_ops.gemv_lowbit(x[s:e], w.data, w.qtype, w.N, w.K, out=out[s:e], norm_weight=norm_w, eps=self.eps,
                                 bias=bias if bias is not None else w.bias,
                                 residual=residual[s:e] if residual is not None else None, act=act,
                                 pdl=self.use_pdl, wf=w.wf)

    def _lm_head(self, x, B: int):
        """Final norm + lm_head for ``B`` rows into ``logits[:B]`` (the full vocabulary on every rank)."""
        if self.lm_gather is None:
            self._gemv(self.lm_head, x, self.logits[:B], norm_w=self.final_norm)
            return
        off, n = self.vocab_offset, self.lm_head.N
        self._gemv(self.lm_head, x, self.logits[:B, off:off + n], norm_w=self.final_norm)
        self.gather_logits(B)

    def gather_logits(self, B: int):
        """Vocabulary-parallel lm_head: every rank holds its slice of ``logits[:B]``; exchange the slices (a library
        all-gather, issued outside graph capture)."""
        if self.lm_gather is None:
            return self.logits[:B]
        off, n = self.vocab_offset, self.lm_head.N
        full = self.lm_gather.all_gather_last_dim(self.logits[:B, off:off + n].contiguous())
        self.logits[:B].copy_(full)
        return self.logits[:B]

    def mega_step(self, B: int):
        """The whole-step kernel launcher when the model and batch fit it (see engine/mega.py), else None."""
        if self._mega is None:
            from .mega import MegaStep
            why = MegaStep.supported(self)
            self._mega = MegaStep(self) if why is None else False
            self.mega_reason = why
        if self._mega is False or B > self._mega.max_batch:
            return None
        return self._mega

    @property
    def kernel_launches_per_step(self) -> int:
        n = len(self.layers)
        if self.mega_step(getattr(self, "batch", 1) or 1) is not None:
            return 1                          # embedding ... arg-max in one persistent kernel
        if self.has_moe:
            # per layer: qkv, attention, o_proj, norm, router GEMM, softmax/top-k, two expert GEMVs, combine, residual
            n_moe = sum(1 for L in self.layers if L.moe is not None)
            return 1 + 5 * (n - n_moe) + 10 * n_moe + 2
        if self.layers[0].o.tp is not None:
            return 1 + 7 * n + 2              # tensor parallel: + one all-reduce kernel after o_proj and down_proj
        return 1 + 5 * n + 2

    def _moe_mlp(self, L: _Layer, h1, out):
        """``out = h1 + experts(norm(h1))`` of a sparse mixture-of-experts layer: router scores, fused softmax /
        top-k, per-slot expert GEMVs through a device pointer table (few rows) or expert-sorted tcgen05 GEMMs that
        read their row ranges on the device (prompts).  Nothing synchronises with the host, so the sequence is
        captured into the decode graph like the dense layers."""
        x = cuda_ops.rms_norm(h1, L.ln2, self.eps)
        scores = torch.matmul(x, L.router.t())
        _, w, idx = cuda_ops.moe_softmax_topk(scores, L.top_k, L.renorm)
        y = cuda_ops.moe_forward(L.moe, x, idx, w, residual=h1, out=out)
        if y.data_ptr() != out.data_ptr():
            out.copy_(y)
        return out

    def _pick_splits(self, B: int) -> int:
        """KV splits of the decode attention, sized for the context this generation will actually reach (the next
        power of two above prompt + 256 tokens) rather than for the cache capacity: the kernel divides whatever
        length it finds by this count, and 2816 tokens of capacity gave a 1024-token prompt 22 splits of 48 tokens
        where 11 splits are best (Llama-2-7B: 2.00 ms per token against 1.86 ms).  The count is part of the
        captured graph, so graphs are kept per (batch, splits)."""
        hint = self._kv_hint if self._kv_hint else self.max_len
        target = 512
        while target < hint + 256:
            target *= 2
        target = min(target, self.max_len)
        return cuda_ops.pick_nsplit(B, self.n_kv, target, rows=self.n_heads // self.n_kv)

    def _attention(self, L: _Layer, B: int, Sq: int = 1):
        """Rope + cache append + attention for ``B`` sequences of ``Sq`` new tokens each; rows of the activation
        buffers are ordered (sequence, position)."""
        lib = self._lib
        layer = self.cache.layers[L.layer_idx]
        kc, vc = layer._k, layer._v
        D, Hq, Hkv = self.hd, self.n_heads, self.n_kv
        q_off_k = Hq * D
        q_off_v = (Hq + Hkv) * D
        qkv = self.qkv_buf[:B * Sq]
        ld = qkv.stride(0)
        knew = qkv[:, q_off_k:]
        vnew = qkv[:, q_off_v:]
        out = self.attn_buf[:B * Sq]
        ldo = out.stride(0)
        G = Hq // Hkv
        nsplit = self._nsplit
        floats = lib.ipex_attn_decode_scratch_floats(B, Hkv, G, Sq, D, nsplit)
        ints = lib.ipex_attn_decode_counter_ints(B, Hkv, G, Sq)
        scratch, counters = cuda_ops.attn_workspace(self.device, floats, ints)
        strides = (ctypes.c_int64 * 12)(Sq * ld, ld, D, Sq * ld, ld, D, kc.stride(0), kc.stride(1), kc.stride(2),
                                        Sq * ldo, ldo, D)
        rc = lib.ipex_attn_decode(ptr(qkv), ptr(knew), ptr(vnew), ptr(kc), ptr(vc), ptr(out), ptr(self.past_len), 0,
                                  ptr(self.cos), ptr(self.sin), ptr(scratch), ptr(counters), strides, B, Sq, Hq, Hkv,
                                  D, nsplit, 1, self.rot_dim, 1, 0, 1.0 / math.sqrt(D), 0.0, int(self.kv_fp8),
                                  api.dtype_code(self.dtype), int(self.use_pdl), current_stream())
        api.check(rc, "attn_decode")

    # ------------------------------------------------------------------------------------------------
    # multi-token scoring of ONE sequence (self-speculative verification, prompt lookup)
    # ------------------------------------------------------------------------------------------------
    def _verify_kernels(self, S: int):
        lib = self._lib
        dtc = api.dtype_code(self.dtype)
        pdl = int(self.use_pdl)
        h0, h1 = self.h[0][:S], self.h[1][:S]
        rc = lib.ipex_embedding(ptr(self.vtokens), ptr(self.embed), ptr(h0), S, self.H, 1.0, dtc, 0, current_stream())
        api.check(rc, "embedding")
        for L in self.layers:
            self._vproj(L.qkv, h0, self.qkv_buf[:S], norm_w=L.ln1)
            self._attention(L, 1, Sq=S)
            self._vproj(L.o, self.attn_buf[:S], h1, residual=h0)
            if L.moe is not None:
                self._moe_mlp(L, h1, h0)
                continue
            self._vproj(L.gate_up, h1, self.act_buf[:S], norm_w=L.ln2, act=1)
            self._vproj(L.down, self.act_buf[:S], h0, residual=h1)
        if self.lm_gather is None:
            self._vproj(self.lm_head, h0, self.logits[:S], norm_w=self.final_norm)
        else:
            self._lm_head(h0, S)
        rc = lib.ipex_argmax(ptr(self.logits), ptr(self.vout), S, self.vocab, self.logits.stride(0), dtc, pdl,
                             current_stream())
        api.check(rc, "argmax")

    def _vproj(self, w: _W, x, out, norm_w=None, residual=None, act=0):
        """Projection of the multi-token verification pass.  Dense half weights (the speculative target) with more
        than two rows go through the tcgen05 GEMM: its 128-row weight tiles arrive by TMA and amortise the staging
        of the token rows, which the 16-row GEMV CTAs pay per CTA (8 rows measured 2.25x a single-row step there).
        Everything else takes the multi-row GEMV."""
        S = x.shape[0]
        if w.wf in (api.WF_F16, api.WF_BF16) and S > 2 and w.tp is None and w.K % 8 == 0 and \
                (act == 0 or w.N % 32 == 0) and os.environ.get("IPEX_LLM_VERIFY_GEMM", "1") != "0":
            from ..ops import tcgen05_gemm
            xin = cuda_ops.rms_norm(x, norm_w, self.eps) if norm_w is not None else x
            tcgen05_gemm.gemm_dense(xin, w.data, bias=w.bias, residual=residual, out=out, act=act)
            return
        self._gemv(w, x, out, norm_w=norm_w, residual=residual, act=act)

    def verify_step(self, S: int, use_graph: bool = True):
        """Score ``vtokens[:S]`` (1 <= S <= min(8, max_batch)) as the next ``S`` tokens of sequence 0 in one pass:
        their K/V go to cache rows ``past_len[0] ..``, ``logits[:S]`` hold the scores after each of them and
        ``vout[:S]`` the arg-max tokens.  ``past_len`` is left as it was: the caller advances it by the number of
        tokens it keeps, which is all the cropping a rejected draft needs (rows past ``past_len`` are dead).
        The reference verifies drafts with a full module-tree forward and crops the cache tensors afterwards
        (python/llm/src/ipex_llm/transformers/speculative.py:1071-1113, 540-608)."""
        if S < 1 or S > min(8, self.max_batch):
            raise ValueError(f"verify_step scores 1..{min(8, self.max_batch)} tokens, got {S}")
        if self.layers[0].o.tp is not None:
            raise NotImplementedError("verify_step runs on a single GPU")
        self._nsplit = self._pick_splits(1)
        if not use_graph or os.environ.get("IPEX_LLM_ENGINE_GRAPH", "1") == "0":
            self._verify_kernels(S)
            return
        key = ("verify", S, self._nsplit)
        entry = self._graphs.get(key)
        if entry is None:
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._verify_kernels(S)       # warm-up: writes only rows past past_len and scratch buffers
            torch.cuda.current_stream().wait_stream(s)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._verify_kernels(S)
            entry = (g, self.cache, 0)
            self._graphs[key] = entry
        entry[0].replay()

    def _step_kernels(self, B: int):
        """Issue one decode step for ``B`` sequences on the current stream: tokens[:B] -> tokens[:B]."""
        mega = self.mega_step(B)
        if mega is not None:
            mega.step(B)                      # embedding -> layers -> lm_head -> arg-max -> past_len + 1
            return
        lib = self._lib
        dtc = api.dtype_code(self.dtype)
        pdl = int(self.use_pdl)
        h0, h1 = self.h[0][:B], self.h[1][:B]
        if self.first_stage:
            rc = lib.ipex_embedding(ptr(self.tokens), ptr(self.embed), ptr(h0), B, self.H, 1.0, dtc, 0,
                                    current_stream())
            api.check(rc, "embedding")
        # (later pipeline stages: the previous stage's hidden states were received into h[0][:B])
        if B > 24 and self._gemm_decode_ok():
            # many sequences: every projection is one tcgen05 low-bit GEMM with a 32-token tile (the weights are
            # read once per step; eight-row GEMVs read them once per group of eight sequences).  Measured on
            # Llama-2-7B sym_int4: 32 sequences 20.0 ms per step against 22.0 ms, but 16 sequences 14.8 ms against
            # ~10.8 ms: the GEMM's dequantizer warps expand every weight to 16 bits whatever the token count, which
            # bounds it near 0.7 TB/s of packed weights, so the GEMVs keep the smaller batches.
            for L in self.layers:
                x = cuda_ops.rms_norm(h0, L.ln1, self.eps)
                self._gemm(L.qkv, x, out=self.qkv_buf[:B])
                self._attention(L, B)
                self._gemm(L.o, self.attn_buf[:B], residual=h0, out=h1)
                if L.moe is not None:
                    self._moe_mlp(L, h1, h0)
                    continue
                x = cuda_ops.rms_norm(h1, L.ln2, self.eps)
                self._gemm(L.gate_up, x, act=1, out=self.act_buf[:B])
                self._gemm(L.down, self.act_buf[:B], residual=h1, out=h0)
            if self.last_stage:
                x = cuda_ops.rms_norm(h0, self.final_norm, self.eps)
                if self.lm_gather is None:
                    self._gemm(self.lm_head, x, out=self.logits[:B])
                else:
                    off, n = self.vocab_offset, self.lm_head.N
                    self.logits[:B, off:off + n].copy_(self._gemm(self.lm_head, x))
                    self.gather_logits(B)
                rc = lib.ipex_argmax(ptr(self.logits), ptr(self.tokens), B, self.vocab, self.logits.stride(0), dtc, pdl,
                                     current_stream())
                api.check(rc, "argmax")
            self.past_len[:B].add_(1)
            return
        for L in self.layers:
            self._gemv(L.qkv, h0, self.qkv_buf[:B], norm_w=L.ln1)
            self._attention(L, B)
            self._gemv(L.o, self.attn_buf[:B], h1, residual=h0)
            if L.moe is not None:
                self._moe_mlp(L, h1, h0)
                continue
            self._gemv(L.gate_up, h1, self.act_buf[:B], norm_w=L.ln2, act=1)
            self._gemv(L.down, self.act_buf[:B], h0, residual=h1)
        if self.last_stage:
            self._lm_head(h0, B)
            rc = lib.ipex_argmax(ptr(self.logits), ptr(self.tokens), B, self.vocab, self.logits.stride(0), dtc, pdl,
                                 current_stream())
            api.check(rc, "argmax")
        # (earlier pipeline stages hand h[0][:B] to the next stage)
        self.past_len[:B].add_(1)

    def decode_step(self, B: int, use_graph: bool = True):
        """One token for every sequence.  The step is captured once per (batch, cache) and replayed."""
        self._nsplit = self._pick_splits(B)
        if self.lm_gather is not None and self.mega_step(B) is None:
            use_graph = False      # the logits exchange of the per-kernel path is a library collective: not captured
        if not use_graph or os.environ.get("IPEX_LLM_ENGINE_GRAPH", "1") == "0":
            self._step_kernels(B)
            return
        gkey = (B, self._nsplit)
        entry = self._graphs.get(gkey)
        if entry is None:
            # warm up outside capture (lazy allocations, cudaFuncSetAttribute), restoring the state it advances
            saved_tok, saved_len = self.tokens.clone(), self.past_len.clone()
            saved_h = None if self.first_stage else self.h[0].clone()   # a later stage's input arrives in h[0]
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._step_kernels(B)
            torch.cuda.current_stream().wait_stream(s)
            self.tokens.copy_(saved_tok)
            self.past_len.copy_(saved_len)
            if saved_h is not None:
                self.h[0].copy_(saved_h)
            comm = self._tp_comm()
            parity = comm._parity if comm is not None else 0
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._step_kernels(B)
            # capture does not execute: state is unchanged
            entry = (g, self.cache, parity)
            self._graphs[gkey] = entry
        comm = self._tp_comm()
        if comm is not None and comm._parity != entry[2]:
            # the buffer parity of the fused all-reduces is baked into the graph: realign (same on every rank)
            comm.barrier()
        entry[0].replay()

    def _tp_comm(self):
        tp = self.layers[0].o.tp
        return tp.symm() if tp is not None else None

    # ------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, input_ids: torch.Tensor, attention_mask=None):
        """Prompt pass, writing K/V into the engine's cache; returns the logits of the last position ``[B, V]``.
        Unmasked prompts of quantized models take the flattened pass (``_prefill_flat``: tcgen05 GEMMs with fused
        residual / SwiGLU epilogues and the tcgen05 attention, about nine kernels per layer); masked batches, tiny
        prompts and dense-weight models go through the module tree."""
        B, S = input_ids.shape
        if S + 1 > self.max_len:
            raise ValueError(f"prompt of {S} tokens does not fit max_len={self.max_len}")
        cache = self.new_cache(B)
        self.bind_cache(cache, B)
        if attention_mask is None and B * S >= 16 and B <= 8 and self._flat_prefill_ok():
            return self._prefill_flat(input_ids, cache)
        out = self.model(input_ids=input_ids, attention_mask=attention_mask, past_key_values=cache, use_cache=True)
        logits = out.logits[:, -1, :]
        self.past_len[:B] = S
        self._kv_hint = S
        return logits

    # ------------------------------------------------------------------------------------------------
    # flat prompt pass: the same flattened weights as decode, ~9 kernels per layer, no module tree
    # ------------------------------------------------------------------------------------------------
    def _gemm_decode_ok(self) -> bool:
        """Decode steps of more than eight sequences on the tcgen05 GEMMs: quantized weights the GEMM takes, one GPU
        (the tensor-parallel GEMM epilogues allocate their staging on first use, which a graph capture cannot)."""
        return self._flat_prefill_ok() and self.tp_group is None and self.layers[0].o.tp is None and \
            os.environ.get("IPEX_LLM_DECODE_GEMM", "1") != "0"

    def _flat_prefill_ok(self) -> bool:
        ok = self.__dict__.get("_flat_ok")
        if ok is None:
            ws = [w for L in self.layers for w in (L.qkv, L.o, L.gate_up, L.down) if w is not None]
            ok = os.environ.get("IPEX_LLM_FLAT_PREFILL", "1") != "0" and \
                hasattr(self._lib, "ipex_gemm_lowbit_tcgen05") and \
                all(w.K % 128 == 0 and w.N % 16 == 0 and w.wf not in (api.WF_F16, api.WF_BF16) for w in ws)
            self._flat_ok = ok
        return ok

    def _gemm(self, w: _W, x, residual=None, act=0, out=None):
        """``x [T, K]`` through a flattened projection on the tcgen05 path (+bias, +residual or act(gate)*up).
        Row-parallel layers sum their partial outputs over the tensor-parallel group before the residual."""
        from ..ops import tcgen05_gemm
        if w.tp is not None:
            comm = w.tp.symm()
            # The fused epilogue is a one-shot all-reduce: every rank stores its partial tile into EVERY rank's
            # staging buffer, (world - 1) x the output per rank over NVLink.  At two ranks that equals the traffic
            # of reduce-scatter + all-gather; beyond that it only pays for small outputs (a 2048-token prompt of
            # the 70B model at 8 ranks moved 235 MB per layer half and the prompt pass did not scale: 385 ms
            # against 287 ms at 2 ranks), so larger outputs go through the bandwidth-optimal library all-reduce.
            fused_ok = comm is not None and (comm.world <= 2 or x.shape[0] * w.N * x.element_size() <= (2 << 20))
            fused_env = os.environ.get("IPEX_LLM_TP_FUSED_GEMM_AR", "auto")
            if comm is not None and (fused_env == "1" or (fused_env != "0" and fused_ok)):
                # the all-reduce runs inside the GEMM's epilogue (peer stores + arrival counters over NVLink)
                return tcgen05_gemm.gemm_lowbit_ar(x, w.data, w.qtype, w.N, w.K, comm, bias=w.bias,
                                                   residual=residual, wf=w.wf)
            out = tcgen05_gemm.gemm_lowbit(x, w.data, w.qtype, w.N, w.K, wf=w.wf)
            w.tp.all_reduce(out)
            if w.bias is not None:
                out += w.bias
            if residual is not None:
                out += residual
            return out
        M = x.shape[0]
        if M >= cuda_ops.dequant_once_min_tokens() and w.qtype is not None and (act == 0 or w.N % 32 == 0):
            # opt-in for very long prompts (see cuda_ops.dequant_once_min_tokens): expand the packed weight once
            # into a transient half-precision matrix and run the dense TMA-fed kernel; the transient is one layer's
            # weight and is recycled by the allocator.
            wd = cuda_ops.dequantize_device(w.data, (w.N, w.K), w.qtype, x.dtype)
            return tcgen05_gemm.gemm_dense(x, wd, bias=w.bias, residual=residual, act=act)
        return tcgen05_gemm.gemm_lowbit(x, w.data, w.qtype, w.N, w.K, bias=w.bias, residual=residual, act=act,
                                        wf=w.wf, out=out)

    def clone_for_microbatch(self):
        """A second engine over the SAME flattened weights with its own activations, KV cache and graphs (pipeline
        stages keep one per micro-batch in flight)."""
        import copy
        other = copy.copy(self)
        B, dev, dt = self.max_batch, self.device, self.dtype
        other.tokens = torch.zeros(B, dtype=torch.int64, device=dev)
        other.vtokens = torch.zeros(8, dtype=torch.int64, device=dev)
        other.vout = torch.zeros(8, dtype=torch.int64, device=dev)
        other.past_len = torch.zeros(B, dtype=torch.int32, device=dev)
        other.h = [torch.zeros_like(self.h[0]) for _ in range(2)]
        other.qkv_buf = torch.zeros_like(self.qkv_buf)
        other.attn_buf = torch.zeros_like(self.attn_buf)
        other.act_buf = torch.zeros_like(self.act_buf)
        other.logits = torch.zeros_like(self.logits) if self.logits is not None else None
        other.cache = None
        other._graphs = {}
        other._cache_pool = {}
        other._mega = None
        return other

    @torch.no_grad()
    def prefill_stage(self, x: torch.Tensor):
        """Prompt pass of one pipeline stage.  ``x``: token ids ``[B, S]`` on the first stage, the previous stage's
        hidden states ``[B, S, H]`` otherwise.  Returns the last position's logits ``[B, V]`` on the last stage and
        the hidden states ``[B, S, H]`` to hand on elsewhere; K/V go into the engine's own cache."""
        B, S = x.shape[0], x.shape[1]
        if S + 1 > self.max_len:
            raise ValueError(f"prompt of {S} tokens does not fit max_len={self.max_len}")
        cache = self.new_cache(B)
        self.bind_cache(cache, B)
        if B * S >= 16 and B <= 8 and self._flat_prefill_ok():
            return self._prefill_flat(x if self.first_stage else None, cache,
                                      hidden=None if self.first_stage else x)
        kw = {"input_ids": x} if self.first_stage else {"inputs_embeds": x}
        out = self.model(past_key_values=cache, use_cache=True, **kw).logits
        self.past_len[:B] = S
        self._kv_hint = S
        return out[:, -1, :] if self.last_stage else out

    def _prefill_flat(self, input_ids: torch.Tensor, cache, hidden: torch.Tensor = None):
        if hidden is None:
            B, S = input_ids.shape
            h = torch.nn.functional.embedding(input_ids.reshape(-1), self.embed)       # [T, H]
        else:
            B, S = hidden.shape[0], hidden.shape[1]
            h = hidden.reshape(B * S, self.H).to(self.dtype)
        T, H, D = B * S, self.H, self.hd
        Hq, Hkv = self.n_heads, self.n_kv
        cos = torch.cat([self.cos[:S], self.cos[:S]], dim=-1).unsqueeze(0)             # [1, S, R] fp32
        sin = torch.cat([self.sin[:S], self.sin[:S]], dim=-1).unsqueeze(0)
        scale = 1.0 / math.sqrt(D)
        for L in self.layers:
            x = cuda_ops.rms_norm(h, L.ln1, self.eps)
            qkv = self._gemm(L.qkv, x).view(B, S, Hq + 2 * Hkv, D)
            q = qkv[:, :, :Hq].transpose(1, 2)                                          # [B, Hq, S, D] views
            k = qkv[:, :, Hq:Hq + Hkv].transpose(1, 2)
            v = qkv[:, :, Hq + Hkv:].transpose(1, 2)
            q, k = cuda_ops.rotary_inplace(q, k, cos, sin)
            cache.layers[L.layer_idx].update(k, v)
            a = cuda_ops.sdpa_prefill(q, k, v, None, scale, None, None, causal=True)    # [B, Hq, S, D]
            a = a.transpose(1, 2).reshape(T, Hq * D)
            h1 = self._gemm(L.o, a, residual=h)
            if L.moe is not None:
                h = self._moe_mlp(L, h1, torch.empty_like(h1))
                continue
            x = cuda_ops.rms_norm(h1, L.ln2, self.eps)
            act = self._gemm(L.gate_up, x, act=1)                                        # [T, I]
            h = self._gemm(L.down, act, residual=h1)
        self.past_len[:B] = S
        self._kv_hint = S
        if not self.last_stage:
            return h.view(B, S, H)
        last = h.view(B, S, H)[:, -1].contiguous()
        self._lm_head(last, B)
        return self.logits[:B].clone()

    def sync_cache_length(self, n: int):
        for layer in self.cache.layers:
            layer.set_length(n)
