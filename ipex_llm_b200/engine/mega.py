"""Whole-step decode kernel: host side.

``MegaStep`` binds a ``DecoderEngine`` (flattened weights, static activation buffers, KV cache) to the persistent
kernel of ``native/cuda/decode_mega.cu``, which runs embedding -> every layer -> lm_head -> arg-max of one decode
step in a single cooperative launch.  The reference issues the same work as a chain of module calls
(python/llm/src/ipex_llm/transformers/models/llama.py:56-206); the per-kernel path of the engine remains for the
shapes this kernel does not take (more than four sequences, mixed weight families, head sizes other than 64 / 128,
more than 16 query heads per kv head, verification of several tokens).

With tensor parallelism the kernel carries the all-reduce of the row-parallel projections itself: partial tiles are
stored into every peer's symmetric buffer and each CTA sums the rows it owns when the peers' flags arrive
(``_TPBuffers``), so a decode step is one launch per rank with no collective kernels.
"""
from __future__ import annotations

import ctypes
import os

import torch

from ..native import cuda_api as api
from ..native.lib import cuda_lib, current_stream

vp, ci, cf, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong

_N_SM = 148


class _Layer(ctypes.Structure):
    _fields_ = [(n, vp) for n in ("w_qkv", "w_o", "w_gu", "w_down", "ln1", "ln2", "b_qkv", "b_o", "kcache",
                                  "vcache")]


class _Args(ctypes.Structure):
    _fields_ = [(n, vp) for n in ("layers", "embed", "final_norm", "w_lm", "cosp", "sinp", "tokens", "past_len",
                                  "h0", "h1", "qkv", "attn", "act", "logits", "attn_scratch", "attn_counters",
                                  "amax", "barrier", "abort_word", "err")] + \
               [(n, ll) for n in ("c_b", "c_h", "c_s")] + \
               [(n, ci) for n in ("n_layers", "B", "H", "I", "Nqkv", "Hq", "Hkv", "D", "V", "R", "ld_logits",
                                  "nsplit", "stages", "kv_fp8")] + \
               [(n, cf) for n in ("eps", "norm_offset", "scale")] + \
               [(n, ci) for n in ("tp_rank", "tp_world", "tp_npad", "vocab_offset")] + \
               [(n, vp) for n in ("tp_bufs", "tp_flags", "tp_keys", "tp_kflags", "tp_epoch", "prof")]


def _declare(lib):
    if getattr(lib, "_mega_declared", False):
        return
    lib.ipex_decode_mega.argtypes = [vp, ci, ci, ci, ci, ci, vp]
    lib.ipex_decode_mega.restype = ci
    lib.ipex_decode_mega_stages.argtypes = [ci, ci, ci, ci, ci]
    lib.ipex_decode_mega_stages.restype = ci
    for n in ("ipex_decode_mega_args_bytes", "ipex_decode_mega_layer_bytes", "ipex_decode_mega_max_batch"):
        getattr(lib, n).argtypes = []
        getattr(lib, n).restype = ci
    lib._mega_declared = True


class _TPBuffers:
    """Symmetric memory of the fused step: partial tiles [2][world][4][npad] fp32, per-CTA flags [2][world][grid],
    arg-max keys [world][4] and their flags [world], one region per rank mapped by every peer."""

    def __init__(self, group, world, rank, npad, grid, device):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.npad = npad
        part = 2 * world * 4 * npad * 4
        flags = 2 * world * grid * 4
        keys = world * 4 * 8
        kflags = world * 4
        offs, total = [], 0
        for sz in (part, flags, keys, kflags):
            offs.append(total)
            total += (sz + 255) // 256 * 256
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=device)
        self.buf.zero_()
        torch.cuda.synchronize()
        pg = group if group is not None else dist.group.WORLD
        try:
            self.handle = symm_mem.rendezvous(self.buf, pg)
        except Exception:  # noqa: BLE001  (older signatures take the group name)
            self.handle = symm_mem.rendezvous(self.buf, pg.group_name)
        bases = [int(p) for p in self.handle.buffer_ptrs]
        dist.barrier(group=pg)
        self.ptrs = [torch.tensor([b + o for b in bases], dtype=torch.int64, device=device) for o in offs]
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)


class MegaStep:
    """Launcher of the whole-step kernel for one engine.  ``supported(engine)`` tells whether the model fits."""

    @staticmethod
    def supported(eng) -> str | None:
        """None when the engine's model can run on the fused step, else the reason it cannot."""
        mode = os.environ.get("IPEX_LLM_DECODE_MEGA", "auto")
        if mode == "0":
            return "disabled by IPEX_LLM_DECODE_MEGA=0"
        if mode == "auto" and eng.layers[0].o.tp is None:
            # one GPU: the per-projection kernels under programmatic dependent launch measured faster (Llama-2-7B
            # sym_int4, batch 1: 1.95 ms per token against 2.07 ms); the fused step pays off when it also carries
            # the tensor-parallel all-reduces
            return "one GPU: separate kernels are faster (IPEX_LLM_DECODE_MEGA=1 forces the fused step)"
        lib = cuda_lib()
        if not hasattr(lib, "ipex_decode_mega"):
            return "kernel library has no fused step"
        if getattr(eng, "has_moe", False):
            return "mixture-of-experts layers"
        if not (eng.first_stage and eng.last_stage):
            return "pipeline stage"
        ws = [w for L in eng.layers for w in (L.qkv, L.o, L.gate_up, L.down)] + [eng.lm_head]
        wf = ws[0].wf
        if wf not in (api.WF_SYM_INT4, api.WF_FP8_E4M3):
            return "weight family"
        if any(w.wf != wf for w in ws):
            return "mixed weight families"
        if eng.hd not in (64, 128) or eng.n_heads % eng.n_kv != 0 or eng.n_heads // eng.n_kv > 16:
            return "head geometry"
        if eng.rot_dim % 2 != 0 or eng.rot_dim > eng.hd:
            return "rotary size"
        if eng.H % 64 != 0 or eng.inter % 64 != 0 or eng.vocab % 16 != 0 or eng.layers[0].qkv.N % 16 != 0:
            return "dimension alignment"
        if wf == api.WF_FP8_E4M3 and (eng.H % 128 or eng.inter % 128 or (eng.n_heads * eng.hd) % 128):
            return "fp8 blocks need K % 128 == 0"
        for L in eng.layers:
            if L.gate_up.bias is not None or L.down.bias is not None:
                return "mlp bias"
            if (L.o.tp is None) != (L.down.tp is None):
                return "inconsistent tensor-parallel layers"
        if eng.lm_head.bias is not None or eng.lm_head.tp is not None:
            return "lm_head bias / row sharding"
        if eng.lm_head.N % 16 != 0:
            return "lm_head rows"
        return None

    def __init__(self, eng):
        self.eng = eng
        self.lib = cuda_lib()
        _declare(self.lib)
        assert self.lib.ipex_decode_mega_args_bytes() == ctypes.sizeof(_Args), "argument block layout differs"
        assert self.lib.ipex_decode_mega_layer_bytes() == ctypes.sizeof(_Layer), "layer block layout differs"
        self.max_batch = min(self.lib.ipex_decode_mega_max_batch(), eng.max_batch)
        dev = eng.device
        self.wf = eng.layers[0].qkv.wf
        self.kmax = max(eng.H, eng.layers[0].down.K, eng.layers[0].o.K)
        self.grid = int(os.environ.get("IPEX_LLM_MEGA_GRID", str(_N_SM)))
        self.coop = os.environ.get("IPEX_LLM_MEGA_COOP", "1") != "0"
        self.counters = torch.zeros(eng.max_batch * eng.n_kv + 8, dtype=torch.int32, device=dev)
        self.amax = torch.zeros(8, dtype=torch.int64, device=dev)
        self.sync = torch.zeros(4, dtype=torch.int32, device=dev)       # barrier[2], abort word
        from ..ops.cuda_ops import error_flag
        self.err = error_flag(dev)
        self.tp = None
        tpg = eng.layers[0].o.tp
        if tpg is not None:
            npad = (eng.H + 127) // 128 * 128
            self.tp = _TPBuffers(tpg.group, tpg.world_size, tpg.rank, npad, self.grid, dev)
            self.tp_rank, self.tp_world = tpg.rank, tpg.world_size
        # IPEX_LLM_MEGA_PROF=1: per-CTA cycle counters [grid][8] accumulated over the launches (see `profile()`)
        self.prof = torch.zeros(self.grid * 8, dtype=torch.int64, device=dev) \
            if os.environ.get("IPEX_LLM_MEGA_PROF", "0") == "1" else None
        self._layer_tab = None      # (cache id, device tensor holding the _Layer array)
        self._args = {}             # batch -> _Args
        self._scratch = {}

    # ------------------------------------------------------------------------------------------------
    def _nsplit(self, B: int) -> int:
        eng = self.eng
        env = os.environ.get("IPEX_LLM_MEGA_NSPLIT")
        if env:
            return max(1, min(64, int(env)))
        items = max(1, B * eng.n_kv)
        n = max(1, self.grid // items)
        # about 256 tokens per split of the context this generation reaches (next power of two above prompt + 256),
        # not of the cache capacity: 70B at two ranks, 2048-token prompt: 12.7-12.8 ms per token with 8-16 splits
        # against 13.2-13.3 ms with the 28 the capacity gave
        hint = getattr(eng, "_kv_hint", None) or eng.max_len
        target = 512
        while target < hint + 256:
            target *= 2
        target = min(target, eng.max_len)
        n = min(n, max(1, target // 256), 32)
        return n

    def _layers_for(self, cache):
        if self._layer_tab is not None and self._layer_tab[0] is cache:
            return self._layer_tab[1]
        eng = self.eng
        arr = (_Layer * len(eng.layers))()
        for i, L in enumerate(eng.layers):
            lay = cache.layers[L.layer_idx]
            a = arr[i]
            a.w_qkv, a.w_o, a.w_gu, a.w_down = (L.qkv.data.data_ptr(), L.o.data.data_ptr(),
                                                L.gate_up.data.data_ptr(), L.down.data.data_ptr())
            a.ln1, a.ln2 = L.ln1.data_ptr(), L.ln2.data_ptr()
            a.b_qkv = L.qkv.bias.data_ptr() if L.qkv.bias is not None else None
            a.b_o = L.o.bias.data_ptr() if L.o.bias is not None else None
            a.kcache, a.vcache = lay._k.data_ptr(), lay._v.data_ptr()
        raw = bytes(arr)
        tab = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(eng.device)
        self._layer_tab = (cache, tab)
        self._args.clear()
        return tab

    def _build(self, B: int):
        eng = self.eng
        cache = eng.cache
        tab = self._layers_for(cache)
        nsplit = self._nsplit(B)
        stages = self.lib.ipex_decode_mega_stages(self.wf, B, self.kmax, eng.hd, nsplit)
        if stages <= 0:
            raise RuntimeError("fused decode step: the activations of this shape do not fit shared memory")
        env_st = os.environ.get("IPEX_LLM_MEGA_STAGES")
        if env_st:
            stages = max(4, min(stages, int(env_st)))
        need = B * eng.n_kv * nsplit * 16 * (eng.hd + 2)
        scratch = self._scratch.get(B)
        if scratch is None or scratch.numel() < need:
            scratch = torch.empty(need, dtype=torch.float32, device=eng.device)
            self._scratch[B] = scratch
        k0 = cache.layers[eng.layers[0].layer_idx]._k
        for L in eng.layers:
            lay = cache.layers[L.layer_idx]
            assert lay._k.stride() == k0.stride() and lay._v.stride() == k0.stride() and lay._k.stride(3) == 1
        a = _Args()
        a.layers = tab.data_ptr()
        a.embed, a.final_norm, a.w_lm = eng.embed.data_ptr(), eng.final_norm.data_ptr(), eng.lm_head.data.data_ptr()
        a.cosp, a.sinp = eng.cos.data_ptr(), eng.sin.data_ptr()
        a.tokens, a.past_len = eng.tokens.data_ptr(), eng.past_len.data_ptr()
        a.h0, a.h1 = eng.h[0].data_ptr(), eng.h[1].data_ptr()
        # a vocabulary-parallel lm_head writes this rank's slice of the full-width logits rows
        a.qkv, a.attn, a.act, a.logits = (eng.qkv_buf.data_ptr(), eng.attn_buf.data_ptr(), eng.act_buf.data_ptr(),
                                          eng.logits.data_ptr() + eng.vocab_offset * eng.logits.element_size())
        a.attn_scratch, a.attn_counters, a.amax = scratch.data_ptr(), self.counters.data_ptr(), self.amax.data_ptr()
        a.barrier, a.abort_word, a.err = self.sync.data_ptr(), self.sync.data_ptr() + 8, self.err.data_ptr()
        a.c_b, a.c_h, a.c_s = k0.stride(0), k0.stride(1), k0.stride(2)
        a.n_layers, a.B, a.H, a.I = len(eng.layers), B, eng.H, eng.inter
        a.Nqkv, a.Hq, a.Hkv, a.D = eng.layers[0].qkv.N, eng.n_heads, eng.n_kv, eng.hd
        a.V, a.R, a.ld_logits = eng.lm_head.N, eng.rot_dim, eng.logits.stride(0)
        a.nsplit, a.stages, a.kv_fp8 = nsplit, stages, int(eng.kv_fp8)
        a.eps, a.norm_offset, a.scale = eng.eps, 0.0, 1.0 / (eng.hd ** 0.5)
        a.tp_rank, a.tp_world, a.tp_npad, a.vocab_offset = 0, 1, 0, 0
        if self.tp is not None:
            a.tp_rank, a.tp_world, a.tp_npad = self.tp_rank, self.tp_world, self.tp.npad
            a.vocab_offset = eng.vocab_offset
            a.tp_bufs, a.tp_flags, a.tp_keys, a.tp_kflags = (p.data_ptr() for p in self.tp.ptrs)
            a.tp_epoch = self.tp.epoch.data_ptr()
        if self.prof is not None:
            a.prof = self.prof.data_ptr()
        return a

    def profile(self, reset: bool = True):
        """Mean cycles per CTA of each counter since the last reset: x staging, waits for weight stages, stage
        math, grid barriers, attention (consumer thread 0), producer stalls on a full ring, tile reduction +
        epilogue, kernel lifetime."""
        if self.prof is None:
            return None
        names = ("stage_x", "wait_weights", "stage_math", "grid_barrier", "attention", "producer_stall",
                 "tile_reduce", "total")
        v = self.prof.view(self.grid, 8).double().mean(dim=0).tolist()
        mx = self.prof.view(self.grid, 8).max(dim=0).values.tolist()
        if reset:
            self.prof.zero_()
        return {n: (m, int(x)) for n, m, x in zip(names, v, mx)}

    def reset(self):
        """Clear the kernel's counters after a reported error (a completed launch leaves them clear itself)."""
        self.sync.zero_()
        self.counters.zero_()
        self.amax.zero_()

    def step(self, B: int):
        """Enqueue one decode step for ``B`` sequences on the current stream: ``tokens[:B]`` in, next tokens out,
        ``past_len[:B]`` advanced, ``logits[:B]`` filled."""
        key = (B, self._nsplit(B))
        a = self._args.get(key)
        if a is None or self._layer_tab is None or self._layer_tab[0] is not self.eng.cache:
            a = self._build(B)
            self._args[key] = a
        rc = self.lib.ipex_decode_mega(ctypes.byref(a), self.wf, api.dtype_code(self.eng.dtype), self.kmax, self.grid,
                                       int(self.coop), current_stream())
        api.check(rc, "decode_mega")
