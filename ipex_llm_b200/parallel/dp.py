"""Data-parallel training of the (small) trainable parameter set of a LoRA run.

The reference relies on HF ``Trainer`` DDP over oneCCL or on DeepSpeed ZeRO-2/3 with ``torch.optim.AdamW``
(python/llm/example/GPU/LLM-Finetuning/QLoRA/alpaca-qlora/alpaca_qlora_finetuning.py:242-272,
``deepspeed_zero2.json``).  Here every trainable tensor lives in one flat, peer-mapped buffer (parameters and
gradients), optimizer state is sharded over the ranks, and one kernel per step does
reduce-scatter + AdamW + all-gather over NVLink (``native/cuda/lora_rs_adamw.cu``).

``FusedLoraAdamW`` : the optimizer (works on one GPU too: fused flat AdamW; and on CPU with a PyTorch restatement
                     and ``dist.all_reduce`` so that host logic is testable on gloo ranks).
``PagedAdamW``     : single-process AdamW whose state pages live in pinned host memory and stream through the GPU
                     in chunks (``optim="paged_adamw"``; the reference notes paged optimizers as unsupported,
                     .../QLoRA/simple-example/qlora_finetuning.py:106).
"""
from __future__ import annotations

from typing import Iterable, List

import torch
import torch.distributed as dist

from ..utils.common import invalidInputError

_ALIGN = 8  # elements per 16-byte vector of the narrowest dtype handled (bf16)


def _world(group):
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


class FusedLoraAdamW(torch.optim.Optimizer):
    """AdamW over a flat parameter space with sharded state and a fused reduce-scatter/update/all-gather step.

    After construction every parameter is a view into ``self.flat_params`` and its ``.grad`` a view into
    ``self.flat_grads`` (gradients accumulate there; ``zero_grad`` clears the buffer).  Gradients are averaged over
    the ranks.  ``max_grad_norm`` clips each replica's gradient before the reduction.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], lr=2e-4, betas=(0.9, 0.999), eps=1e-8,
                 weight_decay=0.0, max_grad_norm: float = 0.0, group=None):
        plist = [p for p in params if p.requires_grad]
        invalidInputError(len(plist) > 0, "FusedLoraAdamW got no trainable parameters")
        dt = plist[0].dtype
        invalidInputError(all(p.dtype == dt for p in plist), "all trainable parameters must share one dtype")
        invalidInputError(dt in (torch.bfloat16, torch.float16, torch.float32), f"unsupported dtype {dt}")
        super().__init__(plist, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.group = group
        self.rank, self.world = _world(group)
        self.device = plist[0].device
        self.dtype = dt
        self.max_grad_norm = max_grad_norm
        self._step = 0
        n = sum(p.numel() for p in plist)
        unit = self.world * _ALIGN
        self.n = (n + unit - 1) // unit * unit
        self.shard = self.n // self.world
        self._alloc_flat()
        # re-home parameters and gradients
        off = 0
        with torch.no_grad():
            for p in plist:
                k = p.numel()
                view = self.flat_params[off:off + k].view_as(p)
                view.copy_(p.data)
                p.data = view
                p.grad = self.flat_grads[off:off + k].view_as(p)
                off += k
        lo = self.rank * self.shard
        self.master = self.flat_params[lo:lo + self.shard].float().clone()
        self.exp_avg = torch.zeros(self.shard, dtype=torch.float32, device=self.device)
        self.exp_avg_sq = torch.zeros(self.shard, dtype=torch.float32, device=self.device)
        self._plist = plist

    # ------------------------------------------------------------------------------------------------
    def _alloc_flat(self):
        cuda = self.device.type == "cuda"
        if cuda and self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            es = torch.empty(0, dtype=self.dtype).element_size()
            counters = 2 * 64 * 4
            self._symm = symm_mem.empty(2 * self.n * es + counters, dtype=torch.uint8, device=self.device)
            self._symm.zero_()
            torch.cuda.synchronize()
            grp = self.group if self.group is not None else dist.group.WORLD
            try:
                handle = symm_mem.rendezvous(self._symm, grp)
            except Exception:  # noqa: BLE001 (older signatures take the group name)
                handle = symm_mem.rendezvous(self._symm, grp.group_name)
            self._handle = handle
            bases = [int(p) for p in handle.buffer_ptrs]
            self.flat_params = self._symm[: self.n * es].view(self.dtype)
            self.flat_grads = self._symm[self.n * es: 2 * self.n * es].view(self.dtype)

            def arr(off):
                return torch.tensor([b + off for b in bases], dtype=torch.int64, device=self.device)

            self._p_ptrs, self._g_ptrs = arr(0), arr(self.n * es)
            self._fa, self._fb = arr(2 * self.n * es), arr(2 * self.n * es + 64 * 4)
            dist.barrier(group=self.group)
        else:
            self.flat_params = torch.zeros(self.n, dtype=self.dtype, device=self.device)
            self.flat_grads = torch.zeros(self.n, dtype=self.dtype, device=self.device)
            if cuda:
                self._p_ptrs = torch.tensor([self.flat_params.data_ptr()], dtype=torch.int64, device=self.device)
                self._g_ptrs = torch.tensor([self.flat_grads.data_ptr()], dtype=torch.int64, device=self.device)
                self._fa = self._fb = None

    def zero_grad(self, set_to_none: bool = False):
        self.flat_grads.zero_()
        # keep the views attached: autograd accumulates into them in place
        off = 0
        for p in self._plist:
            k = p.numel()
            if p.grad is None or p.grad.data_ptr() != self.flat_grads[off:off + k].data_ptr():
                p.grad = self.flat_grads[off:off + k].view_as(p)
            off += k

    def _reattach_grads(self):
        """Autograd may have replaced ``.grad`` with a fresh tensor (first backward): copy it into the flat buffer."""
        off = 0
        for p in self._plist:
            k = p.numel()
            view = self.flat_grads[off:off + k].view_as(p)
            if p.grad is not None and p.grad.data_ptr() != view.data_ptr():
                view.copy_(p.grad)
                p.grad = view
            off += k

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        self._reattach_grads()
        self._step += 1
        g = self.param_groups[0]
        lr, (b1, b2), eps, wd = g["lr"], g["betas"], g["eps"], g["weight_decay"]
        if self.max_grad_norm and self.max_grad_norm > 0:
            # Clip by the global norm of the AVERAGED gradient, as DDP + clip_grad_norm_ does.  The fused kernel
            # reduces and updates in one pass, so the average is formed first (one extra all-reduce, only when
            # clipping is on); every rank then holds the same clipped gradient and the kernel's own averaging of
            # the world's copies leaves it unchanged.
            if self.world > 1:
                dist.all_reduce(self.flat_grads, group=self.group)
                self.flat_grads.div_(self.world)
            norm = torch.linalg.vector_norm(self.flat_grads.float())
            self.flat_grads.mul_(torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0).to(self.dtype))
        if self.device.type == "cuda":
            self._step_cuda(lr, b1, b2, eps, wd)
        else:
            self._step_host(lr, b1, b2, eps, wd)
        return loss

    def _step_cuda(self, lr, b1, b2, eps, wd):
        from ..native import cuda_api as api
        from ..native.lib import cuda_lib, current_stream, ptr
        from ..ops.cuda_ops import error_flag
        if not hasattr(self, "_scale"):
            self._scale = torch.full((1,), 1.0 / self.world, dtype=torch.float32, device=self.device)
        blocks = max(1, min(64, (self.shard + 4095) // 4096))
        rc = cuda_lib().ipex_lora_rs_adamw(ptr(self._g_ptrs), ptr(self._p_ptrs), ptr(self._fa), ptr(self._fb),
                                           ptr(self.master), ptr(self.exp_avg), ptr(self.exp_avg_sq),
                                           ptr(self._scale), self.shard, self.rank, self.world, float(lr), float(b1),
                                           float(b2), float(eps), float(wd), self._step, api.dtype_code(self.dtype),
                                           blocks, ptr(error_flag(self.device)), current_stream())
        api.check(rc, "lora_rs_adamw")

    def _step_host(self, lr, b1, b2, eps, wd):
        """PyTorch restatement of the kernel (CPU / gloo): same sharding, same arithmetic order."""
        grads = self.flat_grads.float()
        if self.world > 1:
            dist.all_reduce(grads, group=self.group)
        lo = self.rank * self.shard
        gsh = grads[lo:lo + self.shard] / self.world
        self.exp_avg.mul_(b1).add_(gsh, alpha=1 - b1)
        self.exp_avg_sq.mul_(b2).addcmul_(gsh, gsh, value=1 - b2)
        bc1, bc2 = 1 - b1 ** self._step, 1 - b2 ** self._step
        self.master.mul_(1 - lr * wd)
        self.master.addcdiv_(self.exp_avg, (self.exp_avg_sq / bc2).sqrt_().add_(eps), value=-lr / bc1)
        new = self.master.to(self.dtype)
        if self.world > 1:
            parts = [torch.empty_like(new) for _ in range(self.world)]
            dist.all_gather(parts, new, group=self.group)
            self.flat_params.copy_(torch.cat(parts))
        else:
            self.flat_params.copy_(new)

    # state for checkpoint / resume -------------------------------------------------------------------
    def state_dict(self):
        return {"step": self._step, "master": self.master.cpu(), "exp_avg": self.exp_avg.cpu(),
                "exp_avg_sq": self.exp_avg_sq.cpu(), "rank": self.rank, "world": self.world,
                "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}

    def load_state_dict(self, sd):
        invalidInputError(sd["world"] == self.world, "optimizer shards were saved with another world size")
        self._step = sd["step"]
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        for g, s in zip(self.param_groups, sd["param_groups"]):
            g.update(s)
        lo = self.rank * self.shard
        self.flat_params[lo:lo + self.shard].copy_(self.master.to(self.dtype))


class PagedAdamW(torch.optim.Optimizer):
    """AdamW whose moments live in pinned host pages and stream through the device page by page.

    For models whose optimizer state does not fit beside the weights (the reference leaves this to DeepSpeed's
    optimizer offload, python/llm/example/GPU/LLM-Finetuning/QLoRA/alpaca-qlora/deepspeed_zero2.json).  A step
    walks the parameters in pages of at most ``page_elems`` values.  On CUDA the pages are double buffered: a copy
    stream brings the moments of page i + 1 to the device and takes the new moments of page i - 1 back to the host
    while the current stream updates page i; events order the two streams per buffer.  On CPU tensors the same
    arithmetic runs in place.
    """

    def __init__(self, params, lr=2e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, page_elems: int = 1 << 22):
        plist = [p for p in params if p.requires_grad]
        super().__init__(plist, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.page_elems = page_elems
        self._step = 0
        self._host = {}
        pin = torch.cuda.is_available()
        for p in plist:
            self._host[p] = (torch.zeros(p.numel(), dtype=torch.float32, pin_memory=pin),
                             torch.zeros(p.numel(), dtype=torch.float32, pin_memory=pin))
        self._bufs = None
        self._copy = None

    @staticmethod
    def _update(flat_p, flat_g, m, v, lo, hi, lr, b1, b2, eps, wd, bc1, bc2):
        gr = flat_g[lo:hi].float()
        m.mul_(b1).add_(gr, alpha=1 - b1)
        v.mul_(b2).addcmul_(gr, gr, value=1 - b2)
        w = flat_p[lo:hi].float()
        w.mul_(1 - lr * wd).addcdiv_(m, (v / bc2).sqrt_().add_(eps), value=-lr / bc1)
        flat_p[lo:hi].copy_(w)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        self._step += 1
        items = []          # (param, lo, hi, hyper-parameters)
        for g in self.param_groups:
            lr, (b1, b2), eps, wd = g["lr"], g["betas"], g["eps"], g["weight_decay"]
            bc1, bc2 = 1 - b1 ** self._step, 1 - b2 ** self._step
            for p in g["params"]:
                if p.grad is None:
                    continue
                for lo in range(0, p.numel(), self.page_elems):
                    items.append((p, lo, min(lo + self.page_elems, p.numel()), (lr, b1, b2, eps, wd, bc1, bc2)))
        if not items:
            return loss
        dev = items[0][0].device
        if dev.type != "cuda":
            for p, lo, hi, hp in items:
                hm, hv = self._host[p]
                self._update(p.data.view(-1), p.grad.view(-1), hm[lo:hi], hv[lo:hi], lo, hi, *hp)
            return loss
        if self._bufs is None or self._bufs[0][0].device != dev:
            self._bufs = [tuple(torch.empty(self.page_elems, dtype=torch.float32, device=dev) for _ in range(2))
                          for _ in range(2)]
            self._copy = torch.cuda.Stream(device=dev)
            self._ready = [torch.cuda.Event() for _ in range(2)]
            self._done = [torch.cuda.Event() for _ in range(2)]
        cur, cp = torch.cuda.current_stream(dev), self._copy
        cp.wait_stream(cur)                      # the gradients and the previous step's use of the buffers

        def load(i):
            p, lo, hi, _ = items[i]
            hm, hv = self._host[p]
            m, v = self._bufs[i % 2]
            with torch.cuda.stream(cp):
                m[: hi - lo].copy_(hm[lo:hi], non_blocking=True)
                v[: hi - lo].copy_(hv[lo:hi], non_blocking=True)
                self._ready[i % 2].record(cp)

        load(0)
        for i, (p, lo, hi, hp) in enumerate(items):
            slot = i % 2
            if i + 1 < len(items):
                load(i + 1)                      # queued behind the write-back that frees that buffer (same stream)
            cur.wait_event(self._ready[slot])
            m, v = self._bufs[slot]
            self._update(p.data.view(-1), p.grad.view(-1), m[: hi - lo], v[: hi - lo], lo, hi, *hp)
            self._done[slot].record(cur)
            hm, hv = self._host[p]
            with torch.cuda.stream(cp):
                cp.wait_event(self._done[slot])
                hm[lo:hi].copy_(m[: hi - lo], non_blocking=True)
                hv[lo:hi].copy_(v[: hi - lo], non_blocking=True)
        cur.wait_stream(cp)
        cp.synchronize()                         # host pages are complete when step() returns
        return loss
