"""Symmetric peer memory for the tensor-parallel kernels.

Stands in for the reference's oneCCL / ``deepspeed.comm`` backend (component N7: ``dist.init_process_group('ccl')``,
python/llm/src/ipex_llm/transformers/pipeline_parallel.py:108-112; ``inference_all_reduce`` in
low_bit_linear.py:680).  One NCCL process group is still used for bootstrap, pipeline p2p and as a fallback;
the latency-critical decode collectives run on a per-rank buffer that every peer maps (CUDA VMM through
``torch.distributed._symmetric_memory``), so a kernel can store into / load from any GPU of the node directly.

Layout of each rank's buffer, for each of two call parities:
  [ 64 block counters | 2048 tile counters | all-reduce staging (ar_bytes) | GEMV partials [world][8][npad] fp32 ]
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..native import cuda_api as api
from ..native.lib import cuda_lib, current_stream, ptr

_N_BLOCK_FLAGS = 64
_N_TILE_FLAGS = 4096


class SymmComm:
    _instances = {}

    @classmethod
    def get(cls, group=None):
        key = id(group) if group is not None else 0
        if key not in cls._instances:
            cls._instances[key] = cls(group)
        return cls._instances[key]

    def __init__(self, group=None, ar_bytes: int = 8 << 20, npad: int = 32768):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.ar_bytes = ar_bytes
        self.npad = npad
        self.flag_bytes = (_N_BLOCK_FLAGS + _N_TILE_FLAGS) * 4
        self.gemv_bytes = self.world * 8 * npad * 4
        self.parity_bytes = (self.flag_bytes + ar_bytes + self.gemv_bytes + 255) // 256 * 256
        total = 2 * self.parity_bytes
        self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize()
        try:
            self.handle = symm_mem.rendezvous(self.buf, self.group)
        except Exception:  # noqa: BLE001  (older signatures take the group name)
            name = self.group.group_name
            if hasattr(symm_mem, "enable_symm_mem_for_group"):
                symm_mem.enable_symm_mem_for_group(name)
            self.handle = symm_mem.rendezvous(self.buf, name)
        base_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        dist.barrier(group=self.group)

        def ptr_array(offset):
            return torch.tensor([p + offset for p in base_ptrs], dtype=torch.int64, device=self.device)

        self.block_flags, self.tile_flags, self.ar_bufs, self.gemv_bufs = [], [], [], []
        for par in range(2):
            o = par * self.parity_bytes
            self.block_flags.append(ptr_array(o))
            self.tile_flags.append(ptr_array(o + _N_BLOCK_FLAGS * 4))
            self.ar_bufs.append(ptr_array(o + self.flag_bytes))
            self.gemv_bufs.append(ptr_array(o + self.flag_bytes + ar_bytes))
        self._local_ar = [self.buf[par * self.parity_bytes + self.flag_bytes:
                                   par * self.parity_bytes + self.flag_bytes + ar_bytes] for par in range(2)]
        self._parity = 0
        from ..ops.cuda_ops import error_flag
        self.err = error_flag(self.device)

    # ------------------------------------------------------------------------------------------------
    def next_parity(self) -> int:
        """Every collective call (on every rank, in the same order) takes the next parity."""
        p = self._parity
        self._parity ^= 1
        return p

    def can_all_reduce(self, t: torch.Tensor) -> bool:
        return t.is_cuda and t.is_contiguous() and t.numel() * t.element_size() <= self.ar_bytes and \
            t.dtype in (torch.float16, torch.bfloat16, torch.float32)

    def all_reduce(self, t: torch.Tensor, pdl: bool = False) -> torch.Tensor:
        """In-place sum over the group through peer loads (one-shot: every rank reads every peer)."""
        lib = cuda_lib()
        par = self.next_parity()
        nbytes = t.numel() * t.element_size()
        stage = self._local_ar[par][:nbytes].view(t.dtype)
        stage.copy_(t.reshape(-1))
        blocks = max(1, min(_N_BLOCK_FLAGS, (t.numel() + 4095) // 4096))
        rc = lib.ipex_allreduce_oneshot(ptr(self.ar_bufs[par]), ptr(self.block_flags[par]), ptr(t), t.numel(),
                                        api.dtype_code(t.dtype), self.rank, self.world, ptr(self.err), blocks,
                                        int(pdl), current_stream())
        api.check(rc, "allreduce_oneshot")
        return t

    def ar_stage(self, numel: int, dtype):
        """Staging view for the NEXT all-reduce: a producer kernel (the row-parallel GEMV) writes this rank's
        contribution straight into symmetric memory, which saves the copy ``all_reduce`` starts with.  Returns
        ``(view, token)``; pass the token to ``all_reduce_staged``.  Takes this call's parity, so the pair counts as
        one collective in the per-rank call order."""
        par = self.next_parity()
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        return self._local_ar[par][:nbytes].view(dtype), par

    def all_reduce_staged(self, token: int, out: torch.Tensor, residual: torch.Tensor = None,
                          bias: torch.Tensor = None, pdl: bool = False) -> torch.Tensor:
        """Second half of ``ar_stage``: ``out = sum over ranks of the staged vectors (+ residual) (+ bias per
        column)``, in one kernel.  ``out`` and ``residual`` are contiguous and may be the same tensor."""
        lib = cuda_lib()
        n = out.numel()
        blocks = max(1, min(_N_BLOCK_FLAGS, (n + 4095) // 4096))
        rc = lib.ipex_allreduce_oneshot_epi(ptr(self.ar_bufs[token]), ptr(self.block_flags[token]), ptr(out), n,
                                            api.dtype_code(out.dtype), self.rank, self.world, ptr(self.err), blocks,
                                            int(pdl), ptr(residual), ptr(bias), out.shape[-1], current_stream())
        api.check(rc, "allreduce_oneshot_epi")
        return out

    def barrier(self):
        lib = cuda_lib()
        par = self.next_parity()
        rc = lib.ipex_symm_barrier(ptr(self.block_flags[par]), self.rank, self.world, ptr(self.err),
                                   current_stream())
        api.check(rc, "symm_barrier")

    def gemv_ar_args(self):
        """(rank, world, npad, bufs_ptr_array, tile_flags_ptr_array) for the next fused GEMV+all-reduce call."""
        par = self.next_parity()
        return self.rank, self.world, self.npad, self.gemv_bufs[par], self.tile_flags[par]

    # ------------------------------------------------------------------------------------------------
    def gemm_ar_args(self, stage_bytes: int, n_counters: int):
        """Staging + counters for the next GEMM fused with its all-reduce (``ipex_gemm_lowbit_tcgen05_ar``): returns
        ``(rank, world, stage_ptr_array, flag_ptr_array)`` for this call's parity.  The symmetric buffer is created
        on first use and grown when a larger product comes along; both are collective, so every rank must call this
        with the same sizes in the same order (they do: the ranks run the same layers on the same token count)."""
        import torch.distributed._symmetric_memory as symm_mem
        need_stage = (stage_bytes + 255) // 256 * 256
        need_flags = (n_counters * 4 + 255) // 256 * 256 + 256      # last 256 bytes: epoch flags of the all-gather
        cur = getattr(self, "_gemm_cap", (0, 0))
        if need_stage > cur[0] or need_flags > cur[1]:
            cap_stage = max(need_stage, cur[0], 32 << 20)
            cap_flags = max(need_flags, cur[1], 64 << 10)
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            per = cap_stage + cap_flags
            buf = symm_mem.empty(2 * per, dtype=torch.uint8, device=self.device)
            buf.zero_()
            torch.cuda.synchronize()
            try:
                handle = symm_mem.rendezvous(buf, self.group)
            except Exception:  # noqa: BLE001 (older signatures take the group name)
                handle = symm_mem.rendezvous(buf, self.group.group_name)
            bases = [int(p) for p in handle.buffer_ptrs]
            dist.barrier(group=self.group)
            self._gemm_buf, self._gemm_handle, self._gemm_cap = buf, handle, (cap_stage, cap_flags)
            self._gemm_stage, self._gemm_flags, self._gemm_ag_flags = [], [], []
            for par in range(2):
                o = par * per
                self._gemm_stage.append(torch.tensor([b + o for b in bases], dtype=torch.int64, device=self.device))
                self._gemm_flags.append(torch.tensor([b + o + cap_stage for b in bases], dtype=torch.int64,
                                                     device=self.device))
                self._gemm_ag_flags.append(torch.tensor([b + o + per - 256 for b in bases], dtype=torch.int64,
                                                        device=self.device))
            self._gemm_local = [(bases[self.rank] + par * per, bases[self.rank] + par * per + per - 256)
                                for par in range(2)]
            self._gemm_parity = 0
            self._ag_epoch = 0          # the fresh buffer holds zeros: epochs restart (same on every rank)
        par = self._gemm_parity
        self._gemm_parity ^= 1
        return self.rank, self.world, self._gemm_stage[par], self._gemm_flags[par]

    def gemm_ag_args(self, gather_bytes: int):
        """Buffers for the next GEMM whose activation is all-gathered inside the kernel
        (``ipex_gemm_lowbit_tcgen05_ag``): returns ``(rank, world, local_gather_ptr, gather_ptr_array,
        flag_ptr_array, local_flags_ptr, ticket_ptr, epoch)``.  Shares the two-parity symmetric buffer (and the
        parity alternation) with the fused all-reduce GEMM, so consecutive fused ops never write the region a peer
        may still be reading.  Collective: same sizes, same order on every rank."""
        rank, world, stage, _ = self.gemm_ar_args(gather_bytes, 0)
        par = self._gemm_parity ^ 1                      # the parity gemm_ar_args just handed out
        self._ag_epoch += 1
        if getattr(self, "_ag_ticket", None) is None:
            self._ag_ticket = torch.zeros(1, dtype=torch.int32, device=self.device)
        local_gather, local_flags = self._gemm_local[par]
        return (rank, world, local_gather, stage, self._gemm_ag_flags[par], local_flags,
                self._ag_ticket.data_ptr(), self._ag_epoch)
