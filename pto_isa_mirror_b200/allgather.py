"""AllGather + GEMM across the GPUs of one node (one process per GPU), one kernel launch per rank and step.

Reference shape of the computation: kernels/manual/a2a3/allgather_gemm (README.md:28-60): every rank holds an M slice
of A, B is replicated, every rank computes the whole C = A @ B; the communication kernel pushes chunks of A to the
other ranks and counts them (allgather_gemm_comm_kernel.cpp), the compute kernel multiplies its local rows first and
waits per chunk for the remote ones (allgather_gemm_compute_kernel.cpp), both running at once on two streams.

Here both halves are one persistent kernel (``pto_b200_allgather_gemm``): four extra warps per CTA push this rank's
slice block by block into every rank's copy of A - through the NVSwitch multicast address when the platform maps one,
else with one store per peer - and the tile loop's TMA loads wait for a remote block's flag before they touch it.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


BLOCK_ROWS = 256   # rows of A one arrival flag covers: one row of 256 x 256 output tiles


def slice_rows(m: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [r0, r1) of A that rank ``rank`` owns: m / world consecutive rows, a whole number of 256-row blocks."""
    if world < 1 or not 0 <= rank < world or m % (BLOCK_ROWS * world):
        raise ValueError("m must be a multiple of 256 * ranks")
    rows = m // world
    return rank * rows, (rank + 1) * rows


def block_schedule(m: int, world: int, rank: int) -> list[tuple[int, int]]:
    """The order in which rank ``rank``'s tile loop visits the 256-row blocks of A, as (block, owner) pairs: the raster
    is rotated so that the rank's own blocks come first (they need no arrival flag) and the remote ones follow in the
    order their owners push them."""
    r0, _ = slice_rows(m, world, rank)
    blocks = m // BLOCK_ROWS
    per_rank = blocks // world
    first = r0 // BLOCK_ROWS
    return [((first + i) % blocks, ((first + i) % blocks) // per_rank) for i in range(blocks)]


class AllGatherGemm:
    """``a_local()`` is this rank's slice of the symmetric A buffer: write the slice there, then ``step(b_dn)``.

    Without an initialised process group the instance is a single rank on plain device memory (the whole A is the
    local slice): the one-GPU test and profiling form of the same kernel.
    """

    def __init__(self, m: int, n: int, k: int, dtype: torch.dtype = torch.bfloat16,
                 out_dtype: torch.dtype = torch.float32, group: Optional[dist.ProcessGroup] = None,
                 device: Optional[torch.device] = None, launch_block_count: int = 0, use_multicast: bool = True):
        import ctypes

        from . import _capi

        self._capi = _capi
        self.lib = _capi.load()
        self.distributed = dist.is_initialized()
        self.group = (group if group is not None else dist.group.WORLD) if self.distributed else None
        self.world_size = dist.get_world_size(self.group) if self.distributed else 1
        self.rank = dist.get_rank(self.group) if self.distributed else 0
        if self.world_size > 8:
            raise ValueError("at most 8 ranks (one NVSwitch domain)")
        if m % (256 * self.world_size) or k % 8:
            raise ValueError("m must be a multiple of 256 * ranks and k of 8")
        if dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("A and B are float16 or bfloat16")
        self.m, self.n, self.k = m, n, k
        self.dtype, self.out_dtype = dtype, out_dtype
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.launch_block_count = launch_block_count
        ws = self.world_size
        n_flags = m // 256 + 8
        if self.distributed:
            import torch.distributed._symmetric_memory as symm_mem

            self.a_full = symm_mem.empty((m, k), dtype=dtype, device=self.device)
            self.flags = symm_mem.empty((n_flags,), dtype=torch.int32, device=self.device)
            self.flags.zero_()
            torch.cuda.synchronize(self.device)
            h_a = symm_mem.rendezvous(self.a_full, self.group)
            h_f = symm_mem.rendezvous(self.flags, self.group)
            self._handles = (h_a, h_f)
            a_base = [int(h_a.buffer_ptrs[r]) for r in range(ws)]
            f_base = [int(h_f.buffer_ptrs[r]) for r in range(ws)]
            mc = int(getattr(h_a, "multicast_ptr", 0) or 0) if use_multicast else 0
        else:
            self.a_full = torch.empty((m, k), dtype=dtype, device=self.device)
            self.flags = torch.zeros((n_flags,), dtype=torch.int32, device=self.device)
            self._handles = ()
            a_base, f_base, mc = [self.a_full.data_ptr()], [self.flags.data_ptr()], 0
        PtrArray = ctypes.c_void_p * ws
        self._a_ptrs = PtrArray(*a_base)
        self._flag_ptrs = PtrArray(*f_base)
        self.multicast = bool(mc)
        self._mc_a = mc if mc else None
        self.block_counters = torch.zeros(max(1, m // (256 * ws)), dtype=torch.int32, device=self.device)
        self.done_counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.out = torch.empty((m, n), dtype=out_dtype, device=self.device)
        self.epoch = 0
        if self.distributed:
            dist.barrier(self.group)      # every rank's flags are zero and mapped before anyone pushes
        torch.cuda.synchronize(self.device)

    def a_local(self) -> torch.Tensor:
        r0, r1 = slice_rows(self.m, self.world_size, self.rank)
        return self.a_full[r0:r1]

    def step(self, b_dn: torch.Tensor) -> torch.Tensor:
        """b_dn: B column-major [n, k], identical on every rank. Returns this rank's C [m, n] (rewritten by the next step)."""
        from .gemm import _TORCH_TO_PTO, _require_cuda_2d

        _require_cuda_2d(b_dn, "b_dn")
        if b_dn.dtype != self.dtype or tuple(b_dn.shape) != (self.n, self.k):
            raise ValueError("b_dn must be [n, k] of the operand dtype")
        self.epoch += 1
        stream = torch.cuda.current_stream(self.device)
        rc = self.lib.pto_b200_allgather_gemm(
            stream.cuda_stream, self.out.data_ptr(), self._a_ptrs, b_dn.data_ptr(), self.m, self.n, self.k,
            self.a_full.stride(0), b_dn.stride(0), self.out.stride(0), _TORCH_TO_PTO[self.dtype],
            _TORCH_TO_PTO[self.out_dtype], self._flag_ptrs, self.block_counters.data_ptr(),
            self.done_counter.data_ptr(), self.world_size, self.rank, self.epoch, self._mc_a, self.launch_block_count)
        self._capi.check(rc, "pto_b200_allgather_gemm")
        return self.out

    def release(self):
        """Drop the symmetric buffers; call on every rank at the same point with nothing in flight."""
        torch.cuda.synchronize(self.device)
        for name in ("a_full", "flags", "_handles"):
            if hasattr(self, name):
                delattr(self, name)
