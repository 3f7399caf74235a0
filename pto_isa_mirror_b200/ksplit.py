"""K-split GEMM + allreduce across the GPUs of one node (one process per GPU).

Reference shape of the computation: kernels/manual/a2a3/gemm_ar (README.md:33-46): every rank multiplies its
own K slice (the compute kernel takes a ``k_per_rank`` stride, gemm_compute_kernel.cpp:150-165), the fp32
partials are summed across ranks (reduce-scatter by atomic add into the owner's window, comm_kernel.cpp:165-210),
and every rank ends with the full result (all-gather, comm_kernel.cpp:377-400), compute and communication running
on two streams (main.cpp:761-800).

Here rank r computes P_r = A[:, K_r] @ B[K_r, :] with the tcgen05 tile loop, panel by panel over M, and each
panel's fp32 partial is reduced across the ranks while later panels are being multiplied; the reduced panel is cast
to bf16 (the TSTORE cast). Three implementations, fastest first:

* :class:`KSplitGemmFused`  - one kernel launch per step: the GEMM's own extra warps exchange the finished panels
  over peer memory (NVSwitch multimem or plain peer loads);
* :class:`KSplitGemmP2P`    - one GEMM launch per panel plus this library's reduction kernels on a second stream;
* :class:`KSplitGemmAllReduce` - the same panel pipeline with NCCL collectives (the baseline), two reductions:

* ``"allreduce"``: ncclAllReduce(fp32 sum) then cast;
* ``"rs_ag"``    : reduce-scatter (fp32) -> cast of the owned shard -> all-gather (bf16), which moves 25 % fewer
  bytes per GPU than the fp32 allreduce.

The result is bf16(sum_r P_r); the order of the cross-rank sum is NCCL's, so parity is by tolerance (1e-3).
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch
import torch.distributed as dist


def panel_bounds(m: int, panels: int, align: int) -> List[tuple]:
    """Split [0, m) into at most ``panels`` contiguous row ranges whose sizes are multiples of ``align``
    (the last takes the remainder). Empty ranges are dropped."""
    if m <= 0:
        return []
    panels = max(1, panels)
    per = -(-m // panels)
    per = -(-per // align) * align
    out = []
    r0 = 0
    while r0 < m:
        r1 = min(m, r0 + per)
        out.append((r0, r1))
        r0 = r1
    return out


def panels_from_rows(m: int, rows: List[int], align: int) -> List[tuple]:
    """Row panels of the given heights (each a multiple of ``align``; the last one absorbs what is left of m)."""
    out, r0 = [], 0
    for h in rows:
        if h <= 0 or h % align:
            raise ValueError(f"panel height {h} is not a positive multiple of {align}")
        if r0 >= m:
            break
        out.append((r0, min(m, r0 + h)))
        r0 += h
    if r0 < m:
        out.append((r0, m))
    return out


def k_slice(k: int, world_size: int, rank: int) -> tuple:
    """The K range owned by ``rank``: K is partitioned evenly (the benchmark's K-split configuration)."""
    if k % world_size != 0:
        raise ValueError(f"K={k} is not divisible by {world_size} ranks")
    kr = k // world_size
    return rank * kr, (rank + 1) * kr


class KSplitGemmAllReduce:
    """Pipelined per-rank GEMM + cross-rank reduction + bf16 cast.

    ``gemm_fn(a, b_dn, out_f32)`` and ``cast_fn(src_f32, out_bf16)`` default to the CUDA library; the CPU tests
    pass stand-ins so the scheduling, slicing and collective logic run under gloo without a GPU.
    """

    def __init__(self, m: int, n: int, group: Optional[dist.ProcessGroup] = None, panels: int = 4,
                 mode: str = "rs_ag", device: Optional[torch.device] = None,
                 gemm_fn: Optional[Callable] = None, cast_fn: Optional[Callable] = None, single_rank: bool = False,
                 launch_block_count: int = 0):
        if mode not in ("allreduce", "rs_ag"):
            raise ValueError("mode must be 'allreduce' or 'rs_ag'")
        self.m, self.n = m, n
        self.group = group
        # single_rank: this instance multiplies the unsplit product on its own GPU and issues no collective, even
        # inside an initialised process group (the one-GPU base case measured next to a multi-rank run)
        distributed = dist.is_initialized() and not single_rank
        self.world_size = dist.get_world_size(group) if distributed else 1
        self.rank = dist.get_rank(group) if distributed else 0
        self.mode = mode if self.world_size > 1 else "allreduce"
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.on_cuda = self.device.type == "cuda"
        # panel rows are multiples of 128 * world_size so that tiles and reduce-scatter shards both divide evenly
        self.panels = panel_bounds(m, panels, 128 * self.world_size)
        if self.mode == "rs_ag" and any((r1 - r0) % self.world_size for r0, r1 in self.panels):
            self.mode = "allreduce"
        if gemm_fn is None or cast_fn is None:
            from .gemm import cast_f32_to_bf16 as _cast
            from .gemm import gemm as _gemm

            # launch_block_count: SMs the GEMM may occupy while a reduction runs beside it (0 = all)
            lbc = launch_block_count if self.world_size > 1 else 0
            gemm_fn = gemm_fn or (lambda a, b, out: _gemm(a, b, out=out, launch_block_count=lbc))
            cast_fn = cast_fn or (lambda src, out: _cast(src, out=out))
        self.gemm_fn, self.cast_fn = gemm_fn, cast_fn
        self.partial = torch.empty((m, n), dtype=torch.float32, device=self.device)
        if self.mode == "rs_ag":
            max_rows = max(r1 - r0 for r0, r1 in self.panels) // self.world_size
            self.shard_f32 = torch.empty((max_rows, n), dtype=torch.float32, device=self.device)
            self.shard_bf16 = torch.empty((max_rows, n), dtype=torch.bfloat16, device=self.device)
        if self.on_cuda:
            self.comm_stream = torch.cuda.Stream(device=self.device)
            self.events = [torch.cuda.Event() for _ in self.panels]
            self.shard_free = torch.cuda.Event()

    def step(self, a_slice: torch.Tensor, b_slice_dn: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """a_slice [m, K/ranks], b_slice_dn [n, K/ranks] (strided views of the full operands are fine),
        out [m, n] bf16 contiguous. Enqueues everything; the caller's current stream ends up waiting for the result."""
        assert tuple(out.shape) == (self.m, self.n) and out.is_contiguous()
        if not self.on_cuda:
            return self._step_serial(a_slice, b_slice_dn, out)
        main = torch.cuda.current_stream(self.device)
        self.comm_stream.wait_stream(main)
        for i, (r0, r1) in enumerate(self.panels):
            self.gemm_fn(a_slice[r0:r1], b_slice_dn, self.partial[r0:r1])
            self.events[i].record(main)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(self.events[i])
                self._reduce_panel(r0, r1, out)
        main.wait_stream(self.comm_stream)
        return out

    def _reduce_panel(self, r0: int, r1: int, out: torch.Tensor) -> None:
        part = self.partial[r0:r1]
        if self.world_size == 1:
            self.cast_fn(part, out[r0:r1])
        elif self.mode == "allreduce":
            dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
            self.cast_fn(part, out[r0:r1])
        else:
            rows = (r1 - r0) // self.world_size
            shard = self.shard_f32[:rows]
            shard16 = self.shard_bf16[:rows]
            dist.reduce_scatter_tensor(shard, part, op=dist.ReduceOp.SUM, group=self.group)
            self.cast_fn(shard, shard16)
            dist.all_gather_into_tensor(out[r0:r1], shard16, group=self.group)

    def _step_serial(self, a_slice, b_slice_dn, out):
        for r0, r1 in self.panels:
            self.gemm_fn(a_slice[r0:r1], b_slice_dn, self.partial[r0:r1])
            self._reduce_panel(r0, r1, out)
        return out


class KSplitGemmP2P:
    """K-split GEMM with the reduction done by this library's own kernels over peer memory (NVLink / NVSwitch).

    The structure is the reference's (kernels/manual/a2a3/gemm_ar): symmetric buffers mapped into every rank
    (its HCCL windows; here torch symmetric memory), a per-rank GEMM stream and a communication stream
    (main.cpp:761-800), reduce-scatter into the owner of each row shard followed by an all-gather of the finished
    shard (comm_kernel.cpp:165-210, 377-400), and flag counters between the two (comm_kernel.cpp:111-123, 528-590).
    Per row panel: GEMM -> fp32 partial in this rank's symmetric buffer -> ready flag to every rank; on the second
    stream the owner of each shard pulls that shard from every rank, sums in rank order, casts to bf16 and pushes the
    result into every rank's output, so a panel's reduction runs under the next panel's GEMM. No NCCL call is made
    on the data path. Partials are double-buffered by step parity, so a rank never overwrites a partial that a
    slower peer may still be reading.

    ``step`` returns this rank's output buffer (symmetric memory, rewritten by the next ``step``).
    """

    def __init__(self, m: int, n: int, group: Optional[dist.ProcessGroup] = None, panels: int = 4,
                 device: Optional[torch.device] = None, reduce_blocks: int = 32, launch_block_count: int = 0,
                 panel_rows: Optional[List[int]] = None, reduce_blocks_last: int = 0, use_multicast: bool = True,
                 gemm_streams: int = 2):
        """``panels`` equal row panels, or explicit ``panel_rows`` heights (decreasing heights leave only a small
        reduction exposed after the last GEMM). ``reduce_blocks`` thread blocks run each reduction beside the next
        GEMM; ``reduce_blocks_last`` (0 = four times that) run the last one, which has the GPU to itself."""
        if not dist.is_initialized():
            raise RuntimeError("KSplitGemmP2P needs an initialised process group (one process per GPU)")
        self._setup_ranks(group, device, m, n)
        align = 128 * self.world_size
        self.panels = panels_from_rows(m, panel_rows, align) if panel_rows else panel_bounds(m, panels, align)
        if any((r1 - r0) % self.world_size for r0, r1 in self.panels) or n % 4:
            raise ValueError("panel rows must divide by the rank count and n by 4")
        self.reduce_blocks = reduce_blocks
        self.reduce_blocks_last = reduce_blocks_last if reduce_blocks_last > 0 else 4 * reduce_blocks
        self.launch_block_count = launch_block_count
        self._allocate(use_multicast)
        self.cta_counters = torch.zeros(self.num_slots, dtype=torch.int32, device=self.device)
        self.comm_stream = torch.cuda.Stream(device=self.device)
        # With two GEMM streams consecutive panels' persistent GEMM kernels overlap at their edges: the CTAs of panel
        # p+1 start on the SMs that ran out of tiles in the last wave of panel p, so the partly filled last wave is
        # paid once per step instead of once per panel.
        self.aux_stream = torch.cuda.Stream(device=self.device) if gemm_streams > 1 else None
        self.events = [torch.cuda.Event() for _ in self.panels]
        self.start_event = torch.cuda.Event()
        self._ready_to_start()

    # ---------------------------------------------------------------- shared set-up of the peer-memory variants
    def _setup_ranks(self, group, device, m, n):
        import ctypes

        from . import _capi

        self._ctypes = ctypes
        self._capi = _capi
        self.lib = _capi.load()
        self.distributed = dist.is_initialized()
        self.group = (group if group is not None else dist.group.WORLD) if self.distributed else None
        self.world_size = dist.get_world_size(self.group) if self.distributed else 1
        self.rank = dist.get_rank(self.group) if self.distributed else 0
        if self.world_size > 8:
            raise ValueError("at most 8 ranks (one NVSwitch domain)")
        self.m, self.n = m, n
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())

    def _allocate(self, use_multicast: bool):
        """Two fp32 partial buffers (alternating by step), the bf16 output and the ready / done flags, mapped into
        every rank (torch symmetric memory); a single process without a process group gets plain device memory."""
        ctypes = self._ctypes
        m, n, ws = self.m, self.n, self.world_size
        self.num_slots = 2 * len(self.panels)
        if self.distributed:
            import torch.distributed._symmetric_memory as symm_mem

            self.partial = symm_mem.empty((2, m, n), dtype=torch.float32, device=self.device)
            self.out = symm_mem.empty((m, n), dtype=torch.bfloat16, device=self.device)
            self.flags = symm_mem.empty((2, self.num_slots, 8), dtype=torch.int32, device=self.device)
            self.flags.zero_()
            torch.cuda.synchronize(self.device)
            h_partial = symm_mem.rendezvous(self.partial, self.group)
            h_out = symm_mem.rendezvous(self.out, self.group)
            h_flags = symm_mem.rendezvous(self.flags, self.group)
            self._handles = (h_partial, h_out, h_flags)
            partial_base = [int(h_partial.buffer_ptrs[r]) for r in range(ws)]
            out_base = [int(h_out.buffer_ptrs[r]) for r in range(ws)]
            flag_base = [int(h_flags.buffer_ptrs[r]) for r in range(ws)]
            # NVSwitch multicast addresses (NVLS) of the partial and output buffers, when the platform maps them:
            # the reduction then happens inside the switch (multimem.ld_reduce), the result is broadcast by one store
            mc_p = int(getattr(h_partial, "multicast_ptr", 0) or 0) if use_multicast else 0
            mc_o = int(getattr(h_out, "multicast_ptr", 0) or 0) if use_multicast else 0
        else:
            self.partial = torch.empty((2, m, n), dtype=torch.float32, device=self.device)
            self.out = torch.empty((m, n), dtype=torch.bfloat16, device=self.device)
            self.flags = torch.zeros((2, self.num_slots, 8), dtype=torch.int32, device=self.device)
            self._handles = ()
            partial_base, out_base, flag_base = [self.partial.data_ptr()], [self.out.data_ptr()], [self.flags.data_ptr()]
            mc_p = mc_o = 0
        PtrArray = ctypes.c_void_p * ws
        pbytes = m * n * 4
        fbytes = self.num_slots * 8 * 4
        self._partial_ptrs = [PtrArray(*[base + b * pbytes for base in partial_base]) for b in (0, 1)]
        self._out_ptrs = PtrArray(*out_base)
        self._ready_ptrs = PtrArray(*flag_base)
        self._done_ptrs = PtrArray(*[base + fbytes for base in flag_base])
        self.multicast = bool(mc_p and mc_o)
        self._mc_partial = [mc_p + b * pbytes if self.multicast else None for b in (0, 1)]
        self._mc_out = mc_o if self.multicast else None
        self._ready_local = self.flags[0].data_ptr()
        self._done_local = self.flags[1].data_ptr()
        self.epoch = 0

    def _ready_to_start(self):
        if self.distributed:
            dist.barrier(self.group)      # every rank's flags are zero and mapped before anyone signals
        torch.cuda.synchronize(self.device)

    def release(self):
        """Drop the symmetric buffers. Call on every rank at the same point (after a barrier, nothing in flight): the
        peers' mappings, and the NVSwitch multicast bindings, then go away together."""
        torch.cuda.synchronize(self.device)
        for name in ("partial", "out", "flags", "_handles"):
            if hasattr(self, name):
                delattr(self, name)

    def step(self, a_slice: torch.Tensor, b_slice_dn: torch.Tensor) -> torch.Tensor:
        from .gemm import gemm as _gemm

        lib, check = self.lib, self._capi.check
        self.epoch += 1
        buf = self.epoch & 1
        partial = self.partial[buf]
        main = torch.cuda.current_stream(self.device)
        ws, rank, npan = self.world_size, self.rank, len(self.panels)
        self.comm_stream.wait_stream(main)
        if self.aux_stream is not None:
            self.aux_stream.wait_stream(main)
        for i, (r0, r1) in enumerate(self.panels):
            slot = buf * npan + i
            gs = self.aux_stream if (self.aux_stream is not None and i % 2 == 1) else main
            _gemm(a_slice[r0:r1], b_slice_dn, out=partial[r0:r1], launch_block_count=self.launch_block_count, stream=gs)
            check(lib.pto_b200_ksplit_signal(gs.cuda_stream, self._ready_ptrs, ws, rank, slot, self.epoch),
                  "pto_b200_ksplit_signal")
            self.events[i].record(gs)
            self.comm_stream.wait_event(self.events[i])
            shard = (r1 - r0) // ws
            check(lib.pto_b200_ksplit_reduce(self.comm_stream.cuda_stream, self._partial_ptrs[buf], self._out_ptrs,
                                             self._done_ptrs, self._ready_local, self.cta_counters.data_ptr(), ws, rank,
                                             slot, self.epoch, r0 + rank * shard, shard, self.n, self.n, self.n,
                                             self.reduce_blocks_last if i == npan - 1 else self.reduce_blocks,
                                             self._mc_partial[buf], self._mc_out),
                  "pto_b200_ksplit_reduce")
        check(lib.pto_b200_ksplit_wait(self.comm_stream.cuda_stream, self._done_local, ws, buf * npan, npan, self.epoch),
              "pto_b200_ksplit_wait")
        main.wait_stream(self.comm_stream)
        return self.out


class KSplitGemmFused(KSplitGemmP2P):
    """K-split GEMM + allreduce as ONE kernel launch per rank and step (``pto_b200_ksplit_gemm_allreduce``).

    The reference runs its compute kernel and its communication kernel side by side on two streams and couples them
    with a device-side ready queue that the compute kernel fills tile by tile (kernels/manual/a2a3/gemm_ar/
    gemm_compute_kernel.cpp:150-240, comm_kernel.cpp:528-590). Here the two are one persistent kernel: the tile loop
    walks the output panel by panel, the warp that finishes a panel publishes the ready flag to every rank, and four
    extra warps per CTA reduce this rank's row shard of each ready panel over peer memory and deliver the bf16 result
    to every rank while the tensor cores work on later panels. Against one launch per panel this removes the partly
    filled last wave of every panel and all launch seams; only the last panel's exchange is exposed.

    Without an initialised process group the instance runs as a single rank on plain device memory (the exchange
    warps then cast this GPU's own partial): the one-GPU test and profiling form of the same kernel.
    """

    def __init__(self, m: int, n: int, group: Optional[dist.ProcessGroup] = None, panels: int = 8,
                 device: Optional[torch.device] = None, launch_block_count: int = 0, use_multicast: bool = True):
        self._setup_ranks(group, device, m, n)
        if n % 4:
            raise ValueError("n must be a multiple of 4")
        per = -(-m // max(1, panels))
        self.panel_rows = -(-per // 256) * 256          # whole 256-row tiles per panel
        self.panels = [(r0, min(m, r0 + self.panel_rows)) for r0 in range(0, m, self.panel_rows)]
        self.launch_block_count = launch_block_count
        self._allocate(use_multicast)
        self.panel_counters = torch.zeros(self.num_slots, dtype=torch.int32, device=self.device)
        self.exchange_counters = torch.zeros(self.num_slots, dtype=torch.int32, device=self.device)
        self._ready_to_start()

    def step(self, a_slice: torch.Tensor, b_slice_dn: torch.Tensor) -> torch.Tensor:
        from .gemm import _TORCH_TO_PTO, _require_cuda_2d

        _require_cuda_2d(a_slice, "a_slice")
        _require_cuda_2d(b_slice_dn, "b_slice_dn")
        if a_slice.dtype != b_slice_dn.dtype or a_slice.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError("operands must both be float16 or bfloat16")
        if a_slice.shape[0] != self.m or b_slice_dn.shape[0] != self.n or a_slice.shape[1] != b_slice_dn.shape[1]:
            raise ValueError("operand slices must be [m, k_local] and [n, k_local]")
        self.epoch += 1
        buf = self.epoch & 1
        stream = torch.cuda.current_stream(self.device)
        rc = self.lib.pto_b200_ksplit_gemm_allreduce(
            stream.cuda_stream, a_slice.data_ptr(), b_slice_dn.data_ptr(), self.m, self.n, a_slice.shape[1],
            a_slice.stride(0), b_slice_dn.stride(0), _TORCH_TO_PTO[a_slice.dtype], self._partial_ptrs[buf],
            self._out_ptrs, self._ready_ptrs, self._done_ptrs, self.panel_counters.data_ptr(),
            self.exchange_counters.data_ptr(), self.world_size, self.rank, buf * len(self.panels), self.epoch,
            self.panel_rows, self.n, self.n, self._mc_partial[buf], self._mc_out, self.launch_block_count)
        self._capi.check(rc, "pto_b200_ksplit_gemm_allreduce")
        return self.out
