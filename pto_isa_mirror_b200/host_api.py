"""Host-buffer front end: what the reference's kernel ``main.cpp`` does around a launch.

kernels/manual/a2a3/gemm_performance/main.cpp:23-80 allocates device buffers, copies the two inputs host to
device, launches on a stream, synchronises and copies the result back. ``HostGemm`` keeps the device buffers and
pinned staging buffers alive between calls so that a call is: H2D of A and B, one launch through the C ABI, D2H of C.
"""
from __future__ import annotations

from typing import Optional

import torch

from .gemm import gemm as _gemm
from ._capi import B_DN

_NP_VIEW = {torch.bfloat16: torch.int16, torch.float16: torch.int16}


class HostGemm:
    """C = A @ B for host-resident operands. a: [m, k], b_dn: [n, k] (column-major B), out: [m, n]."""

    def __init__(self, m: int, n: int, k: int, in_dtype: torch.dtype = torch.bfloat16,
                 out_dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None):
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.m, self.n, self.k = m, n, k
        self.d_a = torch.empty((m, k), dtype=in_dtype, device=self.device)
        self.d_b = torch.empty((n, k), dtype=in_dtype, device=self.device)
        self.d_c = torch.empty((m, n), dtype=out_dtype, device=self.device)
        self.h_c = torch.empty((m, n), dtype=out_dtype, pin_memory=True)
        self.stream = torch.cuda.Stream(device=self.device)

    @property
    def h2d_bytes(self) -> int:
        return self.d_a.numel() * self.d_a.element_size() + self.d_b.numel() * self.d_b.element_size()

    @property
    def d2h_bytes(self) -> int:
        return self.d_c.numel() * self.d_c.element_size()

    def run(self, h_a: torch.Tensor, h_b_dn: torch.Tensor) -> torch.Tensor:
        """h_a / h_b_dn: host tensors (pinned for full copy speed). Returns the pinned host result after a
        stream synchronise."""
        with torch.cuda.stream(self.stream):
            self.d_a.copy_(h_a, non_blocking=True)
            self.d_b.copy_(h_b_dn, non_blocking=True)
            _gemm(self.d_a, self.d_b, b_layout=B_DN, out=self.d_c, stream=self.stream)
            self.h_c.copy_(self.d_c, non_blocking=True)
        self.stream.synchronize()
        return self.h_c


class HostGemmPipeline:
    """HostGemm for a stream of independent products: while product i runs on the GPU, the operands of product i+1
    travel host to device and the result of product i-1 travels back (PCIe carries both directions at once, and the
    GPU has separate copy engines for them). Every product still pays its own H2D of A and B and its own D2H of C.

    ``submit`` enqueues one product and returns a ticket; ``result(ticket)`` waits for that product's copy-back and
    returns its pinned host tensor, which stays valid until ``depth`` further products have been submitted.
    The reference's harness is strictly one product at a time (kernels/manual/a2a3/gemm_performance/main.cpp:23-80);
    this is the throughput form of the same three steps.
    """

    def __init__(self, m: int, n: int, k: int, in_dtype: torch.dtype = torch.bfloat16,
                 out_dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None, depth: int = 3):
        if depth < 2:
            raise ValueError("depth must be at least 2")
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.m, self.n, self.k, self.depth = m, n, k, depth
        self.sets = []
        for _ in range(depth):
            self.sets.append({
                "d_a": torch.empty((m, k), dtype=in_dtype, device=self.device),
                "d_b": torch.empty((n, k), dtype=in_dtype, device=self.device),
                "d_c": torch.empty((m, n), dtype=out_dtype, device=self.device),
                "h_c": torch.empty((m, n), dtype=out_dtype, pin_memory=True),
                "loaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "stored": torch.cuda.Event(),
            })
        self.s_in = torch.cuda.Stream(device=self.device)
        self.s_mm = torch.cuda.Stream(device=self.device)
        self.s_out = torch.cuda.Stream(device=self.device)
        self.submitted = 0

    @property
    def h2d_bytes(self) -> int:
        s = self.sets[0]
        return s["d_a"].numel() * s["d_a"].element_size() + s["d_b"].numel() * s["d_b"].element_size()

    @property
    def d2h_bytes(self) -> int:
        s = self.sets[0]
        return s["d_c"].numel() * s["d_c"].element_size()

    def submit(self, h_a: torch.Tensor, h_b_dn: torch.Tensor) -> int:
        ticket = self.submitted
        s = self.sets[ticket % self.depth]
        if ticket >= self.depth:
            # the set is reused: its previous product must have left the device (its GEMM read d_a / d_b before that)
            s["stored"].synchronize()
        with torch.cuda.stream(self.s_in):
            s["d_a"].copy_(h_a, non_blocking=True)
            s["d_b"].copy_(h_b_dn, non_blocking=True)
            s["loaded"].record(self.s_in)
        self.s_mm.wait_event(s["loaded"])
        with torch.cuda.stream(self.s_mm):
            _gemm(s["d_a"], s["d_b"], b_layout=B_DN, out=s["d_c"], stream=self.s_mm)
            s["computed"].record(self.s_mm)
        self.s_out.wait_event(s["computed"])
        with torch.cuda.stream(self.s_out):
            s["h_c"].copy_(s["d_c"], non_blocking=True)
            s["stored"].record(self.s_out)
        self.submitted += 1
        return ticket

    def result(self, ticket: int) -> torch.Tensor:
        if not (self.submitted - self.depth <= ticket < self.submitted):
            raise ValueError("ticket is not in flight (already overwritten or never submitted)")
        s = self.sets[ticket % self.depth]
        s["stored"].synchronize()
        return s["h_c"]
