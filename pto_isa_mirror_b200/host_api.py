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
