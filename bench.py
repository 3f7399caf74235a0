#!/usr/bin/env python
"""Benchmark of the B200 GEMM hot path:  python bench.py --gpus N --steps K --warmup W

Prints ONE JSON line. Metric: GEMM TFLOP/s = 2*M*N*K / time / 1e12 (the reference's definition,
docs/figures/performance/gemm_performance_a3.svg:9). Workloads (synthetic, seeded):

  N = 1 : dense bf16 GEMM M=N=K=4096, A row-major, B column-major, fp32 accumulate, bf16 output
          (other single-GPU configurations are timed briefly and reported under "all_configs").
  N > 1 : K-split GEMM + allreduce, bf16 A[8192 x 65536] x B[65536 x 8192], K partitioned over the ranks,
          fp32 partials reduced over NCCL, bf16 result on every rank (strong scaling: total work is fixed).

`--impl reference` times the reference's own CPU simulator (oracle/_ref, built from the reference's headers)
on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}

TRAFFIC_TABLE = os.path.join(ROOT, "profiles", "dram_traffic.txt")


def ncu_dram_traffic(workload: str):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the workload's dominant kernel, from the table of
    ncu captures kept beside the profile summaries (lines: workload, read bytes, written bytes, kernel). None when the
    workload was never captured."""
    try:
        with open(TRAFFIC_TABLE) as f:
            for raw in f:
                parts = raw.split()
                if len(parts) >= 3 and not raw.startswith("#") and parts[0] == workload:
                    return int(parts[1]) + int(parts[2])
    except OSError:
        pass
    return None


WORKLOADS = {
    "c1_f16_128x256x256": dict(kind="dense", m=128, n=256, k=256, dtype="f16", out="f32"),
    "bf16_4096": dict(kind="dense", m=4096, n=4096, k=4096, dtype="bf16", out="bf16"),
    "s8_8192_dequant": dict(kind="s8", m=8192, n=8192, k=8192),
    "mxfp8_16384x8192x8192": dict(kind="mx", m=16384, n=8192, k=8192),
    # the reference's MXFP8 kernel as it ships: e5m2 x e5m2, bf16 out, 6144^3
    # (kernels/manual/a5/matmul_mxfp8_performance/mxmatmul_performance_kernel.cpp:354-380)
    "mxfp8_e5m2_6144cubed": dict(kind="mx", m=6144, n=6144, k=6144, fmt="e5m2"),
    # the shape of the reference's MXFP4 kernel (kernels/manual/a5/matmul_mxfp4_performance/mxmatmul_performance_kernel.cpp:
    # 446-463): float4_e2m1x2_t operands, e8m0 scales, bf16 out, ragged M and N
    "mxfp4_2040x8100x8192": dict(kind="mx", m=2040, n=8100, k=8192, fmt="e2m1"),
    "ksplit_bf16_8192x65536x8192": dict(kind="ksplit", m=8192, n=8192, k=65536),
    # the largest shape of the reference's AllGather + GEMM table (kernels/manual/a2a3/allgather_gemm/README.md:112-125):
    # A split along M over the ranks, B replicated, every rank computes the whole C; run with --workload at any N
    "allgather_bf16_8192x4096x4096": dict(kind="allgather", m=8192, n=4096, k=4096),
    # one rank's share of the 8-GPU K-split step on one GPU: the fused kernel with its exchange warps reducing this GPU's
    # own partial (no peers), the form that can be profiled on a single GPU
    "ksplit_rank_share_bf16_8192x8192x8192": dict(kind="ksplit1", m=8192, n=8192, k=8192),
    "bf16_8192": dict(kind="dense", m=8192, n=8192, k=8192, dtype="bf16", out="bf16"),
    # HBM-bound neighbours of the tile loop (metric GB/s of algorithmic bytes)
    "gemv_bf16_8192x8192": dict(kind="gemv", m=1, n=8192, k=8192),
    "mx_quantize_8192x8192": dict(kind="quant", m=8192, n=1, k=8192),
    # the same two kernels on four times the bytes: start-up and the last blocks weigh less
    "gemv_bf16_8192x32768": dict(kind="gemv", m=1, n=32768, k=8192),
    "gemv_mx_e4m3_8192x32768": dict(kind="gemv_mx", m=1, n=32768, k=8192),
    "mx_quantize_32768x8192": dict(kind="quant", m=32768, n=1, k=8192),
    "mxfp4_quantize_32768x8192": dict(kind="quant", m=32768, n=1, k=8192, fmt="e2m1"),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


# --------------------------------------------------------------------------------------- clocks

class ClockSampler:
    """Polls NVML for the SM clock and the clock-event reasons of one GPU while a timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            uuid = None
            try:
                import torch

                uuid = str(torch.cuda.get_device_properties(index).uuid)
            except Exception:  # noqa: BLE001
                uuid = None
            self.h = None
            if uuid:
                for i in range(pynvml.nvmlDeviceGetCount()):
                    h = pynvml.nvmlDeviceGetHandleByIndex(i)
                    u = pynvml.nvmlDeviceGetUUID(h)
                    u = u.decode() if isinstance(u, bytes) else u
                    if uuid in u:
                        self.h = h
            if self.h is None:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    def _poll(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:  # noqa: BLE001
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# --------------------------------------------------------------------------------------- inputs (on the device)

def _randn_scaled(shape, k, dtype, gen, dev):
    import torch

    return (torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) / (k ** 0.5)).to(dtype)


def mx_quantize_torch(x, fp8=None):
    """OCP MX quantisation along K in blocks of 32 (include/pto/cpu/TQuant.hpp:178-190,226-237,461-494), as data
    preparation on the device: e8m0 = max(biased_exp(absmax) - 8, 0), element = e4m3fn(x * 2^(127 - e8m0)); with
    ``fp8 = torch.float8_e5m2`` the scaled values (at most 448 in magnitude) are stored as e5m2 instead."""
    import torch

    fp8 = fp8 or torch.float8_e4m3fn

    rows, k = x.shape
    g = x.view(rows, k // 32, 32)
    amax = g.abs().amax(dim=-1)
    exp = (amax.view(torch.int32) >> 23) & 0xFF
    e8m0 = torch.clamp(exp - 8, min=0)
    scaling = ((254 - e8m0) << 23).view(torch.float32)
    y = (g * scaling.unsqueeze(-1)).clamp(-448.0, 448.0)
    return y.to(fp8).view(torch.uint8).view(rows, k), e8m0.to(torch.uint8)


# --------------------------------------------------------------------------------------- parity (outside timed regions)

def _bits16(t):
    import numpy as np
    import torch

    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def _tile_origins(m, n, count, seed):
    """`count` seeded 128 x 256 output tiles (row, column origins)."""
    import random

    rng = random.Random(seed)
    return [(rng.randrange(max(m // 128, 1)) * 128, rng.randrange(max(n // 256, 1)) * 256) for _ in range(count)]


def _dense_tile_report(acc32_tiles, out16_tiles, refs, tol):
    """acc32_tiles: fp32 accumulators (numpy) per tile; out16_tiles: bf16/fp16 bit patterns per tile or None; refs: the
    oracle's fp32 tiles. max_rel_err is max |acc - ref| / max |ref| (the specification's measure); bf16_ulp_max
    compares the stored 16-bit values with the oracle's own cast wherever the value is not near zero."""
    import numpy as np

    import oracle

    worst, ulp = 0.0, 0
    for i, ref in enumerate(refs):
        d = np.abs(acc32_tiles[i].astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-300)
        worst = max(worst, float(d))
        if out16_tiles is not None:
            want = oracle.f32_to_bf16_bits(ref)
            big = np.abs(ref) >= np.sqrt(np.mean(ref.astype(np.float64) ** 2)) / 16

            def ordinal(u):
                u = u.astype(np.int32)
                return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)

            ulp = max(ulp, int(np.abs(ordinal(out16_tiles[i][big]) - ordinal(want[big])).max()))
    rep = {"tiles": len(refs), "max_rel_err": worst, "tol": tol, "ok": bool(worst <= tol)}
    if out16_tiles is not None:
        rep["bf16_ulp_max"] = ulp
        rep["ok"] = bool(rep["ok"] and ulp <= 1)
    return rep


def make_step(name: str, spec: dict, dev, seed: int, world=1, rank=0, panels=8, mode="fused", gemm_blocks=0,
              reduce_blocks=48, panel_rows=None, use_multicast=True, gemm_streams=2):
    """Returns (step_fn, flops_per_step, working_set_bytes, launches_hint). step_fn(i) enqueues one pass;
    step_fn.parity() (run outside any timed region) checks sampled output tiles against the oracle and returns the
    report that goes into the JSON line."""
    import numpy as np
    import torch

    import pto_isa_mirror_b200 as pto

    gen = torch.Generator(device=dev).manual_seed(seed)
    m, n, k = spec["m"], spec["n"], spec["k"]
    kind = spec["kind"]
    flops = 2.0 * m * n * k
    if kind == "dense":
        dt = torch.bfloat16 if spec["dtype"] == "bf16" else torch.float16
        odt = {"bf16": torch.bfloat16, "f32": torch.float32, "f16": torch.float16}[spec["out"]]
        per_set = (m * k + n * k) * 2 + m * n * (4 if odt == torch.float32 else 2)
        sets = max(2, -(-3 * L2_BYTES // per_set)) if per_set < 3 * L2_BYTES else 1
        sets = min(sets, 64)
        bufs = [(_randn_scaled((m, k), k, dt, gen, dev), _randn_scaled((n, k), k, dt, gen, dev),
                 torch.empty((m, n), dtype=odt, device=dev)) for _ in range(sets)]

        # the host layer's per-stream workspace lets a partly filled last wave be split along K (4096^3: 34 of 256
        # tiles); shapes whose last wave is more than half full run unsplit
        def step(i):
            a, b, c = bufs[i % sets]
            pto.gemm(a, b, out=c, workspace="auto")

        def parity():
            import oracle

            a, b, c = bufs[0]
            pto.gemm(a, b, out=c, workspace="auto")
            c32 = pto.gemm(a, b, torch.float32)      # the same product with the fp32 accumulators stored
            torch.cuda.synchronize(dev)
            code = oracle.BF16 if dt == torch.bfloat16 else oracle.F16
            acc, out16, refs = [], [], []
            for r0, c0 in _tile_origins(m, n, 2, 101):
                r1, c1 = min(r0 + 128, m), min(c0 + 256, n)
                refs.append(oracle.gemm_f32acc(_bits16(a[r0:r1]), _bits16(b[c0:c1]), code))
                acc.append(c32[r0:r1, c0:c1].cpu().numpy())
                out16.append(_bits16(c[r0:r1, c0:c1]) if odt == torch.bfloat16 else None)
            return _dense_tile_report(acc, out16 if odt == torch.bfloat16 else None, refs, 1e-3)

        step.parity = parity
        return step, flops, per_set * sets, sets
    if kind == "s8":
        per_set = 2 * m * k + m * n * 2
        sets = 2
        bufs = []
        for _ in range(sets):
            a = torch.randint(-127, 128, (m, k), generator=gen, device=dev, dtype=torch.int8)
            b = torch.randint(-127, 128, (n, k), generator=gen, device=dev, dtype=torch.int8)
            s_row = torch.rand(m, generator=gen, device=dev) * 9e-3 + 1e-3
            s_col = ((torch.rand(n, generator=gen, device=dev) * 9e-3 + 1e-3).view(torch.int32) & ~0x1FFF).view(
                torch.float32)
            bufs.append((a, b, s_row, s_col, torch.empty((m, n), dtype=torch.bfloat16, device=dev)))

        def step(i):
            a, b, sr, sc, c = bufs[i % sets]
            pto.gemm_s8_dequant(a, b, sr, sc, out=c)

        def parity():
            import oracle

            a, b, sr, sc, c = bufs[0]
            pto.gemm_s8_dequant(a, b, sr, sc, out=c)
            torch.cuda.synchronize(dev)
            exact = True
            origins = _tile_origins(m, n, 2, 102)
            for r0, c0 in origins:
                ref = oracle.gemm_s8(a[r0:r0 + 128].cpu().numpy(), b[c0:c0 + 256].cpu().numpy())
                want = oracle.dequant_bf16(ref, sr[r0:r0 + 128].cpu().numpy(), sc[c0:c0 + 256].cpu().numpy(), True)
                exact = exact and bool(np.array_equal(_bits16(c[r0:r0 + 128, c0:c0 + 256]), want))
            return {"tiles": len(origins), "bit_exact": exact, "ok": exact,
                    "what": "bf16((float(int32 acc) * s_col) * s_row) against the oracle's int32 chain and store"}

        step.parity = parity
        return step, flops, per_set * sets, sets
    if kind == "mx" and spec.get("fmt") == "e2m1":
        # inputs as the reference's generator draws them (matmul_mxfp4_performance/scripts/gen_data.py:46-52): values
        # -1, 0, 1 (codes 0xA, 0x0, 0x2), two per byte with the even element in the low nibble, scales 2^0..2^2
        codes = torch.tensor([0xA, 0x0, 0x2], dtype=torch.uint8, device=dev)

        def draw(rows):
            v = codes[torch.randint(0, 3, (rows, k), generator=gen, device=dev)]
            return (v[:, 0::2] | (v[:, 1::2] << 4)).contiguous()

        per_set = (m * k + n * k) // 2 + (m + n) * (k // 32) + m * n * 2
        sets = min(16, max(2, -(-3 * L2_BYTES // per_set))) if per_set < 3 * L2_BYTES else 1
        bufs = []
        for _ in range(sets):
            bufs.append((draw(m), draw(n),
                         torch.randint(127, 130, (m, k // 32), generator=gen, device=dev, dtype=torch.uint8),
                         torch.randint(127, 130, (n, k // 32), generator=gen, device=dev, dtype=torch.uint8),
                         torch.empty((m, n), dtype=torch.bfloat16, device=dev)))
        ws = torch.zeros(pto.gemm_mx_workspace_bytes(m, n, k, split_last_wave=True), dtype=torch.uint8, device=dev)

        def step(i):
            a, b, sfa, sfb, c = bufs[i % sets]
            pto.gemm_mx(a, b, sfa, sfb, torch.bfloat16, pto.E2M1, pto.E2M1, workspace=ws, out=c)

        def parity():
            import oracle

            a, b, sfa, sfb, c = bufs[0]
            step(0)
            torch.cuda.synchronize(dev)
            ok, tiles = True, []
            for r0, c0 in _tile_origins(m, n, 2, 103):
                ref = oracle.gemm_mx(a[r0:r0 + 128].cpu().numpy(), b[c0:c0 + 256].cpu().numpy(),
                                     sfa[r0:r0 + 128].cpu().numpy(), sfb[c0:c0 + 256].cpu().numpy(), oracle.E2M1,
                                     oracle.E2M1)
                same = np.array_equal(_bits16(c[r0:r0 + 128, c0:c0 + 256]), oracle.f32_to_bf16_bits(ref))
                ok = ok and same
                tiles.append([r0, c0])
            return {"ok": bool(ok), "tiles": tiles,
                    "what": "bf16 store against the RNE cast of the oracle's chain: every sum is an integer below 2^18, "
                            "so the comparison is exact"}

        step.parity = parity
        return step, flops, per_set * sets, sets
    if kind == "mx":
        e5m2 = spec.get("fmt") == "e5m2"
        fp8 = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
        fmt = pto.E5M2 if e5m2 else pto.E4M3
        a, sfa = mx_quantize_torch(torch.randn((m, k), generator=gen, device=dev), fp8)
        b, sfb = mx_quantize_torch(torch.randn((n, k), generator=gen, device=dev), fp8)
        c = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        ws = torch.zeros(pto.gemm_mx_workspace_bytes(m, n, k, split_last_wave=True), dtype=torch.uint8, device=dev)

        def step(i):
            pto.gemm_mx(a, b, sfa, sfb, torch.bfloat16, fmt, fmt, workspace=ws, out=c)

        # the same product with the scales re-tiled once beforehand (weights' scales, or a producer that writes the
        # tiled form): one kernel launch per step
        ws_tiled = pto.mx_retile_scales(sfa, sfb, k)
        c2 = torch.empty((m, n), dtype=torch.bfloat16, device=dev)

        def pretiled(i):
            pto.gemm_mx_pretiled(a, b, ws_tiled, torch.bfloat16, fmt, fmt, out=c2)

        step.pretiled = pretiled
        step.pretiled_matches = lambda: bool(torch.equal(c.view(torch.int16), c2.view(torch.int16)))

        def parity():
            import oracle

            step(0)
            c32 = pto.gemm_mx(a, b, sfa, sfb, torch.float32, fmt, fmt, workspace=ws)
            torch.cuda.synchronize(dev)
            ofmt = oracle.E5M2 if e5m2 else oracle.E4M3
            acc, out16, refs = [], [], []
            for r0, c0 in _tile_origins(m, n, 2, 103):
                refs.append(oracle.gemm_mx(a[r0:r0 + 128].cpu().numpy(), b[c0:c0 + 256].cpu().numpy(),
                                           sfa[r0:r0 + 128].cpu().numpy(), sfb[c0:c0 + 256].cpu().numpy(), ofmt, ofmt))
                acc.append(c32[r0:r0 + 128, c0:c0 + 256].cpu().numpy())
                out16.append(_bits16(c[r0:r0 + 128, c0:c0 + 256]))
            rep = _dense_tile_report(acc, None, refs, 1e-2)
            same = all(np.array_equal(out16[i], oracle.f32_to_bf16_bits(acc[i])) for i in range(len(acc)))
            rep["bf16_store_is_rne_of_fp32"] = bool(same)
            rep["ok"] = bool(rep["ok"] and same)
            return rep

        step.parity = parity
        return step, flops, m * k + n * k + m * n * 2, 1
    if kind == "ksplit":
        import torch.distributed as dist

        from pto_isa_mirror_b200.ksplit import KSplitGemmAllReduce, k_slice

        k0, k1 = k_slice(k, world, rank)
        kr = k1 - k0
        # every rank draws its own K slice of the operands (values N(0,1)/sqrt(K) as for the unsplit matrix)
        gen.manual_seed(seed * 1000 + rank)
        a = _randn_scaled((m, kr), k, torch.bfloat16, gen, dev)
        b = _randn_scaled((n, kr), k, torch.bfloat16, gen, dev)
        op = None
        reduce_used = mode
        if world > 1 and mode in ("fused", "p2p"):
            from pto_isa_mirror_b200.ksplit import KSplitGemmFused, KSplitGemmP2P

            align = 128 * world
            rows = [h for h in (panel_rows or []) if h % align == 0]
            try:
                if mode == "fused":
                    op = KSplitGemmFused(m, n, panels=panels, device=dev, launch_block_count=gemm_blocks,
                                         use_multicast=use_multicast)
                else:
                    op = KSplitGemmP2P(m, n, panels=panels, device=dev, reduce_blocks=reduce_blocks,
                                       launch_block_count=gemm_blocks, use_multicast=use_multicast,
                                       gemm_streams=gemm_streams,
                                       panel_rows=rows if rows and len(rows) == len(panel_rows) else None)
                ok = torch.ones(1, device=dev)
            except Exception as e:  # noqa: BLE001  (peer mapping unavailable on this box: use the NCCL reduction)
                if rank == 0:
                    print(f"[bench] peer-memory reduction unavailable ({e!r}); using NCCL rs_ag", file=sys.stderr)
                ok = torch.zeros(1, device=dev)
                op = None
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)      # every rank takes the same path
            if ok.item() == 0:
                op = None
        nccl = None
        if op is not None:
            out = op.out
            p2p = op

            def step(i):
                p2p.step(a, b)

            step.panel_rows = [r1 - r0 for r0, r1 in op.panels]
            step.op = op
            how = "fused_one_kernel" if mode == "fused" else "p2p_panel_kernels"
            reduce_used = how + ("_nvls_multimem" if op.multicast else "_peer_loads")
        else:
            if mode in ("fused", "p2p"):
                reduce_used = "rs_ag" if world > 1 else "none"
            out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
            nccl = KSplitGemmAllReduce(m, n, panels=panels if world > 1 else 1,
                                       mode=mode if mode not in ("fused", "p2p") else "rs_ag", device=dev,
                                       single_rank=(world == 1), launch_block_count=gemm_blocks)

            def step(i):
                nccl.step(a, b, out)

        def parity():
            """Sampled 128 x 256 output tiles over the full K, against the oracle's sequential chain: the rows of every
            rank's A slice and the columns of every rank's B slice of a tile are gathered on rank 0 (a few MB)."""
            import oracle

            step(0)
            torch.cuda.synchronize(dev)
            origins = _tile_origins(m, n, 2, 104)
            acc, out16, refs, identical = [], [], [], True
            for r0, c0 in origins:
                pieces = [a[r0:r0 + 128].contiguous(), b[c0:c0 + 256].contiguous(),
                          out[r0:r0 + 128, c0:c0 + 256].contiguous()]
                # this rank's fp32 partial of the tile (peer-memory variants keep it; the unsplit run holds the product)
                if op is not None:
                    pieces.append(op.partial[op.epoch & 1][r0:r0 + 128, c0:c0 + 256].contiguous())
                elif world == 1:
                    pieces.append(nccl.partial[r0:r0 + 128, c0:c0 + 256].contiguous())
                gathered = []
                for t in pieces:
                    if world > 1:
                        parts = [torch.empty_like(t) for _ in range(world)]
                        dist.all_gather(parts, t)
                    else:
                        parts = [t]
                    gathered.append(parts)
                if rank != 0:
                    continue
                a_full = np.concatenate([_bits16(x) for x in gathered[0]], axis=1)
                b_full = np.concatenate([_bits16(x) for x in gathered[1]], axis=1)
                outs = [_bits16(x) for x in gathered[2]]
                identical = identical and all(np.array_equal(outs[0], o) for o in outs[1:])
                ref = oracle.gemm_f32acc(a_full, b_full, oracle.BF16)
                refs.append(ref)
                out16.append(outs[0])
                if len(gathered) > 3:
                    total = gathered[3][0].cpu().numpy().copy()
                    for x in gathered[3][1:]:
                        total += x.cpu().numpy()            # fp32, rank order
                    acc.append(total)
                else:
                    acc.append(oracle.bf16_bits_to_f32(outs[0]))
            if rank != 0:
                return None
            have_acc = op is not None or world == 1
            # with the fp32 partials at hand the accumulators meet the specification's 1e-3; a bf16-only comparison
            # carries one more bf16 rounding (2^-8 of the largest value)
            rep = _dense_tile_report(acc, out16, refs, 1e-3 if have_acc else 1e-3 + 2.0 ** -8)
            rep["compared"] = ("rank-ordered fp32 sum of the ranks' partial tiles, and the delivered bf16 tile"
                               if have_acc else "the delivered bf16 tile")
            rep["all_ranks_identical"] = bool(identical)
            rep["ok"] = bool(rep["ok"] and identical)
            return rep

        step.parity = parity
        step.reduce_used = reduce_used
        step.tensors = (a, b, out)
        return step, flops, (m + n) * kr * 2 + m * n * 6, 1
    if kind == "ksplit1":
        from pto_isa_mirror_b200.ksplit import KSplitGemmFused

        a = _randn_scaled((m, k), k, torch.bfloat16, gen, dev)
        b = _randn_scaled((n, k), k, torch.bfloat16, gen, dev)
        op = KSplitGemmFused(m, n, panels=panels, device=dev)

        def step(i):
            op.step(a, b)

        def parity():
            import oracle

            step(0)
            want = pto.cast_f32_to_bf16(pto.gemm(a, b, torch.float32))
            torch.cuda.synchronize(dev)
            same = bool(torch.equal(op.out.view(torch.int16), want.view(torch.int16)))
            acc, out16, refs = [], [], []
            for r0, c0 in _tile_origins(m, n, 1, 106):
                refs.append(oracle.gemm_f32acc(_bits16(a[r0:r0 + 128]), _bits16(b[c0:c0 + 256]), oracle.BF16))
                acc.append(op.partial[op.epoch & 1][r0:r0 + 128, c0:c0 + 256].cpu().numpy())
                out16.append(_bits16(op.out[r0:r0 + 128, c0:c0 + 256]))
            rep = _dense_tile_report(acc, out16, refs, 1e-3)
            rep["equals_plain_gemm_then_cast"] = same
            rep["ok"] = bool(rep["ok"] and same)
            return rep

        step.parity = parity
        step.reduce_used = "fused_one_kernel_single_rank"
        return step, flops, (m + n) * k * 2 + m * n * 6, 1
    if kind == "gemv":
        mats = [_randn_scaled((n, k), k, torch.bfloat16, gen, dev) for _ in range(4)]      # 512 MiB > L2
        x = _randn_scaled((k,), k, torch.bfloat16, gen, dev)
        y = torch.empty((n,), dtype=torch.float32, device=dev)

        def step(i):
            pto.gemv(x, mats[i % 4], out=y)

        def parity():
            import oracle

            pto.gemv(x, mats[0], out=y)
            torch.cuda.synchronize(dev)
            ref = oracle.gemm_f32acc(_bits16(x.view(1, k)), _bits16(mats[0][:2048]), oracle.BF16)[0]
            err = float(np.abs(y[:2048].cpu().numpy() - ref).max() / np.abs(ref).max())
            return {"rows": 2048, "max_rel_err": err, "tol": 1e-3, "ok": bool(err <= 1e-3)}

        step.parity = parity
        step.bytes = n * k * 2 + k * 2 + n * 4
        return step, 2.0 * n * k, 4 * n * k * 2, 4
    if kind == "gemv_mx":
        xq, sfx = mx_quantize_torch(torch.randn((1, k), generator=gen, device=dev))
        mats = [mx_quantize_torch(torch.randn((n, k), generator=gen, device=dev)) for _ in range(2)]   # 2 x 264 MiB > L2
        y = torch.empty((n,), dtype=torch.float32, device=dev)

        def step(i):
            pto.gemv_mx(xq[0], mats[i % 2][0], sfx[0], mats[i % 2][1], out=y)

        def parity():
            import oracle

            pto.gemv_mx(xq[0], mats[0][0], sfx[0], mats[0][1], out=y)
            torch.cuda.synchronize(dev)
            ref = oracle.gemm_mx(xq.cpu().numpy(), mats[0][0][:256].cpu().numpy(), sfx.cpu().numpy(),
                                 mats[0][1][:256].cpu().numpy())[0]
            err = float(np.abs(y[:256].cpu().numpy() - ref).max() / np.abs(ref).max())
            return {"columns": 256, "max_rel_err": err, "tol": 1e-2, "ok": bool(err <= 1e-2)}

        step.parity = parity
        step.bytes = n * k + n * k // 32 + k + k // 32 + n * 4
        return step, 2.0 * n * k, 2 * (n * k + n * k // 32), 2
    if kind == "quant":
        fp4 = spec.get("fmt") == "e2m1"                                                       # MXFP4: two codes per byte
        srcs = [torch.randn((m, k), generator=gen, device=dev) for _ in range(2)]             # at least 512 MiB > L2
        q_data = torch.empty((m, k // 2 if fp4 else k), dtype=torch.uint8, device=dev)
        q_scales = torch.empty((m, k // 32), dtype=torch.uint8, device=dev)
        quantise = pto.mx_quantize_e2m1 if fp4 else pto.mx_quantize_e4m3

        def step(i):
            quantise(srcs[i % 2], data=q_data, scales=q_scales)

        def parity():
            import oracle

            quantise(srcs[0], data=q_data, scales=q_scales)
            torch.cuda.synchronize(dev)
            rd, rs = (oracle.mx_quantize_e2m1 if fp4 else oracle.mx_quantize_e4m3)(srcs[0][:256].cpu().numpy())
            exact = bool(np.array_equal(q_data[:256].cpu().numpy(), rd) and np.array_equal(q_scales[:256].cpu().numpy(), rs))
            return {"rows": 256, "bit_exact": exact, "ok": exact}

        step.parity = parity
        step.bytes = int(m * k * (4 + (0.5 if fp4 else 1) + 1 / 32))
        return step, 0.0, 2 * m * k * 4, 2
    if kind == "allgather":
        import torch.distributed as dist

        from pto_isa_mirror_b200.allgather import AllGatherGemm

        op = AllGatherGemm(m, n, k, torch.bfloat16, torch.float32, device=dev, use_multicast=use_multicast,
                           launch_block_count=gemm_blocks)
        gen.manual_seed(seed * 1000 + rank)
        op.a_local().copy_(_randn_scaled((m // world, k), k, torch.bfloat16, gen, dev))
        gen.manual_seed(seed * 1000 + 999)                 # B is the same on every rank
        b = _randn_scaled((n, k), k, torch.bfloat16, gen, dev)

        def step(i):
            op.step(b)

        def parity():
            import oracle

            step(0)
            torch.cuda.synchronize(dev)
            rows_per_rank = m // world
            acc, refs, identical, received = [], [], True, True
            for r0, c0 in _tile_origins(m, n, 2, 105):
                owner = r0 // rows_per_rank
                rows = op.a_full[r0:r0 + 128].clone()          # this rank's copy: pushed here by the owner
                sent = rows.clone()
                if world > 1:
                    dist.broadcast(sent, src=owner)            # the owner's original rows
                ok = torch.tensor([int(torch.equal(rows.view(torch.int16), sent.view(torch.int16)))], device=dev)
                tile = op.out[r0:r0 + 128, c0:c0 + 256].contiguous()
                tiles = [tile]
                if world > 1:
                    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                    tiles = [torch.empty_like(tile) for _ in range(world)]
                    dist.all_gather(tiles, tile)
                received = received and bool(ok.item())
                if rank != 0:
                    continue
                identical = identical and all(torch.equal(tiles[0].view(torch.int32), t.view(torch.int32)) for t in tiles[1:])
                refs.append(oracle.gemm_f32acc(_bits16(sent), _bits16(b[c0:c0 + 256]), oracle.BF16))
                acc.append(tiles[0].cpu().numpy())
            if rank != 0:
                return None
            rep = _dense_tile_report(acc, None, refs, 1e-3)
            rep["gathered_rows_equal_owners_rows"] = bool(received)
            rep["all_ranks_identical"] = bool(identical)
            rep["ok"] = bool(rep["ok"] and received and identical)
            return rep

        step.parity = parity
        step.reduce_used = "allgather_one_kernel" + ("_nvls_multimem" if op.multicast else "_peer_stores")
        step.op = op
        return step, flops, (m + n) * k * 2 + m * n * 4, 1
    raise ValueError(kind)


# The shapes of the reference's own published table (fp16 in, fp32 out, m = n = k), timed briefly under "all_configs".
REF_TABLE_SHAPES = (1536, 3072, 6144, 7680)


def aux_configs(dev, peaks):
    """Brief timings of the neighbours of the GEMM path: the reference table's fp16 -> fp32 cubes (tensor-bound), the
    one-row TGEMV and the MX quantiser (both HBM-bound: GB/s of algorithmic bytes against the measured copy peak)."""
    import torch

    import pto_isa_mirror_b200 as pto

    out = {}
    gen = torch.Generator(device=dev).manual_seed(11)
    peak_tf = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    peak_gbs = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    for size in REF_TABLE_SHAPES:
        step, flops, _, _ = make_step(f"f16_f32_{size}", dict(kind="dense", m=size, n=size, k=size, dtype="f16", out="f32"),
                                      dev, seed=3)
        ms = time_steps(step, 20, 3, dev, 1) / 20
        entry = {"tflops": flops / (ms * 1e-3) / 1e12, "ms": ms,
                 "frac_of_peak": flops / (ms * 1e-3) / 1e12 / peak_tf, "peak": peak_tf, "launch": "one call per step"}
        if ms < 0.1:
            # a kernel of a few microseconds is hidden behind the host's launch path (Python, ctypes, descriptor
            # encoding): replay 20 launches from a CUDA graph so that the device time is what is measured
            try:
                side = torch.cuda.Stream(device=dev)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.stream(side):
                    step(0)
                    torch.cuda.synchronize(dev)
                    with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                        for j in range(20):
                            step(j)
                gms = time_steps(lambda i: graph.replay(), 5, 3, dev, 1) / (5 * 20)
                entry.update({"tflops": flops / (gms * 1e-3) / 1e12, "ms": gms,
                              "frac_of_peak": flops / (gms * 1e-3) / 1e12 / peak_tf, "ms_one_call_per_step": ms,
                              "launch": "20 launches per CUDA graph replay"})
                del graph
            except Exception as e:  # noqa: BLE001
                entry["graph_error"] = repr(e)
        out[f"f16_f32_{size}cubed"] = entry
        del step
        torch.cuda.empty_cache()
    # TGEMV: bf16 n x 8192 matrix per launch, rotating matrices (at least 512 MiB > L2); the larger one shows how
    # much of the small one's gap is start-up and the last blocks
    k = 8192
    for n in (8192, 32768):
        count = 4 if n == 8192 else 2
        mats = [_randn_scaled((n, k), k, torch.bfloat16, gen, dev) for _ in range(count)]
        x = _randn_scaled((k,), k, torch.bfloat16, gen, dev)
        y = torch.empty((n,), dtype=torch.float32, device=dev)
        ms = time_steps(lambda i: pto.gemv(x, mats[i % count], out=y), 40, 5, dev, 1) / 40
        gbytes = (n * k * 2 + k * 2 + n * 4) / 1e9
        out[f"gemv_bf16_8192x{n}"] = {"gbs": gbytes / (ms * 1e-3), "ms": ms, "bytes": int(gbytes * 1e9),
                                      "frac_of_hbm_peak": gbytes / (ms * 1e-3) / peak_gbs, "peak_gbs": peak_gbs}
        del mats
        torch.cuda.empty_cache()
    # TGEMV_MX: one e4m3 row against a block-scaled e4m3 matrix of 32768 x 8192 (256 MiB + 8 MiB of scales per
    # launch, 2 rotating matrices), checked against the oracle's chain on the first 256 columns
    n = 32768
    xq, sfx = mx_quantize_torch(torch.randn((1, k), generator=gen, device=dev))
    mats = [mx_quantize_torch(torch.randn((n, k), generator=gen, device=dev)) for _ in range(2)]
    y = torch.empty((n,), dtype=torch.float32, device=dev)
    ms = time_steps(lambda i: pto.gemv_mx(xq[0], mats[i % 2][0], sfx[0], mats[i % 2][1], out=y), 40, 5, dev, 1) / 40
    gbytes = (n * k + n * k // 32 + k + k // 32 + n * 4) / 1e9
    entry = {"gbs": gbytes / (ms * 1e-3), "ms": ms, "bytes": int(gbytes * 1e9),
             "frac_of_hbm_peak": gbytes / (ms * 1e-3) / peak_gbs, "peak_gbs": peak_gbs}
    try:
        import numpy as np

        import oracle

        pto.gemv_mx(xq[0], mats[0][0], sfx[0], mats[0][1], out=y)
        torch.cuda.synchronize(dev)
        ref = oracle.gemm_mx(xq.cpu().numpy(), mats[0][0][:256].cpu().numpy(), sfx.cpu().numpy(),
                             mats[0][1][:256].cpu().numpy())[0]
        err = float(np.abs(y[:256].cpu().numpy() - ref).max() / np.abs(ref).max())
        entry["parity"] = {"columns": 256, "max_rel_err": err, "tol": 1e-2, "ok": bool(err <= 1e-2)}
    except Exception as e:  # noqa: BLE001
        entry["parity"] = {"ok": False, "error": repr(e)[:300]}
    out["gemv_mx_e4m3_8192x32768"] = entry
    del mats
    torch.cuda.empty_cache()
    # MX quantiser: fp32 rows x 8192 per launch (4 bytes read + 1 1/32 written per element), 2 rotating sources
    kq = 8192
    for rows in (8192, 32768):
        srcs = [torch.randn((rows, kq), generator=gen, device=dev) for _ in range(2)]
        q_data = torch.empty((rows, kq), dtype=torch.uint8, device=dev)
        q_scales = torch.empty((rows, kq // 32), dtype=torch.uint8, device=dev)
        ms = time_steps(lambda i: pto.mx_quantize_e4m3(srcs[i % 2], data=q_data, scales=q_scales), 20, 3, dev, 1) / 20
        gbytes = rows * kq * (4 + 1 + 1 / 32) / 1e9
        out[f"mx_quantize_{rows}x8192"] = {"gbs": gbytes / (ms * 1e-3), "ms": ms, "bytes": int(gbytes * 1e9),
                                           "frac_of_hbm_peak": gbytes / (ms * 1e-3) / peak_gbs, "peak_gbs": peak_gbs}
        del srcs, q_data, q_scales
        torch.cuda.empty_cache()
    # the same source quantised to MXFP4: 4 bytes read + 1/2 + 1/32 written per element
    rows = 32768
    srcs = [torch.randn((rows, kq), generator=gen, device=dev) for _ in range(2)]
    q_data = torch.empty((rows, kq // 2), dtype=torch.uint8, device=dev)
    q_scales = torch.empty((rows, kq // 32), dtype=torch.uint8, device=dev)
    ms = time_steps(lambda i: pto.mx_quantize_e2m1(srcs[i % 2], data=q_data, scales=q_scales), 20, 3, dev, 1) / 20
    gbytes = rows * kq * (4 + 0.5 + 1 / 32) / 1e9
    out[f"mxfp4_quantize_{rows}x8192"] = {"gbs": gbytes / (ms * 1e-3), "ms": ms, "bytes": int(gbytes * 1e9),
                                          "frac_of_hbm_peak": gbytes / (ms * 1e-3) / peak_gbs, "peak_gbs": peak_gbs}
    del srcs, q_data, q_scales
    torch.cuda.empty_cache()
    return out


def library_yardsticks(dev):
    """Vendor-library 8-bit GEMMs timed once on this GPU as measuring sticks for the int8 and fp8 kernels (no measured
    8-bit peak exists beside the bf16 one). Library calls, never on the product path; absent ops are reported as such."""
    import torch

    out = {}
    try:
        m = n = k = 8192
        a = torch.randint(-127, 128, (m, k), device=dev, dtype=torch.int8)
        b = torch.randint(-127, 128, (n, k), device=dev, dtype=torch.int8)
        ms = time_steps(lambda i: torch._int_mm(a, b.t()), 10, 3, dev, 1) / 10
        out["int8_torch_int_mm_8192cubed_tops"] = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        del a, b
    except Exception as e:  # noqa: BLE001
        out["int8_torch_int_mm_8192cubed_tops"] = None
        out["int8_error"] = repr(e)[:200]
    try:
        m, n, k = 16384, 8192, 8192
        a = torch.randn((m, k), device=dev).to(torch.float8_e4m3fn)
        b = torch.randn((n, k), device=dev).to(torch.float8_e4m3fn)
        one = torch.ones((), device=dev)
        ms = time_steps(lambda i: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16),
                        10, 3, dev, 1) / 10
        out["fp8_torch_scaled_mm_16384x8192x8192_tflops"] = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        out["fp8_note"] = "per-tensor scales (cuBLASLt fp8), not block-scaled: an upper measuring stick for MXFP8"
        del a, b
    except Exception as e:  # noqa: BLE001
        out["fp8_torch_scaled_mm_16384x8192x8192_tflops"] = None
        out["fp8_error"] = repr(e)[:200]
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------------------- timing

def time_steps(step, steps, warmup, dev, world):
    import torch
    import torch.distributed as dist

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize(dev)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        step(warmup + i)
    end.record()
    torch.cuda.synchronize(dev)
    ms = start.elapsed_time(end)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize(dev)
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


# --------------------------------------------------------------------------------------- CPU baselines

def cpu_tile_runner(kind: str, k: int, single_thread=False):
    """A closure that runs ONE 128 x 256 x k output tile of the workload through the reference CPU simulator
    (or, where it was never built, the C restatement), plus a description of what runs."""
    import numpy as np

    import oracle
    from pto_isa_mirror_b200 import gen_data as gd

    use_ref = oracle.Ref.available(single_thread)
    cores = 1 if single_thread else (os.cpu_count() or 1)
    sim = oracle.Ref(single_thread) if use_ref else None
    if kind == "s8":
        a, b, _, _ = gd.s8_inputs(128, 256, k, 2)
        run = (lambda: sim.tile_s8(a, b)) if use_ref else (lambda: oracle.gemm_s8(a, b, cores))
    elif kind == "mx4":
        a = gd.randint((128, k // 2), 0, 255, 5, 0).astype(np.uint8)
        b = gd.randint((256, k // 2), 0, 255, 5, 1).astype(np.uint8)
        sfa = gd.randint((128, k // 32), 127, 129, 5, 2).astype(np.uint8)
        sfb = gd.randint((256, k // 32), 127, 129, 5, 3).astype(np.uint8)
        run = (lambda: sim.tile_mx(a, b, sfa, sfb, oracle.E2M1, oracle.E2M1)) if use_ref else (
            lambda: oracle.gemm_mx(a, b, sfa, sfb, oracle.E2M1, oracle.E2M1, threads=cores))
    elif kind == "mx":
        a, b, sfa, sfb = gd.mx_inputs(128, 256, k, 3)
        run = (lambda: sim.tile_mx(a, b, sfa, sfb)) if use_ref else (
            lambda: oracle.gemm_mx(a, b, sfa, sfb, threads=cores))
    else:
        a16, b16 = gd.dense_inputs(128, 256, k, "bf16", 1)
        if use_ref:
            af, bf = gd.bf16_bits_to_f32(a16), gd.bf16_bits_to_f32(b16)
            run = lambda: sim.tile_f32(af, bf)  # noqa: E731
        else:
            run = lambda: oracle.gemm_f32acc(a16, b16, oracle.BF16, threads=cores)  # noqa: E731
    what = ("RunGemmE2E / TMATMUL of the reference CPU simulator (oracle/_ref)" if use_ref
            else "the C restatement (oracle/pto_gemm_oracle.c)")
    return run, {"kind": "reference" if use_ref else "port", "cores": cores, "what": what}


def cpu_reference_sample(kind: str, k: int, budget_s: float, single_thread: bool = False):
    """Times output tiles of the workload on the host cores until `budget_s` has elapsed."""
    run, info = cpu_tile_runner(kind, k, single_thread)
    flops = 2.0 * 128 * 256 * k
    run()
    n, t0 = 0, time.perf_counter()
    while True:
        run()
        n += 1
        el = time.perf_counter() - t0
        if el >= budget_s:
            break
    return flops * n / el / 1e12, {
        "kind": info["kind"], "cores": info["cores"],
        "sample": f"{n} output tile(s) 128x256 with K={k} ({flops * n / 1e9:.2f} GFLOP) in {el:.1f} s through "
                  + info["what"],
    }


def reference_arm(args, world, rank):
    """`--impl reference`: the reference's CPU implementation on the host cores, bounded sample per step."""
    if rank != 0:
        return
    name = args.workload or ("bf16_4096" if args.gpus == 1 else "ksplit_bf16_8192x65536x8192")
    spec = WORKLOADS[name]
    kind = spec["kind"]
    import oracle

    if not (oracle.Ref.available() or os.path.exists(oracle.ORACLE_LIB)):
        oracle.build()
    # one step = one 128 x 256 output tile over a K that keeps the whole run within a few minutes
    full_k = spec["k"] if kind != "ksplit" else spec["k"] // max(args.gpus, 1)
    sk = "dense" if kind in ("ksplit", "allgather") else ("mx4" if spec.get("fmt") == "e2m1" else kind)
    depths = (8192, 4096, 1024, 256) if sk == "dense" else (8192, 1024, 256)
    candidates = [kk for kk in depths if kk <= full_k] or [256]
    total_steps = args.steps + args.warmup
    run, info, chosen = None, None, candidates[-1]
    for kk in candidates:
        run, info = cpu_tile_runner(sk, kk)
        t0 = time.perf_counter()
        run()
        if (time.perf_counter() - t0) * total_steps <= 150.0 or kk == candidates[-1]:
            chosen = kk
            break
    for _ in range(args.warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    el = time.perf_counter() - t0
    flops = 2.0 * 128 * 256 * chosen * args.steps
    value = flops / el / 1e12
    line = {
        "impl": "reference", "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": el / max(args.steps, 1) * 1e3,
        "higher_is_better": True, "scaling": "strong" if kind == "ksplit" else "weak", "vs_baseline": None,
        "dtype": "mxfp4_e2m1" if spec.get("fmt") == "e2m1" else "mxfp8_e5m2" if spec.get("fmt") == "e5m2" else
                 {"dense": "bf16", "ksplit": "bf16", "allgather": "bf16", "s8": "s8", "mx": "mxfp8_e4m3"}[kind],
        "data": "synthetic",
        "config": {"workload": name, "m": spec["m"], "n": spec["n"], "k": spec["k"],
                   "note": "reference CPU simulator on host cores; each step is one 128x256 output tile over "
                           f"K={chosen} of this workload"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": info["cores"], "kind": info["kind"],
                         "sample": f"{args.steps} steps, each one 128x256xK={chosen} output tile "
                                   f"({2.0 * 128 * 256 * chosen / 1e9:.3f} GFLOP) through {info['what']}, "
                                   "simulator default threading"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------- main arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--panels", type=int, default=8)
    ap.add_argument("--mode", default="auto", choices=["auto", "fused", "p2p", "rs_ag", "allreduce"],
                    help="K-split step: fused = one kernel per rank (GEMM + exchange over peer memory); p2p = one GEMM "
                         "per panel + this library's reduction kernels; rs_ag / allreduce = NCCL collectives; auto = "
                         "p2p on two GPUs (a rank multiplies for 3 ms per step there and the per-panel form is the "
                         "faster one under the power cap, measured 3.4-3.5 against 3.7-3.9 ms), fused on more")
    ap.add_argument("--regions", type=int, default=5, help="timed regions of exactly --steps steps each")
    ap.add_argument("--reduce-blocks", type=int, default=32)
    ap.add_argument("--gemm-streams", type=int, default=2, help="p2p mode: streams the panel GEMMs alternate between")
    ap.add_argument("--no-multicast", action="store_true", help="p2p mode: plain peer loads instead of NVLS multimem")
    ap.add_argument("--panel-rows", default="",
                    help="p2p mode: row-panel heights (comma separated); empty = --panels equal panels")
    ap.add_argument("--gemm-blocks", type=int, default=0,
                    help="K-split only: thread blocks (SMs) the GEMM may occupy beside the reduction, 0 = all")
    ap.add_argument("--no-extras", action="store_true", help="skip all_configs / cpu_baseline / e2e (profiling runs)")
    ap.add_argument("--cpu-budget", type=float, default=10.0)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, world, rank)
        return

    import torch
    import torch.distributed as dist

    import pto_isa_mirror_b200 as pto

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU arm)")
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run --nproc-per-node N")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime

        # a short collective timeout: a rank that never joins ends the run with an error instead of hanging it
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))

    name = args.workload or ("bf16_4096" if world == 1 else "ksplit_bf16_8192x65536x8192")
    spec = WORKLOADS[name]
    peaks = load_peaks()
    mode = args.mode if args.mode != "auto" else ("p2p" if world == 2 else "fused")
    step, flops, ws_bytes, sets = make_step(name, spec, dev, seed=1, world=world, rank=rank, panels=args.panels,
                                            mode=mode, gemm_blocks=args.gemm_blocks,
                                            reduce_blocks=args.reduce_blocks,
                                            panel_rows=[int(x) for x in args.panel_rows.split(",") if x],
                                            use_multicast=not args.no_multicast, gemm_streams=args.gemm_streams)

    # `regions` timed regions of exactly `steps` steps each (barrier + synchronize on both sides, CUDA events, max over
    # ranks); the line's value is the median region, the spread is printed beside it
    launches0 = pto.launch_count()
    region_ms = []
    with ClockSampler(local_rank) as clk:
        for r in range(max(1, args.regions)):
            region_ms.append(time_steps(step, args.steps, args.warmup if r == 0 else 1, dev, world))
    launches_total = pto.launch_count() - launches0
    steps_run = max(1, args.regions) * args.steps + args.warmup + (max(1, args.regions) - 1)
    launches = launches_total * args.steps // steps_run
    status = pto.device_status()
    ms = sorted(region_ms)[len(region_ms) // 2]
    ms_per_step = ms / args.steps
    tflops = flops / (ms_per_step * 1e-3) / 1e12

    kind = spec["kind"]
    dtype = {"dense": spec.get("dtype", "bf16"), "ksplit": "bf16", "ksplit1": "bf16", "allgather": "bf16", "s8": "s8",
             "mx": "mxfp8_e4m3", "gemv": "bf16", "gemv_mx": "mxfp8_e4m3", "quant": "f32"}[kind]
    if spec.get("fmt") == "e2m1":
        dtype = "mxfp4_e2m1"   # through kind::mxf8f6f4: 4-bit operands in memory, the 8-bit kinds' tensor rate
    elif spec.get("fmt") == "e5m2":
        dtype = "mxfp8_e5m2"
    peak_scale = {"s8": 2.0, "mx": 2.0}.get(kind, 1.0)
    # a single kernel timed back to back for a short region: burst peak; the long K-split step: sustained
    peak_key = "bf16_tflops" if ms < 500.0 else "bf16_tflops_sustained"
    peak = float(peaks.get(peak_key, FALLBACK_PEAKS["bf16_tflops"])) * peak_scale
    # K-split: the ranks share one product; all-gather: every rank computes the whole product (the reference's
    # 2 M N K / time counts it once), so a GPU achieves the line's value
    achieved = tflops / world if kind == "ksplit" else tflops
    line = {
        "metric": "gemm_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if kind == "ksplit" else "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": name, "m": spec["m"], "n": spec["n"], "k": spec["k"],
                   "layout": "A row-major, B column-major, fp32 accumulate",
                   "l2": (f"rotating {sets} input/output sets, {ws_bytes / 2**20:.0f} MiB > 126 MiB L2"
                          if sets > 1 else f"working set {ws_bytes / 2**20:.0f} MiB > 126 MiB L2"),
                   "inputs": ("seeded torch.randn on device, N(0,1)/sqrt(K)" if kind in ("dense", "ksplit", "allgather")
                              else "seeded"),
                   **({"parallelism": f"ksplit{world}", "panels": args.panels,
                       "reduce": getattr(step, "reduce_used", mode),
                       "gemm_blocks": args.gemm_blocks, "reduce_blocks": args.reduce_blocks,
                       "gemm_streams": args.gemm_streams,
                       "panel_rows": getattr(step, "panel_rows", None)}
                      if kind == "ksplit" else
                      ({"parallelism": f"allgather{world}", "reduce": getattr(step, "reduce_used", None)}
                       if kind == "allgather" else {}))},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak, "traffic": ncu_dram_traffic(name),
                     "peak_source": f"{peaks['_source']}: {peak_key}" + (" x2 (8-bit kinds, nominal ratio)" if peak_scale > 1 else ""),
                     "frac_of_sustained": achieved / (float(peaks.get("bf16_tflops_sustained", 1400.0)) * peak_scale),
                     "per": "GPU"},
        "clocks": clk.summary(),
        "gpu_launches": int(launches),
        "device_status": status,
        "timed_regions": {"n": len(region_ms), "steps_each": args.steps,
                          "ms_per_step_median": ms_per_step,
                          "ms_per_step_min": min(region_ms) / args.steps,
                          "ms_per_step_max": max(region_ms) / args.steps,
                          "ms_per_step_each": [round(x / args.steps, 6) for x in region_ms]},
    }
    # sampled output tiles against the oracle, outside every timed region (all ranks take part in the gathers)
    try:
        par = step.parity()
    except Exception as e:  # noqa: BLE001
        par = {"ok": False, "error": repr(e)[:300]}
    if par is not None:
        line["parity"] = par

    if kind in ("gemv", "gemv_mx", "quant"):
        # HBM-bound neighbours: GB/s of algorithmic bytes against the measured copy bandwidth
        gbs = step.bytes / (ms_per_step * 1e-3) / 1e9
        hbm = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
        line.update({"metric": "hbm_gbs", "value": gbs, "unit": "GB/s"})
        line["roofline"] = {"bound": "hbm", "achieved": gbs, "peak": hbm, "unit": "GB/s", "frac": gbs / hbm,
                            "traffic": ncu_dram_traffic(name), "peak_source": f"{peaks['_source']}: hbm_gbs",
                            "algorithmic_bytes": step.bytes, "per": "GPU"}
    if rank == 0 and world == 1 and not args.no_extras:
        # end to end through the host-buffer API: H2D of A and B, one launch, D2H of C, every step
        if kind == "dense":
            from pto_isa_mirror_b200.host_api import HostGemm

            idt = torch.bfloat16 if spec["dtype"] == "bf16" else torch.float16
            odt = {"bf16": torch.bfloat16, "f32": torch.float32, "f16": torch.float16}[spec["out"]]
            hg = HostGemm(spec["m"], spec["n"], spec["k"], idt, odt, dev)
            h_a = torch.randn((spec["m"], spec["k"])).mul_(spec["k"] ** -0.5).to(idt).pin_memory()
            h_b = torch.randn((spec["n"], spec["k"])).mul_(spec["k"] ** -0.5).to(idt).pin_memory()
            for _ in range(3):
                hg.run(h_a, h_b)
            e2e_steps = max(3, min(args.steps, 20))
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                hg.run(h_a, h_b)
            el = time.perf_counter() - t0
            sync_value = flops * e2e_steps / el / 1e12
            line["e2e"] = {"value": sync_value, "unit": "TFLOP/s",
                           "h2d_bytes_per_step": hg.h2d_bytes, "d2h_bytes_per_step": hg.d2h_bytes,
                           "steps": e2e_steps, "timer": "host wall clock around HostGemm.run (stream-synchronised)"}
            del hg
            # the same three steps per product, pipelined over three buffer sets: H2D of product i+1 and D2H of
            # product i-1 overlap the GEMM of product i; every product still pays its own copies
            try:
                from pto_isa_mirror_b200.host_api import HostGemmPipeline

                pipe = HostGemmPipeline(spec["m"], spec["n"], spec["k"], idt, odt, dev, depth=3)
                checksum = 0.0
                for i in range(3):
                    pipe.result(pipe.submit(h_a, h_b))
                torch.cuda.synchronize(dev)
                t0 = time.perf_counter()
                for i in range(e2e_steps):
                    t = pipe.submit(h_a, h_b)
                    if t >= 2:
                        checksum += float(pipe.result(t - 2)[0, 0])      # a host read of an earlier product's result
                for t in range(max(pipe.submitted - 2, 0), pipe.submitted):
                    checksum += float(pipe.result(t)[0, 0])
                el = time.perf_counter() - t0
                line["e2e"] = {"value": flops * e2e_steps / el / 1e12, "unit": "TFLOP/s",
                               "h2d_bytes_per_step": pipe.h2d_bytes, "d2h_bytes_per_step": pipe.d2h_bytes,
                               "steps": e2e_steps, "one_product_at_a_time": sync_value,
                               "timer": "host wall clock around HostGemmPipeline.submit / result, three products in "
                                        "flight, drained inside the timed region"}
                del pipe
            except Exception as e:  # noqa: BLE001
                line["e2e"]["pipeline_error"] = repr(e)
        # the other single-GPU configurations, briefly
        others = {}
        for oname in ("c1_f16_128x256x256", "s8_8192_dequant", "mxfp8_16384x8192x8192", "mxfp8_e5m2_6144cubed",
                      "mxfp4_2040x8100x8192", "ksplit_bf16_8192x65536x8192"):
            if oname == name:
                continue
            try:
                ostep, oflops, _, _ = make_step(oname, WORKLOADS[oname], dev, seed=2)
                osteps = 20 if oname != "ksplit_bf16_8192x65536x8192" else 5
                oms = time_steps(ostep, osteps, 3, dev, 1) / osteps
                okind = WORKLOADS[oname]["kind"]
                opeak = float(peaks.get("bf16_tflops", 1590.0)) * (2.0 if okind in ("s8", "mx") else 1.0)
                others[oname] = {"tflops": oflops / (oms * 1e-3) / 1e12, "ms": oms,
                                 "frac_of_peak": oflops / (oms * 1e-3) / 1e12 / opeak, "peak": opeak,
                                 "traffic": ncu_dram_traffic(oname)}
                try:
                    others[oname]["parity"] = ostep.parity()
                except Exception as e:  # noqa: BLE001
                    others[oname]["parity"] = {"ok": False, "error": repr(e)[:300]}
                if hasattr(ostep, "pretiled"):
                    pms = time_steps(ostep.pretiled, osteps, 3, dev, 1) / osteps
                    ostep(0)
                    torch.cuda.synchronize(dev)
                    others[oname]["pretiled_scales"] = {"tflops": oflops / (pms * 1e-3) / 1e12, "ms": pms,
                                                        "frac_of_peak": oflops / (pms * 1e-3) / 1e12 / opeak,
                                                        "same_bits_as_default_call": ostep.pretiled_matches()}
                del ostep
                torch.cuda.empty_cache()
            except Exception as e:  # noqa: BLE001
                others[oname] = {"error": repr(e)}
        try:
            others.update(aux_configs(dev, peaks))
        except Exception as e:  # noqa: BLE001
            others["aux"] = {"error": repr(e)}
        line["all_configs"] = others
        try:
            line["peak_yardstick"] = library_yardsticks(dev)
        except Exception as e:  # noqa: BLE001
            line["peak_yardstick"] = {"error": repr(e)[:200]}
        try:
            v, info = cpu_reference_sample("dense", spec["k"] if spec["k"] <= 8192 else 8192, args.cpu_budget)
            line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", **info}
            # the simulator built with PTO_CPU_MAX_THREADS=1 (the reference's own single-thread knob), briefly
            v1, info1 = cpu_reference_sample("dense", spec["k"] if spec["k"] <= 8192 else 8192,
                                             max(1.0, args.cpu_budget / 5), single_thread=True)
            line["cpu_baseline"]["single_thread"] = {"value": v1, "cores": info1["cores"], "sample": info1["sample"]}
        except Exception as e:  # noqa: BLE001
            line["cpu_baseline"] = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "port", "sample": repr(e)}
    elif world > 1 and kind == "ksplit":
        # end to end for the K-split step: H2D of this rank's operand slices, the step, D2H of the bf16 result
        a, b, out = step.tensors
        h_a = torch.empty(a.shape, dtype=a.dtype).pin_memory()
        h_b = torch.empty(b.shape, dtype=b.dtype).pin_memory()
        h_o = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        h_a.copy_(a)
        h_b.copy_(b)

        def e2e_step(i):
            a.copy_(h_a, non_blocking=True)
            b.copy_(h_b, non_blocking=True)
            step(i)
            h_o.copy_(out, non_blocking=True)

        e2e_steps = max(3, min(args.steps, 5))
        e_ms = time_steps(e2e_step, e2e_steps, 1, dev, world)
        line["e2e"] = {"value": flops * e2e_steps / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                       "h2d_bytes_per_step": (a.numel() + b.numel()) * 2 * world,
                       "d2h_bytes_per_step": out.numel() * 2 * world, "steps": e2e_steps}
        if rank == 0:
            # the unsplit product on one GPU, for the scaling base of this same workload
            try:
                if hasattr(step, "op"):
                    step.op = None
                del a, b, out, step
                torch.cuda.empty_cache()
                ustep, uflops, _, _ = make_step(name, spec, dev, seed=1, world=1, rank=0)
                u_regions = [time_steps(ustep, args.steps, args.warmup if r == 0 else 1, dev, 1) / args.steps
                             for r in range(max(1, args.regions))]
                ums = sorted(u_regions)[len(u_regions) // 2]
                line["unsplit_1gpu"] = {"tflops": uflops / (ums * 1e-3) / 1e12, "ms": ums, "steps": args.steps,
                                        "warmup": args.warmup, "ms_each": [round(x, 6) for x in u_regions]}
                # like for like: the same product unsplit on one GPU of this box over n times the n-GPU step
                line["scaling_efficiency"] = ums / (world * ms_per_step)
            except Exception as e:  # noqa: BLE001
                line["unsplit_1gpu"] = {"error": repr(e)}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
