"""K-split GEMM + allreduce on real GPUs: the fused one-kernel step, the per-panel peer-memory reduction and the NCCL
baselines (the multi-rank cases need at least two GPUs and are skipped otherwise; the one-rank form of the fused kernel
runs on one GPU).

The rank processes never assert: each saves what it computed, all ranks pass the same barrier, drop their symmetric
buffers together and leave together; the parent process does every comparison from the saved files. A rank that left
early on a failed check would end its peers in the middle of a step while their memory is still bound to the NVSwitch
multicast object.
"""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MODES = ["allreduce", "rs_ag", "p2p", "p2p_pull", "fused", "fused_pull"]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, m, n, k, result_dir):
    import torch.distributed as dist

    from pto_isa_mirror_b200 import gen_data as gd
    from pto_isa_mirror_b200.ksplit import KSplitGemmAllReduce, KSplitGemmFused, KSplitGemmP2P, k_slice
    import pto_isa_mirror_b200 as pto

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    report = {"error": ""}
    op = None
    try:
        a_bits, b_bits = gd.dense_inputs(m, n, k, "bf16", 4)
        k0, k1 = k_slice(k, world, rank)
        a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
        b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
        if mode.startswith("fused"):
            op = KSplitGemmFused(m, n, panels=2, device=dev, use_multicast=(mode == "fused"))
            for _ in range(3):                  # three steps: both partial buffers and growing epochs
                out = op.step(a[:, k0:k1], b[:, k0:k1])
        elif mode.startswith("p2p"):
            op = KSplitGemmP2P(m, n, panels=2, device=dev, reduce_blocks=8, use_multicast=(mode == "p2p"))
            for _ in range(3):
                out = op.step(a[:, k0:k1], b[:, k0:k1])
        else:
            op = KSplitGemmAllReduce(m, n, panels=2, mode=mode, device=dev)
            out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
            for _ in range(2):                  # twice: buffers and streams are reused across steps
                op.step(a[:, k0:k1], b[:, k0:k1], out)
        torch.cuda.synchronize(dev)
        report["status"] = int(pto.device_status())
        report["multicast"] = bool(getattr(op, "multicast", False))
        # the rank-ordered fp32 sum of the ranks' GEMM partials followed by one bf16 cast, from this rank's view of
        # every partial (gathered with NCCL): what the peer-load reduction must reproduce bit for bit
        mine = pto.gemm(a[:, k0:k1], b[:, k0:k1], torch.float32)
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        total = parts[0].clone()
        for r in range(1, world):
            total += parts[r]
        ordered = pto.cast_f32_to_bf16(total)
        torch.cuda.synchronize(dev)
        np.save(os.path.join(result_dir, f"out_{rank}.npy"), out.view(torch.int16).cpu().numpy())
        np.save(os.path.join(result_dir, f"ordered_{rank}.npy"), ordered.view(torch.int16).cpu().numpy())
    except Exception as e:  # noqa: BLE001  (reported to the parent; the rank still leaves with the others)
        report["error"] = repr(e)
    np.save(os.path.join(result_dir, f"report_{rank}.npy"), np.array([repr(report)]))
    try:
        out = mine = parts = total = ordered = None  # noqa: F841  (drop every view of the symmetric buffers)
        torch.cuda.synchronize(dev)
        dist.barrier()
        if op is not None and hasattr(op, "release"):
            op.release()
        del op
        torch.cuda.synchronize(dev)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", MODES)
def test_ksplit_multi_gpu(tmp_path, mode):
    import torch.multiprocessing as mp

    import oracle
    from pto_isa_mirror_b200 import gen_data as gd

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    m, n, k = 1024, 512, 2048
    mp.spawn(_worker, args=(world, _free_port(), mode, m, n, k, str(tmp_path)), nprocs=world, join=True)
    reports = [eval(str(np.load(tmp_path / f"report_{r}.npy")[0])) for r in range(world)]  # noqa: S307 (own repr)
    for r, rep in enumerate(reports):
        assert rep["error"] == "", f"rank {r}: {rep['error']}"
        assert rep["status"] == 0, f"rank {r}: a bounded wait gave up (status {rep['status']})"
    outs = [np.load(tmp_path / f"out_{r}.npy").view(np.uint16) for r in range(world)]
    for r in range(1, world):
        assert np.array_equal(outs[0], outs[r]), "every rank must hold the same result"
    ordered = np.load(tmp_path / "ordered_0.npy").view(np.uint16)
    if mode in ("p2p_pull", "fused_pull"):
        assert np.array_equal(outs[0], ordered), "peer loads are summed in rank order: bit-exact"
    elif mode in ("p2p", "fused") and reports[0]["multicast"]:
        # summed inside the NVSwitch in its own order: equal up to fp32 rounding of a few terms before the bf16 cast
        got, ref16 = gd.bf16_bits_to_f32(outs[0]), gd.bf16_bits_to_f32(ordered)
        assert np.abs(got - ref16).max() <= 2.0 ** -7 * np.abs(ref16).max()
    a_bits, b_bits = gd.dense_inputs(m, n, k, "bf16", 4)
    ref = oracle.gemm_f32acc(a_bits[:256], b_bits, oracle.BF16)     # unsplit sequential chain, first 256 rows
    got = gd.bf16_bits_to_f32(outs[0][:256])
    assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-3 + 2.0 ** -8   # dense tolerance + one bf16 rounding


@pytest.mark.parametrize("shape", [(1024, 512, 2048, 2), (4096, 4096, 1024, 4), (2304, 2304, 512, 3), (640, 1000, 192, 2)])
def test_fused_step_one_rank(shape):
    """The one-kernel step with a single rank on one GPU (plain device memory, no process group): every in-kernel
    hand-off runs - panel counters, ready flags, the exchange warps' shard reduction, done flags - and the result must
    be the bf16 cast of this GPU's own fp32 product, bit for bit, on three consecutive steps."""
    import oracle
    import pto_isa_mirror_b200 as pto
    from pto_isa_mirror_b200 import gen_data as gd
    from pto_isa_mirror_b200.ksplit import KSplitGemmFused

    m, n, k, panels = shape
    dev = torch.device("cuda", 0)
    a_bits, b_bits = gd.dense_inputs(m, n, k, "bf16", 9)
    a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    op = KSplitGemmFused(m, n, panels=panels, device=dev)
    want = pto.cast_f32_to_bf16(pto.gemm(a, b, torch.float32)).view(torch.int16).cpu().numpy()
    for step in range(3):
        op.out.zero_()
        out = op.step(a, b)
        torch.cuda.synchronize(dev)
        assert pto.device_status() == 0
        assert np.array_equal(out.view(torch.int16).cpu().numpy(), want), f"step {step}"
    rows = min(m, 128)
    ref = oracle.gemm_f32acc(a_bits[:rows], b_bits, oracle.BF16)
    got = gd.bf16_bits_to_f32(want[:rows].view(np.uint16))
    assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-3 + 2.0 ** -8
