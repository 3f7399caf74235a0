"""AllGather + GEMM (one kernel per rank): every rank must end with C = A @ B for the whole A, bit-identical to the
plain GEMM of the gathered A on the same GPU, identical on all ranks, and within the dense tolerance of the oracle.
Multi-rank cases need at least two GPUs; the one-rank form of the kernel runs on one GPU. Rank processes never assert:
they save what they computed, leave together, and the parent compares."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, use_multicast, m, n, k, result_dir):
    import torch.distributed as dist

    import pto_isa_mirror_b200 as pto
    from pto_isa_mirror_b200 import gen_data as gd
    from pto_isa_mirror_b200.allgather import AllGatherGemm

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    report = {"error": ""}
    op = None
    try:
        a_bits, b_bits = gd.dense_inputs(m, n, k, "bf16", 14)
        a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
        b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
        op = AllGatherGemm(m, n, k, torch.bfloat16, torch.float32, device=dev, use_multicast=use_multicast)
        rows = m // world
        outs = []
        for step in range(3):                      # three steps; the slice changes sign each step
            sign = -1.0 if step % 2 else 1.0
            op.a_full.fill_(float("nan"))          # remote rows must really come from the peers
            torch.cuda.synchronize(dev)
            dist.barrier()
            op.a_local().copy_(a[rank * rows:(rank + 1) * rows] * sign)
            out = op.step(b)
            torch.cuda.synchronize(dev)
            outs.append(out.clone())
            dist.barrier()
        report["status"] = int(pto.device_status())
        report["multicast"] = bool(op.multicast)
        plain = pto.gemm(a, b, torch.float32)
        torch.cuda.synchronize(dev)
        np.save(os.path.join(result_dir, f"out_{rank}.npy"), outs[2].cpu().numpy())
        np.save(os.path.join(result_dir, f"neg_{rank}.npy"), outs[1].cpu().numpy())
        np.save(os.path.join(result_dir, f"plain_{rank}.npy"), plain.cpu().numpy())
    except Exception as e:  # noqa: BLE001
        report["error"] = repr(e)
    np.save(os.path.join(result_dir, f"report_{rank}.npy"), np.array([repr(report)]))
    try:
        out = outs = plain = None  # noqa: F841
        torch.cuda.synchronize(dev)
        dist.barrier()
        if op is not None:
            op.release()
        del op
        torch.cuda.synchronize(dev)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("use_multicast", [True, False])
def test_allgather_gemm_multi_gpu(tmp_path, use_multicast):
    import torch.multiprocessing as mp

    import oracle
    from pto_isa_mirror_b200 import gen_data as gd

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    m, n, k = 256 * world * 2, 768, 1024          # two 256-row blocks per rank
    mp.spawn(_worker, args=(world, _free_port(), use_multicast, m, n, k, str(tmp_path)), nprocs=world, join=True)
    reports = [eval(str(np.load(tmp_path / f"report_{r}.npy")[0])) for r in range(world)]  # noqa: S307 (own repr)
    for r, rep in enumerate(reports):
        assert rep["error"] == "", f"rank {r}: {rep['error']}"
        assert rep["status"] == 0, f"rank {r}: a bounded wait gave up (status {rep['status']})"
    outs = [np.load(tmp_path / f"out_{r}.npy") for r in range(world)]
    for r in range(world):
        assert np.array_equal(outs[0].view(np.uint32), outs[r].view(np.uint32)), "every rank must hold the same C"
        assert np.array_equal(outs[r].view(np.uint32), np.load(tmp_path / f"plain_{r}.npy").view(np.uint32))
        assert np.array_equal(np.load(tmp_path / f"neg_{r}.npy"), -outs[r]), "the second step used the negated slices"
    a_bits, b_bits = gd.dense_inputs(m, n, k, "bf16", 14)
    for r0 in (0, m - 128):
        ref = oracle.gemm_f32acc(a_bits[r0:r0 + 128], b_bits[:256], oracle.BF16)
        assert np.abs(outs[0][r0:r0 + 128, :256] - ref).max() / np.abs(ref).max() <= 1e-3


@pytest.mark.parametrize("shape", [(512, 512, 256), (4096, 2304, 512), (2048, 1000, 264)])
def test_allgather_gemm_one_rank(shape):
    """The all-gather form with a single rank on one GPU: the push role, the block flags and the rotated raster run;
    the result must be the plain GEMM's, bit for bit, on consecutive steps."""
    import oracle
    import pto_isa_mirror_b200 as pto
    from pto_isa_mirror_b200 import gen_data as gd
    from pto_isa_mirror_b200.allgather import AllGatherGemm

    m, n, k = shape
    dev = torch.device("cuda", 0)
    a_bits, b_bits = gd.dense_inputs(m, n, k, "bf16", 15)
    a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
    for odt in (torch.float32, torch.bfloat16):
        op = AllGatherGemm(m, n, k, torch.bfloat16, odt, device=dev)
        op.a_local().copy_(a)
        want = pto.gemm(a, b, odt)
        for step in range(2):
            out = op.step(b)
            torch.cuda.synchronize(dev)
            assert pto.device_status() == 0
            assert torch.equal(out.view(torch.uint8), want.view(torch.uint8)), f"step {step}"
    ref = oracle.gemm_f32acc(a_bits[:128], b_bits[:256], oracle.BF16)
    got = pto.gemm(a, b, torch.float32)[:128, :256].cpu().numpy()
    assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-3
