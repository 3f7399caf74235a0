"""K-split GEMM + allreduce on real GPUs, NCCL and peer-memory reductions (needs at least two GPUs; skipped otherwise)."""
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


def _worker(rank, world, port, mode, m, n, k, result_dir):
    import torch.distributed as dist

    from pto_isa_mirror_b200 import gen_data as gd
    from pto_isa_mirror_b200.ksplit import KSplitGemmAllReduce, k_slice
    import pto_isa_mirror_b200 as pto

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        a_bits, b_bits = gd.dense_inputs(m, n, k, "bf16", 4)
        k0, k1 = k_slice(k, world, rank)
        a = torch.from_numpy(a_bits.view(np.int16)).to(dev).view(torch.bfloat16)
        b = torch.from_numpy(b_bits.view(np.int16)).to(dev).view(torch.bfloat16)
        if mode.startswith("p2p"):
            from pto_isa_mirror_b200.ksplit import KSplitGemmP2P

            op = KSplitGemmP2P(m, n, panels=2, device=dev, reduce_blocks=8, use_multicast=(mode == "p2p"))
            for _ in range(3):                  # three steps: both partial buffers and growing epochs
                out = op.step(a[:, k0:k1], b[:, k0:k1])
        else:
            op = KSplitGemmAllReduce(m, n, panels=2, mode=mode, device=dev)
            out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
            for _ in range(2):                  # twice: buffers and streams are reused across steps
                op.step(a[:, k0:k1], b[:, k0:k1], out)
        torch.cuda.synchronize(dev)
        assert pto.device_status() == 0
        if mode.startswith("p2p"):
            # the reduction is a rank-ordered fp32 sum of the ranks' GEMM partials followed by one bf16 cast:
            # recompute it from this rank's view of every partial (gathered with NCCL) and compare bit for bit
            mine = pto.gemm(a[:, k0:k1], b[:, k0:k1], torch.float32)
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            total = parts[0].clone()
            for r in range(1, world):
                total += parts[r]
            if op.multicast:
                # summed inside the NVSwitch in its own order: equal up to fp32 rounding of a few terms
                ref16 = pto.cast_f32_to_bf16(total).float()
                assert (out.float() - ref16).abs().max().item() <= 2.0 ** -7 * ref16.abs().max().item()
            else:
                assert torch.equal(pto.cast_f32_to_bf16(total), out)
        np.save(os.path.join(result_dir, f"out_{rank}.npy"), out.view(torch.int16).cpu().numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["allreduce", "rs_ag", "p2p", "p2p_pull"])
def test_ksplit_nccl(tmp_path, mode):
    import torch.multiprocessing as mp

    import oracle
    from pto_isa_mirror_b200 import gen_data as gd
    from pto_isa_mirror_b200.ksplit import k_slice

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    m, n, k = 1024, 512, 2048
    mp.spawn(_worker, args=(world, _free_port(), mode, m, n, k, str(tmp_path)), nprocs=world, join=True)
    outs = [np.load(tmp_path / f"out_{r}.npy").view(np.uint16) for r in range(world)]
    for r in range(1, world):
        assert np.array_equal(outs[0], outs[r]), "every rank must hold the same result"
    a_bits, b_bits = gd.dense_inputs(m, n, k, "bf16", 4)
    ref = oracle.gemm_f32acc(a_bits[:256], b_bits, oracle.BF16)     # unsplit sequential chain, first 256 rows
    got = gd.bf16_bits_to_f32(outs[0][:256])
    assert np.abs(got - ref).max() / np.abs(ref).max() <= 1e-3 + 2.0 ** -8   # dense tolerance + one bf16 rounding

