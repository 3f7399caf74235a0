"""Host logic of the K-split GEMM + allreduce under gloo (world size 2, CPU): partitioning, panel schedule,
both reduction modes and the bf16 cast, with the oracle standing in for the CUDA GEMM."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pto_isa_mirror_b200 import gen_data as gd
from pto_isa_mirror_b200.ksplit import KSplitGemmAllReduce, k_slice, panel_bounds, panels_from_rows


def test_panel_bounds():
    assert panel_bounds(8192, 4, 1024) == [(0, 2048), (2048, 4096), (4096, 6144), (6144, 8192)]
    assert panel_bounds(300, 4, 128) == [(0, 128), (128, 256), (256, 300)]
    assert panel_bounds(100, 1, 256) == [(0, 100)]
    assert panel_bounds(0, 4, 128) == []
    covered = panel_bounds(5000, 3, 256)
    assert covered[0][0] == 0 and covered[-1][1] == 5000
    assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))


def test_panels_from_rows():
    assert panels_from_rows(8192, [4096, 2048, 1024, 1024], 1024) == [(0, 4096), (4096, 6144), (6144, 7168), (7168, 8192)]
    assert panels_from_rows(8192, [6144], 1024) == [(0, 6144), (6144, 8192)]          # the remainder becomes a panel
    assert panels_from_rows(2048, [1024, 1024, 1024], 1024) == [(0, 1024), (1024, 2048)]
    with pytest.raises(ValueError):
        panels_from_rows(8192, [1000], 1024)


def test_k_slice():
    assert k_slice(65536, 8, 3) == (24576, 32768)
    assert [k_slice(64, 4, r) for r in range(4)] == [(0, 16), (16, 32), (32, 48), (48, 64)]
    with pytest.raises(ValueError):
        k_slice(100, 8, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_gemm(a, b_dn, out):
    import oracle

    a16 = gd.f32_to_bf16_bits(a.float().numpy())
    b16 = gd.f32_to_bf16_bits(b_dn.float().numpy())
    out.copy_(torch.from_numpy(oracle.gemm_f32acc(a16, b16, oracle.BF16, threads=2)))


def _cast(src, out):
    out.copy_(torch.from_numpy(gd.f32_to_bf16_bits(src.numpy()).view(np.int16)).view(torch.bfloat16))


def _worker(rank, world, port, mode, m, n, k, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a_bits, b_bits = gd.dense_inputs(m, n, k, "bf16", 4)
        a = torch.from_numpy(gd.bf16_bits_to_f32(a_bits)).bfloat16()
        b = torch.from_numpy(gd.bf16_bits_to_f32(b_bits)).bfloat16()
        k0, k1 = k_slice(k, world, rank)
        op = KSplitGemmAllReduce(m, n, panels=2, mode=mode, device=torch.device("cpu"), gemm_fn=_oracle_gemm,
                                 cast_fn=_cast)
        out = torch.empty((m, n), dtype=torch.bfloat16)
        op.step(a[:, k0:k1], b[:, k0:k1], out)
        np.save(os.path.join(result_dir, f"out_{rank}.npy"), out.view(torch.int16).numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["allreduce", "rs_ag"])
def test_ksplit_two_ranks_gloo(tmp_path, mode):
    import oracle

    m, n, k, world = 512, 64, 256, 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, mode, m, n, k, str(tmp_path)), nprocs=world, join=True)
    outs = [np.load(tmp_path / f"out_{r}.npy").view(np.uint16) for r in range(world)]
    assert np.array_equal(outs[0], outs[1]), "every rank must end with the same full result"
    a_bits, b_bits = gd.dense_inputs(m, n, k, "bf16", 4)
    # reference: fp32 partial of each K slice summed in rank order, then one bf16 cast
    total = np.zeros((m, n), dtype=np.float32)
    for r in range(world):
        k0, k1 = k_slice(k, world, r)
        total += oracle.gemm_f32acc(np.ascontiguousarray(a_bits[:, k0:k1]), np.ascontiguousarray(b_bits[:, k0:k1]),
                                    oracle.BF16)
    assert np.array_equal(outs[0], gd.f32_to_bf16_bits(total))
    # and it agrees with the unsplit chain within the dense tolerance
    unsplit = oracle.gemm_f32acc(a_bits, b_bits, oracle.BF16)
    got = gd.bf16_bits_to_f32(outs[0])
    assert np.abs(got - unsplit).max() / np.abs(unsplit).max() <= 8e-3  # bf16 output rounding dominates


# ------------------------------------------------------------------ AllGather + GEMM: the schedule, under gloo

def test_allgather_block_schedule():
    from pto_isa_mirror_b200.allgather import block_schedule, slice_rows

    assert slice_rows(8192, 2, 1) == (4096, 8192)
    assert [slice_rows(2048, 4, r) for r in range(4)] == [(0, 512), (512, 1024), (1024, 1536), (1536, 2048)]
    with pytest.raises(ValueError):
        slice_rows(1000, 2, 0)
    for world in (1, 2, 4, 8):
        m = 256 * world * 3
        for rank in range(world):
            order = block_schedule(m, world, rank)
            assert sorted(b for b, _ in order) == list(range(m // 256))          # every block exactly once
            assert all(owner == rank for _, owner in order[:3])                   # own rows first: no waiting
            assert all(owner == b // 3 for b, owner in order)
    assert block_schedule(1024, 2, 1) == [(2, 1), (3, 1), (0, 0), (1, 0)]


def _allgather_worker(rank, world, port, m, n, k, result_dir):
    import oracle
    from pto_isa_mirror_b200.allgather import block_schedule, slice_rows

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a_bits, b_bits = gd.dense_inputs(m, n, k, "bf16", 9)
        r0, r1 = slice_rows(m, world, rank)
        mine = torch.from_numpy(a_bits[r0:r1].view(np.uint8).copy())              # this rank holds only its M slice
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)                                              # the pushes of every owner
        gathered = torch.cat(parts).numpy().view(np.uint16)
        out = np.zeros((m, n), dtype=np.float32)
        for block, owner in block_schedule(m, world, rank):                       # the tile loop's order of row blocks
            rows = slice(block * 256, (block + 1) * 256)
            assert slice_rows(m, world, owner)[0] <= rows.start < slice_rows(m, world, owner)[1]
            out[rows] = oracle.gemm_f32acc(gathered[rows], b_bits, oracle.BF16, threads=2)
        np.save(os.path.join(result_dir, f"ag_out_{rank}.npy"), out)
        np.save(os.path.join(result_dir, f"ag_a_{rank}.npy"), gathered)
    finally:
        dist.destroy_process_group()


def test_allgather_gemm_two_ranks_gloo(tmp_path):
    """Two CPU ranks each hold half of A's rows; after the gather every rank multiplies all row blocks in its own
    schedule order and must hold the whole product, bit-identical on both ranks and to the unsplit product."""
    import oracle

    m, n, k = 1024, 64, 128
    mp.spawn(_allgather_worker, args=(2, _free_port(), m, n, k, str(tmp_path)), nprocs=2, join=True)
    a_bits, b_bits = gd.dense_inputs(m, n, k, "bf16", 9)
    ref = oracle.gemm_f32acc(a_bits, b_bits, oracle.BF16, threads=2)
    for r in range(2):
        assert np.array_equal(np.load(tmp_path / f"ag_a_{r}.npy"), a_bits)
        assert np.array_equal(np.load(tmp_path / f"ag_out_{r}.npy"), ref)
