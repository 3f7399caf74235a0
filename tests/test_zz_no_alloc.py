"""The workspace-free MX entry point (pto_b200_gemm_mx_static) against the ordinary one, through the C ABI.

Some users of the library cannot hand over a scratch buffer and cannot allocate one when they call: a launcher
that keeps the reference's six-argument LaunchMxMatmul shape, or a process that gave its whole device memory
to its own pool at start-up. For them the re-tiled scale factors live in an array built into the library. This
test runs the new entry point three times in a row on different problems (the second large enough for the two-CTA
kernel), so that bytes left in the shared array by an earlier call would show up as wrong results if any were
read, and checks every result bit for bit against pto_b200_gemm_mx given a fresh workspace. It also checks that a problem larger than the
built-in array is refused before anything is launched.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from pto_isa_mirror_b200 import _capi
from pto_isa_mirror_b200 import gen_data as gd

pytestmark = pytest.mark.gpu


def _call_pair(lib, m, n, k, seed):
    dev = "cuda"
    a, b, sfa, sfb = gd.mx_inputs(m, n, k, seed)
    ta, tb, tsa, tsb = (torch.from_numpy(x).to(dev) for x in (a, b, sfa, sfb))
    stream = torch.cuda.current_stream().cuda_stream
    args_tail = (m, n, k, k, k, n, k // 32, k // 32, _capi.E4M3, _capi.E4M3, _capi.F32)

    need = lib.pto_b200_gemm_mx_workspace_bytes(m, n, k)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    ref = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
    rc = lib.pto_b200_gemm_mx(stream, ref.data_ptr(), ta.data_ptr(), tb.data_ptr(), tsa.data_ptr(), tsb.data_ptr(),
                              ws.data_ptr(), need, *args_tail)
    assert rc == _capi.OK, lib.pto_b200_error_string(rc)

    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=dev)
    before = lib.pto_b200_launch_count()
    rc = lib.pto_b200_gemm_mx_static(stream, out.data_ptr(), ta.data_ptr(), tb.data_ptr(), tsa.data_ptr(),
                                     tsb.data_ptr(), *args_tail)
    assert rc == _capi.OK, lib.pto_b200_error_string(rc)
    assert lib.pto_b200_launch_count() == before + 2          # the re-tile kernel and the GEMM
    torch.cuda.synchronize()
    return out.cpu().numpy(), ref.cpu().numpy()


def test_static_scratch_matches_workspace_variant_on_calls_in_a_row():
    lib = _capi.load()
    # first call: several tiles in M, N and K, ragged in every dimension
    out1, ref1 = _call_pair(lib, 640, 1000, 1056, seed=51)
    assert not np.isnan(ref1).any()
    assert np.array_equal(out1.view(np.uint32), ref1.view(np.uint32))
    # second call, straight after, over the first call's leftovers in the shared array: 100 tiles of 256 x 256, so
    # the two-CTA kernel runs, whose scale loads go through tensor maps encoded over the array's device address
    out2, ref2 = _call_pair(lib, 2560, 2560, 512, seed=53)
    assert not np.isnan(ref2).any()
    assert np.array_equal(out2.view(np.uint32), ref2.view(np.uint32))
    # third call: smaller and different again, back on the one-CTA kernel
    out3, ref3 = _call_pair(lib, 130, 260, 160, seed=52)
    assert not np.isnan(ref3).any()
    assert np.array_equal(out3.view(np.uint32), ref3.view(np.uint32))
    st = ctypes.c_int(0)
    assert lib.pto_b200_device_status(ctypes.byref(st)) == _capi.OK and st.value == 0


def test_static_scratch_refuses_oversized_problems():
    lib = _capi.load()
    m, n, k = 32768, 8192, 8192
    assert lib.pto_b200_gemm_mx_workspace_bytes(m, n, k) > _capi.MX_STATIC_SCRATCH_BYTES
    dummy = torch.zeros(64, dtype=torch.uint8, device="cuda")
    p = dummy.data_ptr()
    before = lib.pto_b200_launch_count()
    rc = lib.pto_b200_gemm_mx_static(torch.cuda.current_stream().cuda_stream, p, p, p, p, p, m, n, k, k, k, n,
                                     k // 32, k // 32, _capi.E4M3, _capi.E4M3, _capi.BF16)
    assert rc == _capi.ESCRATCH
    assert b"PTO_B200_MX_STATIC_SCRATCH_BYTES" in lib.pto_b200_error_string(rc)
    assert lib.pto_b200_launch_count() == before
