"""The allocation-free sparse GEMV entry point (scratch inside the library image) against the
regular entry point. Collected last on purpose: a failure here never hides another test's result."""

import pytest
import torch

from leankv_b200 import _native, workloads

pytestmark = pytest.mark.gpu


def _regular(lib, wt, x, n, z, t):
    y = torch.empty(n, dtype=torch.float16, device=wt.device)
    ws = torch.zeros(max(lib.leankv_sparse_gemv_workspace_bytes(n, z), 256), dtype=torch.uint8, device=wt.device)
    _native.check(lib.leankv_sparse_gemv_f16(wt.data_ptr(), x.data_ptr(), y.data_ptr(), n, z, t, None, None,
                                             ws.data_ptr(), ws.numel(), None,
                                             torch.cuda.current_stream().cuda_stream), "regular gemv")
    return y


def _static(lib, wt, x, n, z, t):
    # the output buffer comes from the caller (here: torch); the entry point itself allocates nothing
    y = torch.full((n,), float("nan"), dtype=torch.float16, device=wt.device)
    _native.check(lib.leankv_sparse_gemv_f16_static(wt.data_ptr(), x.data_ptr(), y.data_ptr(), n, z, t,
                                                    torch.cuda.current_stream().cuda_stream), "static gemv")
    return y


def test_static_scratch_gemv_matches_regular_entry_point_twice_in_a_row():
    lib = _native.lib()
    dev = torch.device("cuda:0")
    # two different shapes back to back: the second call finds the first call's partial sums in the
    # shared array and must not be disturbed by them
    for n, z, seed in ((4096, 14336, 0), (1024, 2500, 7), (4096, 14336, 0)):
        c = workloads.sparse_gemv_case(n, z, 0.4, seed, device=dev)
        wt = c.weight.t().contiguous()
        x = c.x.reshape(-1).contiguous()
        want = _regular(lib, wt, x, n, z, c.threshold)
        first = _static(lib, wt, x, n, z, c.threshold)
        second = _static(lib, wt, x, n, z, c.threshold)
        torch.cuda.synchronize()
        # same kernel, same fixed summation order: the tolerance is zero
        assert torch.equal(first, want)
        assert torch.equal(second, want)
    # beyond the compiled-in maximum: refused before anything is launched. The buffers are real and large
    # enough for the refused shapes, so that a check that stopped working would show as a wrong return
    # code here, not as a stray access on the device.
    for n, z in ((65536 + 8, 64), (64, 65536 + 1)):
        wt = torch.zeros(z, n, dtype=torch.float16, device=dev)
        x = torch.zeros(z, dtype=torch.float16, device=dev)
        y = torch.zeros(n, dtype=torch.float16, device=dev)
        assert lib.leankv_sparse_gemv_f16_static(wt.data_ptr(), x.data_ptr(), y.data_ptr(), n, z, 0.1, None) == -6
    assert b"maximum" in lib.leankv_strerror(-6)


def test_static_scratch_gemv_leaves_free_device_memory_unchanged():
    """The reason this entry point exists: nothing is allocated or freed on the device. After a first
    call (which may load the kernel image on this device) the free-memory figure the driver reports
    must not move over further calls of different shapes."""
    lib = _native.lib()
    dev = torch.device("cuda:0")
    cases = []
    for n, z, seed in ((4096, 14336, 0), (1024, 2500, 7), (8192, 4096, 3)):
        c = workloads.sparse_gemv_case(n, z, 0.4, seed, device=dev)
        cases.append((c.weight.t().contiguous(), c.x.reshape(-1).contiguous(),
                      torch.empty(n, dtype=torch.float16, device=dev), n, z, c.threshold))
    st = torch.cuda.current_stream().cuda_stream

    def call_all():
        for wt, x, y, n, z, t in cases:
            _native.check(lib.leankv_sparse_gemv_f16_static(wt.data_ptr(), x.data_ptr(), y.data_ptr(), n, z, t, st),
                          "static gemv")
        torch.cuda.synchronize()

    call_all()                                  # set-up call: symbol look-up, lazy module load
    free_before, _ = torch.cuda.mem_get_info(dev)
    for _ in range(3):
        call_all()
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before
