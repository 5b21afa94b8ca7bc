"""The allocation-free scan entry point (``fgl_exclusive_sum_noalloc``) against the workspace-backed one.

Hosts that cannot allocate device memory when they need block-CSR offsets (a fixed budget from a
framework allocator, HBM fully handed out to other pools, no tolerance for cudaMalloc's synchronisation)
call this variant; its scratch is a __device__ array inside the library, shared by all calls.  The test
goes through the C ABI directly, twice in a row with different sizes (the second call reuses the scratch
the first one left behind), and must hold both in a fresh process and after every other test has run.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_noalloc_scan_matches_workspace_scan_twice_in_a_row():
    import fastgl
    from fastgl import _capi

    lib = _capi.lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    rng = np.random.default_rng(2718)
    for n in (3_000_001, 70_000, 0, 1):  # large first, then smaller calls over the same scratch
        degs = torch.from_numpy(rng.integers(0, 16, size=n).astype(np.int32)).to(dev)
        expect = fastgl.exclusive_sum(degs)           # existing entry point (workspace scratch)
        out = torch.full((n + 1,), -7, dtype=torch.int32, device=dev)
        if n == 3_000_001:                            # first call on the device: the one-time symbol look-up
            rc = lib.fgl_exclusive_sum_noalloc(ctypes.c_void_p(degs.data_ptr()), ctypes.c_int64(n),
                                               ctypes.c_void_p(out.data_ptr()), stream)
            assert rc == 0, _capi.status_str(rc)
        torch.cuda.synchronize(dev)
        # the driver's own view of free device memory sees any cudaMalloc, whoever makes it (torch's counters
        # would only see torch's allocator)
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc = lib.fgl_exclusive_sum_noalloc(ctypes.c_void_p(degs.data_ptr() if n else 0), ctypes.c_int64(n),
                                           ctypes.c_void_p(out.data_ptr()), stream)
        assert rc == 0, _capi.status_str(rc)
        torch.cuda.synchronize(dev)
        assert torch.cuda.mem_get_info(dev)[0] == free_before
        assert fastgl.exclusive_sum_noalloc_status(dev) == 0      # no scan's barrier gave up
        assert torch.equal(out, expect)               # integer work: bit-exact
        assert np.array_equal(out.cpu().numpy()[1:], np.cumsum(degs.cpu().numpy(), dtype=np.int64).astype(np.int32))


def test_noalloc_scan_rejects_sizes_beyond_its_maximum():
    from fastgl import _capi

    lib = _capi.lib()
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda:0")
    rc = lib.fgl_exclusive_sum_noalloc(ctypes.c_void_p(dummy.data_ptr()), ctypes.c_int64((1 << 27) + 1),
                                       ctypes.c_void_p(dummy.data_ptr()), None)
    assert rc == 4 and "capacity" in _capi.status_str(rc)
