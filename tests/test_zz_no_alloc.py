"""The allocation-free routing entry point against the regular one.

``dpk_route_compact_static`` serves callers that cannot allocate device memory (a
fixed memory pool, a host that only lends input and output buffers): its scratch is
an array inside the library.  This file is named so that pytest collects it last;
the test also has to pass when it runs alone in a fresh process, which is why it
builds and loads the library itself and does not rely on state left by other tests.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(lib, N, mask):
    """Run the regular and the allocation-free entry point on one mask."""
    st = torch.cuda.current_stream().cuda_stream
    m8 = mask.contiguous().view(torch.uint8)
    if m8.dim() == 2:
        batches, (M, NG) = 1, m8.shape
    else:
        batches, M, NG = m8.shape
    outs = []
    for static in (False, True):
        smask = torch.full(m8.shape, 0xAB, dtype=torch.uint8, device="cuda")
        sidx = torch.full(m8.shape, -7, dtype=torch.int64, device="cuda")
        counts = torch.full(m8.shape[:-2] + (NG,), -1, dtype=torch.int32, device="cuda")
        if static:
            rc = lib.dpk_route_compact_static(m8.data_ptr(), batches, M, NG, smask.data_ptr(),
                                              sidx.data_ptr(), counts.data_ptr(), st)
        else:
            nbytes = lib.dpk_route_workspace_bytes(batches, M, NG)
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
            rc = lib.dpk_route_compact(m8.data_ptr(), batches, M, NG, smask.data_ptr(),
                                       sidx.data_ptr(), counts.data_ptr(), ws.data_ptr(), nbytes, st)
        N.check(rc)
        outs.append((smask, sidx, counts))
    torch.cuda.synchronize()
    return outs


def test_static_scratch_matches_regular_entry_point_twice_in_a_row():
    from dpk_b200 import build
    build.build()
    from dpk_b200 import _native as N
    lib = N.load()

    g = torch.Generator().manual_seed(23)
    # two calls in a row with different shapes: the second must not see the first's counters
    masks = [torch.rand(8192, 112, generator=g) > 0.5,
             torch.rand(3, 1000, 8, generator=g) > 0.3,
             torch.rand(8192, 112, generator=g) > 0.7]
    for mask in masks:
        (rs, ri, rc_), (ss, si, sc) = _both(lib, N, mask.cuda())
        assert torch.equal(ss, rs), "sorted_mask differs"
        assert torch.equal(si, ri), "sorted_indices differ"
        assert torch.equal(sc, rc_), "counts differ"
        dim = 0 if mask.dim() == 2 else 1
        es, ei = torch.sort(mask, dim=dim, descending=True, stable=True)
        assert torch.equal(si.cpu(), ei) and torch.equal(ss.cpu().view(torch.bool), es)

    # beyond the built-in capacity of 65536 counters (this call would need 256 row blocks x
    # 512 groups = 131072): refused
    # on the host with a clear message; nothing is launched, so small buffers suffice
    dummy = torch.zeros(64, dtype=torch.int64, device="cuda")
    rc = lib.dpk_route_compact_static(dummy.data_ptr(), 1, 65536, 512, dummy.data_ptr(),
                                      dummy.data_ptr(), dummy.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == N.ERR_INVALID
    assert "built-in scratch" in N.last_error()
