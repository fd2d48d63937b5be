"""The allocation-free route inversion against the ordinary one, through the C ABI.

`vsa_route_invert_static` serves hosts that cannot give the library scratch memory (their own pool
owns the GPU, or allocation is forbidden where they call us): its cursor array is built into the
library.  It must give the same CSR as `vsa_route_invert` on every call, including a second call
that finds the previous call's leftovers in the shared array.  This file sorts last so that a
failure here cannot hide the other GPU tests in a run that stops at the first failure.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _invert(fn_name, selected, Kb):
    from simple_vsa_b200 import _lib
    B, H, Qb, tk = selected.shape
    counts = torch.full((B, H, Kb), -7, device=DEV, dtype=torch.int32)
    offsets = torch.full_like(counts, -7)
    inverse = torch.full((B, H, Qb * tk), -7, device=DEV, dtype=torch.int32)
    st = torch.cuda.current_stream().cuda_stream
    if fn_name == "vsa_route_invert":
        cursor = torch.empty_like(counts)
        _lib.call(fn_name, selected.data_ptr(), counts.data_ptr(), offsets.data_ptr(), inverse.data_ptr(),
                  cursor.data_ptr(), B * H, Qb, Kb, tk, st)
    else:
        _lib.call(fn_name, selected.data_ptr(), counts.data_ptr(), offsets.data_ptr(), inverse.data_ptr(),
                  B * H, Qb, Kb, tk, st)
    torch.cuda.synchronize()
    return counts.cpu().numpy(), offsets.cpu().numpy(), inverse.cpu().numpy()


def _same_csr(a, b):
    np.testing.assert_array_equal(a[0], b[0])          # counts: exact
    np.testing.assert_array_equal(a[1], b[1])          # offsets: exact
    counts, offsets = a[0], a[1]
    B, H, Kb = counts.shape
    for bi in range(B):
        for h in range(H):
            for kb in range(Kb):                        # order inside a key row is unspecified: compare as sets
                lo, n = offsets[bi, h, kb], counts[bi, h, kb]
                assert sorted(a[2][bi, h, lo:lo + n].tolist()) == sorted(b[2][bi, h, lo:lo + n].tolist())


def test_static_route_inversion_matches_on_two_calls_in_a_row():
    from simple_vsa_b200 import _lib
    g = torch.Generator().manual_seed(71)
    # first call: a larger table, so the second (smaller, different) call finds stale cursor entries
    first = torch.stack([torch.randperm(37, generator=g)[:9] for _ in range(2 * 3 * 21)]).to(torch.int32)
    first = first.reshape(2, 3, 21, 9).to(DEV)
    second = torch.stack([torch.randperm(11, generator=g)[:4] for _ in range(1 * 2 * 13)]).to(torch.int32)
    second = second.reshape(1, 2, 13, 4).to(DEV)
    for selected, Kb in ((first, 37), (second, 11)):
        _same_csr(_invert("vsa_route_invert_static", selected, Kb), _invert("vsa_route_invert", selected, Kb))
    assert _lib.device_status() == 0


def test_static_route_inversion_refuses_sizes_beyond_its_array():
    from simple_vsa_b200 import _lib
    x = torch.zeros(8, device=DEV, dtype=torch.int32)
    rc = _lib.lib.vsa_route_invert_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                          1024, 1, 1024, 1, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.ERR_UNSUPPORTED
    assert "exceeds the built-in scratch" in _lib.last_error()
