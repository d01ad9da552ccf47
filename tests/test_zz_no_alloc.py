"""The entry point for callers that cannot allocate device memory.

`tuna_matmul_noalloc` takes no workspace: the streaming kernel's scratch lives in a device array
inside the library.  Servers that give all device memory to their own pool at start-up, or code that
must not trigger an allocation (and the device synchronisation it may imply) in the middle of a
serving loop, call it instead of `tuna_matmul`.  The test calls it through the C ABI twice in a row,
with different inputs, and expects the same bits as `tuna_matmul` (same kernel, same configuration).
It lives in the last-collected file so that a run stopping at the first failure has already run
everything else.
"""

import numpy as np
import pytest
import torch

from oracle import tuna_oracle as orc
from tuna_b200 import _lib
from tests.gpu_util import check_parity, make_case, run_matmul, stream_ptr

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(4096, 16, 4096), (1024, 7, 2048)])
def test_noalloc_matches_workspace_entry_point_twice_in_a_row(m, n, k):
    lib = _lib.load()
    for seed in (31, 32):  # second call: other inputs, scratch still holds the first call's partials
        host, dev = make_case(m, n, k, seed)
        st, ref_out, _ = run_matmul(dev, m, n, k)
        assert st == 0
        xd, qd, sd, cd = dev
        out = torch.full((n, m), float("nan"), dtype=torch.float16, device="cuda")
        st = lib.tuna_matmul_noalloc(qd.data_ptr(), xd.data_ptr(), cd.data_ptr(), sd.data_ptr(), out.data_ptr(),
                                     m, n, k, stream_ptr())
        torch.cuda.synchronize()
        assert st == 0, lib.tuna_status_string(st)
        got = out.cpu().numpy()
        assert np.array_equal(got.view(np.uint16), ref_out.cpu().numpy().view(np.uint16))
        check_parity(got, orc.matmul_ref(*host, m, n, k), 1e-2)


def test_noalloc_validates_like_the_other_entry_points():
    lib = _lib.load()
    t = torch.zeros(64, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    assert lib.tuna_matmul_noalloc(None, p, p, p, p, 64, 16, 64, stream_ptr()) == -1
    assert lib.tuna_matmul_noalloc(p, p, p, p, p, 60, 16, 64, stream_ptr()) == -2
    assert lib.tuna_matmul_noalloc(p + 2, p, p, p, p, 64, 16, 64, stream_ptr()) == -3
