"""The entry point for callers that cannot allocate device memory.

`tuna_matmul_noalloc` takes no workspace: the streaming kernel's scratch lives in a device array
inside the library.  Servers that give all device memory to their own pool at start-up, or code that
must not trigger an allocation (and the device synchronisation it may imply) in the middle of a
serving loop, call it instead of `tuna_matmul`.  The tests call it through the C ABI twice in a row,
with different inputs, and expect `tuna_matmul`'s result within the GEMM tolerance (and the same bits as
the same kernel and configuration run with a caller workspace).
It lives in the last-collected file so that a run stopping at the first failure has already run
everything else.
"""

import ctypes

import numpy as np
import pytest
import torch

from oracle import tuna_oracle as orc
from tuna_b200 import _lib
from tests.gpu_util import check_parity, make_case, run_matmul, stream_ptr

pytestmark = pytest.mark.gpu


def _same_kernel_config(lib, m, n, k):
    """The configuration the entry point uses: the table's when it is a streaming one, else the
    streaming kernel's own heuristic."""
    cfg = _lib.TunaConfig()
    assert lib.tuna_lookup_config(m, n, k, ctypes.byref(cfg)) == 0
    if cfg.path != _lib.PATH_STREAM:
        cfg = _lib.TunaConfig(path=_lib.PATH_STREAM)
    return cfg


def _noalloc(lib, dev, m, n, k):
    xd, qd, sd, cd = dev
    out = torch.full((n, m), float("nan"), dtype=torch.float16, device="cuda")
    st = lib.tuna_matmul_noalloc(qd.data_ptr(), xd.data_ptr(), cd.data_ptr(), sd.data_ptr(), out.data_ptr(),
                                 m, n, k, stream_ptr())
    torch.cuda.synchronize()
    assert st == 0, lib.tuna_status_string(st)
    return out.cpu().numpy()


@pytest.mark.parametrize("m,n,k", [(4096, 16, 4096), (1024, 7, 2048), (1024, 40, 2048), (520, 100, 264)])
def test_noalloc_matches_workspace_entry_point_twice_in_a_row(m, n, k):
    """Against tuna_matmul within the GEMM tolerance (1e-2), and bit for bit against the same
    kernel and configuration run with a caller workspace.  40 and 100 tokens run as several passes."""
    lib = _lib.load()
    for seed in (31, 32):  # second call: other inputs, scratch still holds the first call's partials
        host, dev = make_case(m, n, k, seed)
        st, ref_out, _ = run_matmul(dev, m, n, k)
        assert st == 0
        st, same_out, _ = run_matmul(dev, m, n, k, cfg=_same_kernel_config(lib, m, n, k))
        assert st == 0
        got = _noalloc(lib, dev, m, n, k)
        check_parity(got, ref_out.cpu().numpy(), 1e-2)
        assert np.array_equal(got.view(np.uint16), same_out.cpu().numpy().view(np.uint16))
        check_parity(got, orc.matmul_ref(*host, m, n, k), 1e-2)


def test_noalloc_alternating_shapes_share_the_scratch():
    """Two shapes with different tile counts and split patterns, in turn, on the one array."""
    lib = _lib.load()
    shapes = [(256, 16, 8192), (4096, 16, 2048)]
    cases = [make_case(m, n, k, 60 + i) for i, (m, n, k) in enumerate(shapes)]
    refs = [orc.matmul_ref(*cases[i][0], *shapes[i]) for i in range(2)]
    for rep in range(3):
        for i, (m, n, k) in enumerate(shapes):
            check_parity(_noalloc(lib, cases[i][1], m, n, k), refs[i], 1e-2)


def test_noalloc_refuses_what_does_not_fit():
    """A matrix whose tile counters alone exceed the array: refused before anything is launched
    (the pointers are never dereferenced)."""
    lib = _lib.load()
    t = torch.zeros(64, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    assert lib.tuna_matmul_noalloc(p, p, p, p, p, 8 * 40_000_000, 16, 8, stream_ptr()) == -9


def test_noalloc_validates_like_the_other_entry_points():
    lib = _lib.load()
    t = torch.zeros(64, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    assert lib.tuna_matmul_noalloc(None, p, p, p, p, 64, 16, 64, stream_ptr()) == -1
    assert lib.tuna_matmul_noalloc(p, p, p, p, p, 60, 16, 64, stream_ptr()) == -2
    assert lib.tuna_matmul_noalloc(p + 2, p, p, p, p, 64, 16, 64, stream_ptr()) == -3
