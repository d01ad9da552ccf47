"""The tcgen05/TMEM kernel against the oracle, through the C ABI, with explicit configurations."""

import ctypes

import numpy as np
import pytest
import torch

from oracle import tuna_oracle as orc
from tuna_b200 import _lib
from tests.gpu_util import check_parity, make_case, run_matmul

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _run(m, n, k, seed=0, **cfgd):
    host, dev = make_case(m, n, k, seed)
    cfg = _lib.TunaConfig(path=_lib.PATH_UMMA, **cfgd)
    st, out, holder = run_matmul(dev, m, n, k, cfg=cfg)
    lib = _lib.load()
    assert st == 0, lib.tuna_status_string(st)
    assert lib.tuna_check_device_status(torch.cuda.current_stream().cuda_stream) == 0, "a bounded wait ran out"
    check_parity(out.cpu().numpy(), orc.matmul_ref(*host, m, n, k), TOL)
    assert holder.guards_intact()


@pytest.mark.parametrize("m,n,k", [(128, 16, 64), (128, 16, 256), (256, 16, 512), (512, 16, 1024), (1024, 16, 2048)])
def test_umma_single_tile_then_many(m, n, k):
    _run(m, n, k, seed=m + k, tile_tok=16, row_blocks=1)


@pytest.mark.parametrize("row_blocks", [1, 2, 4])
@pytest.mark.parametrize("m,n,k", [(1024, 16, 1024), (136, 3, 72), (4104, 9, 520), (8, 1, 8)])
def test_umma_row_blocks_and_ragged_edges(m, n, k, row_blocks):
    _run(m, n, k, seed=1, tile_tok=16, row_blocks=row_blocks)


@pytest.mark.parametrize("ctas", [1, 3, 7, 148])
def test_umma_split_across_ctas_is_order_independent(ctas):
    # few tiles, many CTAs: every tile is cut across CTAs and finished through the workspace
    m, n, k = 512, 16, 4096
    host, dev = make_case(m, n, k, 4)
    ref = orc.matmul_ref(*host, m, n, k)
    cfg = _lib.TunaConfig(path=_lib.PATH_UMMA, tile_tok=16, row_blocks=1, ctas=ctas)
    first = None
    for _ in range(5):
        st, out, _h = run_matmul(dev, m, n, k, cfg=cfg)
        assert st == 0
        assert _lib.load().tuna_check_device_status(torch.cuda.current_stream().cuda_stream) == 0
        got = out.cpu().numpy()
        check_parity(got, ref, TOL)
        if first is None:
            first = got.view(np.uint16).copy()
        else:
            assert np.array_equal(first, got.view(np.uint16))


@pytest.mark.parametrize("n,tile_tok", [(17, 32), (64, 64), (100, 128), (256, 256), (300, 128), (520, 256)])
def test_umma_token_tiles(n, tile_tok):
    _run(640, n, 512, seed=n, tile_tok=tile_tok)


@pytest.mark.parametrize("m,k", [(6144, 4096), (28672, 4096), (4096, 14336)])
def test_umma_benchmark_shapes_m16(m, k):
    n = 16
    (x, q, absmax, code), dev = make_case(m, n, k, seed=m + k)
    cfg = _lib.TunaConfig(path=_lib.PATH_UMMA, tile_tok=16)
    st, out, holder = run_matmul(dev, m, n, k, cfg=cfg)
    assert st == 0
    assert _lib.load().tuna_check_device_status(torch.cuda.current_stream().cuda_stream) == 0
    rows = np.unique(np.concatenate([np.random.default_rng(0).integers(0, m // 8, 48), [0, m // 8 - 1]]))
    q3 = q.reshape(m // 8, k // 8, 32)
    ref = orc.matmul_ref(x, q3[rows], absmax.reshape(-1, 8)[rows].ravel(), code, len(rows) * 8, n, k)
    got = out.cpu().numpy().reshape(n, m // 8, 8)[:, rows].reshape(n, -1)
    check_parity(got, ref, TOL)
    assert holder.guards_intact()
