"""The tcgen05 weight-streaming kernel against the oracle, through the C ABI, with explicit configurations."""

import numpy as np
import pytest
import torch

from oracle import tuna_oracle as orc
from tuna_b200 import _lib
from tests.gpu_util import check_parity, make_case, run_matmul

pytestmark = pytest.mark.gpu
TOL = 1e-2  # max relative error budget of the GEMM (fp32 accumulation on both sides)


def _status_ok():
    assert _lib.load().tuna_check_device_status(torch.cuda.current_stream().cuda_stream) == 0, "a bounded wait ran out"


def _run(m, n, k, seed=0, **cfgd):
    host, dev = make_case(m, n, k, seed)
    cfg = _lib.TunaConfig(path=_lib.PATH_TSTREAM, **cfgd)
    st, out, holder = run_matmul(dev, m, n, k, cfg=cfg)
    assert st == 0, _lib.load().tuna_status_string(st)
    _status_ok()
    check_parity(out.cpu().numpy(), orc.matmul_ref(*host, m, n, k), TOL)
    assert holder.guards_intact()


def test_tstream_one_hot_activations_recover_the_weights():
    """x = one-hot rows: o[tok, row] must be the dequantised weight W[row, k_tok] exactly (one
    product, no rounding beyond the scale) - a wrong row or K permutation shows up as a wrong value."""
    m, n, k = 256, 16, 256
    (x, q, absmax, code), _ = make_case(m, n, k, seed=3)
    cols = np.array([0, 1, 2, 5, 8, 13, 31, 32, 47, 100, 127, 128, 129, 200, 254, 255])
    x = np.zeros((n, k), dtype=np.float16)
    x[np.arange(n), cols] = 1.0
    dev = [torch.from_numpy(a).cuda() for a in (x, q, absmax, code)]
    st, out, holder = run_matmul(dev, m, n, k, cfg=_lib.TunaConfig(path=_lib.PATH_TSTREAM, tile_tok=16))
    assert st == 0
    _status_ok()
    w = orc.unpack_codes(q, m, k)
    want = (code[w[:, cols]].astype(np.float16).astype(np.float32) * absmax[:, None]).astype(np.float16).T
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    assert holder.guards_intact()


@pytest.mark.parametrize("k_steps", [4, 8])
@pytest.mark.parametrize("m,n,k", [(128, 16, 128), (128, 16, 256), (256, 16, 512), (512, 16, 1024), (1024, 16, 2048)])
def test_tstream_single_tile_then_many(m, n, k, k_steps):
    _run(m, n, k, seed=m + k, tile_tok=16, row_blocks=1, k_steps=k_steps)


@pytest.mark.parametrize("k_steps", [4, 8])
@pytest.mark.parametrize("row_blocks", [1, 2, 4])
@pytest.mark.parametrize("m,n,k", [(1024, 16, 1024), (136, 3, 72), (4104, 9, 520), (8, 1, 8)])
def test_tstream_row_blocks_and_ragged_edges(m, n, k, row_blocks, k_steps):
    _run(m, n, k, seed=1, tile_tok=16, row_blocks=row_blocks, k_steps=k_steps)


@pytest.mark.parametrize("k_steps", [4, 8])
@pytest.mark.parametrize("ctas", [1, 3, 7, 148])
def test_tstream_split_across_ctas_is_order_independent(ctas, k_steps):
    # few tiles, many CTAs: every tile is cut across CTAs and finished through the workspace
    m, n, k = 512, 16, 4096
    host, dev = make_case(m, n, k, 4)
    ref = orc.matmul_ref(*host, m, n, k)
    cfg = _lib.TunaConfig(path=_lib.PATH_TSTREAM, tile_tok=16, row_blocks=1, ctas=ctas, k_steps=k_steps)
    first = None
    for _ in range(5):
        out = torch.full((n, m), float("nan"), dtype=torch.float16, device="cuda")  # garbage on purpose
        st, out, _h = run_matmul(dev, m, n, k, cfg=cfg, out=out)
        assert st == 0
        _status_ok()
        got = out.cpu().numpy()
        check_parity(got, ref, TOL)
        if first is None:
            first = got.view(np.uint16).copy()
        else:
            assert np.array_equal(first, got.view(np.uint16))


@pytest.mark.parametrize("k_steps", [4, 8])
@pytest.mark.parametrize("n,tile_tok,row_blocks", [(17, 32, 1), (32, 32, 2), (40, 16, 1), (64, 64, 1), (100, 64, 1), (33, 32, 2)])
def test_tstream_token_tiles_and_passes(n, tile_tok, row_blocks, k_steps):
    _run(640, n, 520, seed=n, tile_tok=tile_tok, row_blocks=row_blocks, k_steps=k_steps)


@pytest.mark.parametrize("m,n,k", [(640, 128, 512), (640, 100, 520), (1024, 300, 2048), (264, 129, 200), (28672, 256, 4096)])
def test_tstream_128_token_tiles(m, n, k):
    """Passes of 128 tokens (128-column slots, one row block): every stage layout, ragged token counts."""
    _run(m, n, k, seed=m + n, tile_tok=128, row_blocks=1, k_steps=4)


@pytest.mark.parametrize("k_steps", [4, 8])
@pytest.mark.parametrize("m,n,k,tile_tok", [
    (640, 64, 512, 64), (640, 33, 1024, 64), (1024, 32, 2048, 32),   # 5-D view (m % 32 = 0, k % 64 = 0), larger token tiles
    (136, 16, 96, 16), (256, 16, 160, 16), (1032, 40, 2080, 64),     # 3-D view (k % 32 = 0 only): [step][row group] stages
    (264, 16, 200, 16), (640, 64, 520, 64),                          # 2-D view, one box per step
])
def test_tstream_every_weight_stage_layout(m, n, k, tile_tok, k_steps):
    _run(m, n, k, seed=m + n + k, tile_tok=tile_tok, row_blocks=1, k_steps=k_steps)


@pytest.mark.parametrize("m,k", [(264, 200), (256, 160), (256, 256)])
def test_tstream_one_hot_in_every_stage_layout(m, k):
    """The one-hot check (exact weights back) for the three views of the packed matrix."""
    n = 16
    (x, q, absmax, code), _ = make_case(m, n, k, seed=5)
    cols = np.linspace(0, k - 1, n).astype(np.int64)
    x = np.zeros((n, k), dtype=np.float16)
    x[np.arange(n), cols] = 1.0
    dev = [torch.from_numpy(a).cuda() for a in (x, q, absmax, code)]
    st, out, holder = run_matmul(dev, m, n, k, cfg=_lib.TunaConfig(path=_lib.PATH_TSTREAM, tile_tok=16))
    assert st == 0
    _status_ok()
    w = orc.unpack_codes(q, m, k)
    want = (code[w[:, cols]].astype(np.float16).astype(np.float32) * absmax[:, None]).astype(np.float16).T
    assert np.array_equal(out.cpu().numpy().view(np.uint16), want.view(np.uint16))
    assert holder.guards_intact()


@pytest.mark.parametrize("m,k", [(6144, 4096), (28672, 4096), (4096, 14336), (57344, 8192)])
def test_tstream_benchmark_shapes_m16(m, k):
    n = 16
    (x, q, absmax, code), dev = make_case(m, n, k, seed=m + k)
    cfg = _lib.TunaConfig(path=_lib.PATH_TSTREAM, tile_tok=16)
    st, out, holder = run_matmul(dev, m, n, k, cfg=cfg)
    assert st == 0
    _status_ok()
    rows = np.unique(np.concatenate([np.random.default_rng(0).integers(0, m // 8, 48), [0, m // 8 - 1]]))
    q3 = q.reshape(m // 8, k // 8, 32)
    ref = orc.matmul_ref(x, q3[rows], absmax.reshape(-1, 8)[rows].ravel(), code, len(rows) * 8, n, k)
    got = out.cpu().numpy().reshape(n, m // 8, 8)[:, rows].reshape(n, -1)
    check_parity(got, ref, TOL)
    assert holder.guards_intact()
