"""`tuna_matmul_sequence`: independent GEMMs in one persistent launch, against the oracle."""

import numpy as np
import pytest
import torch

import tuna_b200
from oracle import tuna_oracle as orc
from tuna_b200 import _lib
from tests.gpu_util import Guarded, check_parity, make_case, stream_ptr

pytestmark = pytest.mark.gpu
TOL = 1e-2  # max relative error budget of the GEMM (fp32 accumulation on both sides)


def _build(shapes, seed0=0):
    cases, gemms, holders = [], [], []
    for i, (m, n, k) in enumerate(shapes):
        host, (xd, qd, sd, cd) = make_case(m, n, k, seed0 + i)
        h = Guarded(n * m * 2, torch.float16, (n, m))
        cases.append(host)
        holders.append(h)
        gemms.append((xd, qd, sd, h.view, m, n, k))
    return cases, gemms, holders, cd


def _check(shapes, cases, holders):
    for (m, n, k), host, h in zip(shapes, cases, holders):
        check_parity(h.view.cpu().numpy(), orc.matmul_ref(*host, m, n, k), TOL)
        assert h.guards_intact()


MIXED = [(4096, 16, 1024), (136, 3, 72), (1024, 16, 4096), (8, 1, 8), (520, 9, 264), (2048, 16, 2048), (128, 16, 128)]


def test_sequence_of_mixed_shapes_matches_the_oracle():
    cases, gemms, holders, code = _build(MIXED)
    tuna_b200.matmul_sequence(gemms, code)
    torch.cuda.synchronize()
    assert _lib.load().tuna_check_device_status(stream_ptr()) == 0, "a bounded wait ran out"
    _check(MIXED, cases, holders)


def test_sequence_is_deterministic_and_reusable():
    shapes = [(512, 16, 4096), (4096, 16, 512), (1024, 7, 2048)] * 3
    cases, gemms, holders, code = _build(shapes, seed0=40)
    seq = tuna_b200.MatmulSequence(gemms, code)
    first = None
    for _ in range(4):
        for h in holders:
            h.view.fill_(float("nan"))  # garbage on purpose: the outputs need no zero fill
        seq.run()
        torch.cuda.synchronize()
        got = [h.view.cpu().numpy().view(np.uint16).copy() for h in holders]
        if first is None:
            first = got
        else:
            assert all(np.array_equal(a, b) for a, b in zip(first, got))
    assert _lib.load().tuna_check_device_status(stream_ptr()) == 0
    _check(shapes, cases, holders)


def test_sequence_longer_than_one_launch():
    shapes = [(256 + 8 * (i % 5), 1 + (i % 16), 256 + 64 * (i % 3)) for i in range(70)]  # 64 GEMMs per launch
    cases, gemms, holders, code = _build(shapes, seed0=100)
    tuna_b200.matmul_sequence(gemms, code)
    torch.cuda.synchronize()
    assert _lib.load().tuna_check_device_status(stream_ptr()) == 0
    _check(shapes, cases, holders)


def test_sequence_with_more_tokens_than_one_pass_falls_back_per_gemm():
    shapes = [(512, 100, 512), (256, 16, 1024)]
    cases, gemms, holders, code = _build(shapes, seed0=7)
    tuna_b200.matmul_sequence(gemms, code)
    torch.cuda.synchronize()
    _check(shapes, cases, holders)


def test_sequence_token_tiles_32_and_64():
    for n in (24, 48):
        shapes = [(640, n, 520), (1024, n - 7, 1024), (256, n, 2048)]
        cases, gemms, holders, code = _build(shapes, seed0=n)
        tuna_b200.matmul_sequence(gemms, code)
        torch.cuda.synchronize()
        assert _lib.load().tuna_check_device_status(stream_ptr()) == 0
        _check(shapes, cases, holders)


def test_sequence_mistral_mlp_layers_full_size():
    """Two layers of the benchmark's GEMMs in one launch; the oracle runs on sampled row groups."""
    shapes = [(28672, 16, 4096), (4096, 16, 14336)] * 2
    cases, gemms, holders, code = _build(shapes, seed0=900)
    tuna_b200.matmul_sequence(gemms, code)
    torch.cuda.synchronize()
    assert _lib.load().tuna_check_device_status(stream_ptr()) == 0
    rng = np.random.default_rng(1)
    for (m, n, k), (x, q, absmax, code_h), h in zip(shapes, cases, holders):
        rows = np.unique(np.concatenate([rng.integers(0, m // 8, 24), [0, m // 8 - 1]]))
        q3 = q.reshape(m // 8, k // 8, 32)
        ref = orc.matmul_ref(x, q3[rows], absmax.reshape(-1, 8)[rows].ravel(), code_h, len(rows) * 8, n, k)
        got = h.view.cpu().numpy().reshape(n, m // 8, 8)[:, rows].reshape(n, -1)
        check_parity(got, ref, TOL)
        assert h.guards_intact()


def test_sequence_as_grouped_gemm_with_per_expert_token_lists():
    """Eight experts of one shape, unequal token counts (one expert without tokens): every expert's
    rows of one shared activation / output buffer, one launch; parity per expert."""
    m, k, experts = 1024, 2048, 8
    counts = [5, 0, 16, 1, 9, 3, 12, 7]
    rng = np.random.default_rng(3)
    total = sum(counts)
    x_all = torch.from_numpy(rng.standard_normal((total, k)).astype(np.float16)).cuda()
    o_all = Guarded(total * m * 2, torch.float16, (total, m))
    o_all.view.fill_(float("nan"))
    gemms, hosts, off = [], [], 0
    for e, n in enumerate(counts):
        (x, q, absmax, code), (xd, qd, sd, cd) = make_case(m, max(n, 1), k, 200 + e)
        gemms.append((x_all[off:off + n], qd, sd, o_all.view[off:off + n], m, n, k))
        hosts.append((q, absmax, code, off, n))
        off += n
    tuna_b200.matmul_sequence(gemms, cd)
    torch.cuda.synchronize()
    assert _lib.load().tuna_check_device_status(stream_ptr()) == 0
    xh = x_all.cpu().numpy()
    got = o_all.view.cpu().numpy()
    for q, absmax, code, off, n in hosts:
        if n:
            check_parity(got[off:off + n], orc.matmul_ref(xh[off:off + n], q, absmax, code, m, n, k), TOL)
    assert o_all.guards_intact()


def test_sequence_validates_its_arguments():
    lib = _lib.load()
    t = torch.zeros(256, dtype=torch.uint8, device="cuda")
    p = t.data_ptr()
    d = (_lib.TunaGemmDesc * 1)(_lib.TunaGemmDesc(p, p, p, p, 60, 16, 64, 0))
    assert lib.tuna_matmul_sequence(d, 1, p, p, 1 << 20, stream_ptr()) == -2
    d[0] = _lib.TunaGemmDesc(p, None, p, p, 64, 16, 64, 0)
    assert lib.tuna_matmul_sequence(d, 1, p, p, 1 << 20, stream_ptr()) == -1
    d[0] = _lib.TunaGemmDesc(p, p, p, p, 64, 16, 64, 0)
    assert lib.tuna_matmul_sequence(d, 0, p, p, 1 << 20, stream_ptr()) == -2
    assert lib.tuna_matmul_sequence(d, 1, p, p, 16, stream_ptr()) == -4
