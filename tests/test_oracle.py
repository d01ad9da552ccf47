"""The oracle itself: layout, dequant and GEMM restatements against each other
(numpy vs C) and against the fixtures produced by the reference's own kernels."""

import ctypes
from pathlib import Path

import numpy as np
import pytest

from oracle import tuna_oracle as orc

GOLDEN = Path(__file__).parent / "golden"


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def test_pack_matches_reference_expression():
    # test.py:58-65 written out literally with numpy reshape/permute
    rng = np.random.default_rng(1)
    m, k = 48, 80
    codes = rng.integers(0, 16, (m, k), dtype=np.uint8)
    r = codes.reshape(-1, m // 8, 8, k // 8, 4, 2).transpose(0, 1, 3, 2, 4, 5).reshape(-1, m // 8, k // 8, 32, 2)
    ref = (r[..., 0] * 16 + r[..., 1]).reshape(m // 8, k // 8, 32).astype(np.uint8)
    assert np.array_equal(orc.pack_codes(codes), ref)


def test_byte_position_rule():
    m, k = 16, 24
    codes = (np.arange(m * k).reshape(m, k) % 16).astype(np.uint8)
    q = orc.pack_codes(codes)
    for mt in range(m // 8):
        for kt in range(k // 8):
            for j in range(32):
                hi, lo = q[mt, kt, j] >> 4, q[mt, kt, j] & 15
                assert hi == codes[8 * mt + j // 4, 8 * kt + 2 * (j % 4)]
                assert lo == codes[8 * mt + j // 4, 8 * kt + 2 * (j % 4) + 1]


@pytest.mark.parametrize("m,k", [(8, 8), (64, 64), (128, 72), (24, 4096)])
def test_pack_unpack_roundtrip_numpy_and_c(oracle_c, m, k):
    rng = np.random.default_rng(m * 1000 + k)
    codes = rng.integers(0, 16, (m, k), dtype=np.uint8)
    q = orc.pack_codes(codes)
    assert q.shape == (m // 8, k // 8, 32)
    assert np.array_equal(orc.unpack_codes(q, m, k), codes)
    qc = np.empty(m * k // 2, dtype=np.uint8)
    oracle_c.oracle_pack(_ptr(codes), _ptr(qc), m, k)
    assert np.array_equal(qc, q.ravel())
    back = np.empty((m, k), dtype=np.uint8)
    oracle_c.oracle_unpack(_ptr(qc), _ptr(back), m, k)
    assert np.array_equal(back, codes)


@pytest.mark.parametrize("m,k,seed", [(64, 64, 0), (128, 256, 1), (8, 4096, 2)])
def test_dequant_numpy_equals_c_bitwise(oracle_c, m, k, seed):
    x, q, absmax, code = orc.synth_inputs(m, 1, k, seed)
    ref = orc.dequant_ref(q, absmax, code, m, k)
    out = np.empty((m, k), dtype=np.uint16)
    oracle_c.oracle_dequant(_ptr(q), _ptr(absmax), _ptr(code), _ptr(out), m, k)
    assert np.array_equal(out, ref.view(np.uint16))


def test_dequant_scalar_loop():
    m, k = 16, 16
    _, q, absmax, code = orc.synth_inputs(m, 1, k, 5)
    ref = orc.dequant_ref(q, absmax, code, m, k)
    codes = orc.unpack_codes(q, m, k)
    for r in range(m):
        for c in range(k):
            v = np.float16(np.float32(code[codes[r, c]]) * np.float32(absmax[r]))
            assert v.view(np.uint16) == ref[r, c].view(np.uint16)


def test_two_dequant_definitions_differ_by_at_most_one_ulp():
    m, k = 256, 64
    _, q, absmax, code = orc.synth_inputs(m, 1, k, 7)
    a = orc.dequant_ref(q, absmax, code, m, k).view(np.int16).astype(np.int32)
    b = orc.dequant_gemm_internal(q, absmax, code, m, k).view(np.int16).astype(np.int32)
    assert np.abs(a - b).max() <= 1
    assert (a != b).mean() < 0.5


@pytest.mark.parametrize("m,n,k", [(64, 1, 64), (128, 16, 256), (64, 7, 1024)])
def test_matmul_numpy_vs_c(oracle_c, m, n, k):
    x, q, absmax, code = orc.synth_inputs(m, n, k, 11)
    ref64 = orc.matmul_ref(x, q, absmax, code, m, n, k, accum="f64")
    ref32 = orc.matmul_ref(x, q, absmax, code, m, n, k, accum="f32")
    out = np.empty((n, m), dtype=np.uint16)
    oracle_c.oracle_matmul(_ptr(x), _ptr(q), _ptr(code), _ptr(absmax), _ptr(out), m, n, k)
    outc = out.view(np.float16)
    for ref in (ref64, ref32):
        a, b = orc.parity_error(outc, ref)
        assert a < 2e-3 and b < 4e-3, (a, b)


def test_quantizer_roundtrip():
    rng = np.random.default_rng(3)
    m, k = 32, 128
    w = (rng.standard_normal((m, k)) * 0.05).astype(np.float16)
    q, absmax, code = orc.quantize_blockwise_dynamic_4bit(w)
    assert q.shape == (m // 8, k // 8, 32) and absmax.shape == (m,)
    assert np.allclose(absmax, np.abs(w.astype(np.float32)).max(1))
    deq = orc.dequant_ref(q, absmax, code, m, k).astype(np.float32)
    # NF4 grid spacing is at most ~0.3 of absmax between neighbours
    assert np.abs(deq - w.astype(np.float32)).max() <= 0.16 * absmax.max()
    codes = orc.unpack_codes(q, m, k)
    # the row maximum maps to an end of the codebook
    for r in range(m):
        j = np.abs(w[r].astype(np.float32)).argmax()
        assert codes[r, j] in (0, 15)


def test_synth_scales_are_fp16_representable():
    _, _, absmax, _ = orc.synth_inputs(64, 1, 64, 0)
    assert absmax.dtype == np.float32
    assert np.array_equal(absmax.astype(np.float16).astype(np.float32), absmax)
    assert absmax.min() >= 0.0049 and absmax.max() <= 0.0201


def _golden_files():
    return sorted(GOLDEN.glob("ref_*.npz"))


@pytest.mark.parametrize("path", _golden_files() or [None])
def test_oracle_against_reference_fixtures(path):
    """Fixtures hold what the reference's own CUDA kernels produced on a B200 for seeded
    inputs (tests/golden/make_reference_fixtures.py)."""
    if path is None:
        pytest.skip("no reference fixtures committed yet")
    z = np.load(path)
    m, n, k, seed = (int(z[s]) for s in ("m", "n", "k", "seed"))
    x, q, absmax, code = orc.synth_inputs(m, n, k, seed)
    if "dequant_sample" in z:
        w16 = orc.dequant_ref(q, absmax, code, m, k)
        rows = z["dequant_rows"]
        assert np.array_equal(w16[rows].view(np.uint16), z["dequant_sample"])
    if "matmul" in z:
        ref = orc.matmul_ref(x, q, absmax, code, m, n, k)
        a, b = orc.parity_error(z["matmul"].view(np.float16), ref)
        assert a <= 1e-2 and b <= 2e-2, (a, b)


def test_quantizer_matches_torch_cpu_fixture():
    """The quantizer restatement against outputs of the reference's torch expression evaluated on
    the CPU (tests/golden/make_quantizer_fixture.py): a zero row, a constant row, exact midpoints."""
    d = np.load(GOLDEN / "quantizer_torch_cpu.npz")
    w = d["w_bits"].view(np.float16)
    q, absmax, _ = orc.quantize_blockwise_dynamic_4bit(w)
    assert np.array_equal(absmax, d["absmax"])
    assert np.array_equal(q, d["q"])
