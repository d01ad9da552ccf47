"""Parity of the CUDA path against the oracle, through the C ABI, on a B200."""

import ctypes

import numpy as np
import pytest
import torch

from oracle import tuna_oracle as orc
from tuna_b200 import _lib
from tests.gpu_util import Guarded, check_parity, make_case, run_matmul, stream_ptr, to_dev

pytestmark = pytest.mark.gpu

# max relative error budget of the GEMM: 1e-2 (fp32 accumulation on both sides)
TOL = 1e-2


# ----------------------------------------------------------------- dequant: bit exact

@pytest.mark.parametrize("m,k", [(8, 8), (64, 64), (72, 136), (128, 4096), (4096, 4096), (1000 * 8, 264)])
def test_dequant_bit_exact(m, k):
    lib = _lib.load()
    (x, q, absmax, code), (xd, qd, sd, cd) = make_case(m, 1, k, seed=m + k)
    out = Guarded(m * k * 2, torch.float16, (m, k))
    st = lib.tuna_dequant(qd.data_ptr(), sd.data_ptr(), cd.data_ptr(), out.view.data_ptr(), m, k, stream_ptr())
    torch.cuda.synchronize()
    assert st == 0
    ref = orc.dequant_ref(q, absmax, code, m, k)
    got = out.view.cpu().numpy()
    assert np.array_equal(got.view(np.uint16), ref.view(np.uint16))
    assert out.guards_intact()


def test_dequant_arbitrary_codebook_and_scales():
    lib = _lib.load()
    m, k = 256, 512
    rng = np.random.default_rng(9)
    codes = rng.integers(0, 16, (m, k), dtype=np.uint8)
    q = orc.pack_codes(codes)
    code = rng.standard_normal(16).astype(np.float32)
    absmax = np.exp(rng.uniform(-12, 6, m)).astype(np.float32)  # includes fp16 subnormal products and overflow
    qd, sd, cd = to_dev(q, absmax, code)
    out = torch.empty((m, k), dtype=torch.float16, device="cuda")
    assert lib.tuna_dequant(qd.data_ptr(), sd.data_ptr(), cd.data_ptr(), out.data_ptr(), m, k, stream_ptr()) == 0
    torch.cuda.synchronize()
    ref = orc.dequant_ref(q, absmax, code, m, k)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), ref.view(np.uint16))


# ----------------------------------------------------------------- GEMM: tolerance 1e-2

SMALL_SHAPES = [  # (m, k): awkward sizes, partial tiles, k not a multiple of 32
    (8, 8), (64, 64), (128, 64), (136, 72), (520, 264), (1024, 1024), (4104, 520),
]


@pytest.mark.parametrize("n", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("m,k", SMALL_SHAPES)
def test_matmul_small_shapes(m, k, n):
    host, dev = make_case(m, n, k, seed=m * 7 + k + n)
    st, out, holder = run_matmul(dev, m, n, k)
    assert st == 0, _lib.load().tuna_status_string(st)
    ref = orc.matmul_ref(*host, m, n, k)
    check_parity(out.cpu().numpy(), ref, TOL)
    assert holder.guards_intact()


BASELINE_SHAPES = [
    (6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336),
    (10240, 8192), (8192, 8192), (57344, 8192), (8192, 28672),
]


@pytest.mark.parametrize("m,k", BASELINE_SHAPES)
def test_matmul_baseline_shapes_m16(m, k):
    """Full benchmark sizes; the oracle runs on a random sample of output rows."""
    n = 16
    (x, q, absmax, code), dev = make_case(m, n, k, seed=m + k)
    st, out, holder = run_matmul(dev, m, n, k)
    assert st == 0
    rng = np.random.default_rng(0)
    rows = np.unique(np.concatenate([rng.integers(0, m // 8, 48), [0, m // 8 - 1]]))
    q3 = q.reshape(m // 8, k // 8, 32)
    ref = orc.matmul_ref(x, q3[rows], absmax.reshape(-1, 8)[rows].ravel(), code, len(rows) * 8, n, k)
    got = out.cpu().numpy().reshape(n, m // 8, 8)[:, rows].reshape(n, -1)
    check_parity(got, ref, TOL)
    assert holder.guards_intact()


def test_matmul_linearity_full_size():
    """Size-independent property at a full benchmark size: the op is linear in x, so
    f(x1 + x2) == f(x1) + f(x2) up to fp16 rounding of the three outputs."""
    m, n, k = 28672, 16, 4096
    (x, q, absmax, code), (xd, qd, sd, cd) = make_case(m, n, k, seed=5)
    x2 = np.random.default_rng(6).standard_normal((n, k)).astype(np.float16)
    x2d, = to_dev(x2)
    xsum = (xd.float() + x2d.float()).half()
    outs = []
    for xin in (xd, x2d, xsum):
        st, o, _ = run_matmul((xin, qd, sd, cd), m, n, k)
        assert st == 0
        outs.append(o.float())
    # compare against the sum computed from the rounded inputs' exact linear combination
    lhs = outs[2]
    rhs = outs[0] + outs[1]
    err = (lhs - rhs).abs().max().item() / rhs.abs().max().item()
    assert err < 4e-3, err


@pytest.mark.parametrize("m,k,n", [(4096, 4096, 16), (4096, 14336, 16), (520, 264, 5)])
def test_matmul_is_deterministic_and_needs_no_zero_fill(m, k, n):
    host, dev = make_case(m, n, k, seed=1)
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    first = None
    for it in range(10):
        out = torch.full((n, m), float("nan"), dtype=torch.float16, device="cuda")  # garbage on purpose
        st, out, _ = run_matmul(dev, m, n, k, out=out, ws=ws)
        assert st == 0
        got = out.cpu().numpy().view(np.uint16)
        if first is None:
            first = got
        else:
            assert np.array_equal(first, got), f"run {it} differs"
    # the workspace is left clean: only partial sums may remain; the arrival counters, which live
    # behind the partial region (2 slots x SMs x 192 KB), are zero again
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    counters_at = 2 * sms * 192 * 1024
    need = int(_lib.load().tuna_matmul_workspace_bytes(m, n, k))
    assert need > counters_at
    assert int(ws[counters_at:need].view(torch.int32).abs().sum()) == 0
    assert _lib.load().tuna_check_device_status(stream_ptr()) == 0


STREAM_CONFIGS = [
    dict(rows_per_warp=r, warps_m=wm, warps_k=wk, k_steps=ks, tile_tok=tt, ctas=ctas)
    for (r, wm, wk, ks, tt, ctas) in [
        (1, 1, 1, 8, 16, 0), (1, 16, 1, 8, 16, 0), (1, 4, 4, 8, 16, 0), (2, 4, 4, 4, 16, 0), (2, 16, 1, 16, 16, 0),
        (2, 2, 8, 4, 16, 3), (2, 8, 2, 4, 16, 7), (1, 4, 4, 8, 8, 0), (2, 16, 1, 4, 8, 5), (2, 2, 2, 8, 8, 148),
        (1, 16, 1, 8, 32, 0), (1, 4, 2, 8, 32, 11),
    ]
]


@pytest.mark.parametrize("cfgd", STREAM_CONFIGS)
@pytest.mark.parametrize("m,k,n", [(1024, 2048, 16), (4104, 520, 7)])
def test_stream_kernel_every_template_and_split(m, k, n, cfgd):
    host, dev = make_case(m, n, k, seed=3)
    cfg = _lib.TunaConfig(path=_lib.PATH_STREAM, **cfgd)
    st, out, holder = run_matmul(dev, m, n, k, cfg=cfg)
    assert st == 0, _lib.load().tuna_status_string(st)
    assert _lib.load().tuna_check_device_status(stream_ptr()) == 0, "a bounded wait ran out"
    check_parity(out.cpu().numpy(), orc.matmul_ref(*host, m, n, k), TOL)
    assert holder.guards_intact()


@pytest.mark.parametrize("n", [17, 31, 32, 40])
def test_stream_kernel_token_passes(n):
    """More tokens than one pass holds: the launcher loops over token groups."""
    m, k = 520, 264
    host, dev = make_case(m, n, k, seed=n)
    cfg = _lib.TunaConfig(path=_lib.PATH_STREAM, tile_tok=16)
    st, out, holder = run_matmul(dev, m, n, k, cfg=cfg)
    assert st == 0
    check_parity(out.cpu().numpy(), orc.matmul_ref(*host, m, n, k), TOL)
    assert holder.guards_intact()


def test_matmul_extreme_values():
    """Codes all at the ends of the codebook and large activations: no overflow inside the
    fp32 accumulation, fp16 result saturates only where the oracle's does."""
    m, n, k = 256, 16, 1024
    rng = np.random.default_rng(2)
    codes = rng.choice(np.array([0, 15], dtype=np.uint8), size=(m, k))
    q = orc.pack_codes(codes)
    absmax = np.full(m, 0.02, dtype=np.float32)
    x = (rng.standard_normal((n, k)) * 30).astype(np.float16)
    code = orc.NF4_CODE.copy()
    dev = to_dev(x, q, absmax, code)
    st, out, _ = run_matmul(dev, m, n, k)
    assert st == 0
    check_parity(out.cpu().numpy(), orc.matmul_ref(x, q, absmax, code, m, n, k), TOL)


def test_golden_fixtures_against_cuda():
    """The committed reference-kernel outputs, compared with the CUDA path directly."""
    from pathlib import Path

    files = sorted((Path(__file__).parent / "golden").glob("ref_*.npz"))
    if not files:
        pytest.skip("no reference fixtures committed yet")
    lib = _lib.load()
    for path in files:
        z = np.load(path)
        m, n, k, seed = (int(z[s]) for s in ("m", "n", "k", "seed"))
        (x, q, absmax, code), dev = make_case(m, n, k, seed)
        if "matmul" in z:
            st, out, _ = run_matmul(dev, m, n, k)
            assert st == 0
            check_parity(out.cpu().numpy(), z["matmul"].view(np.float16), 2e-2)
        if "dequant_sample" in z:
            o = torch.empty((m, k), dtype=torch.float16, device="cuda")
            assert lib.tuna_dequant(dev[1].data_ptr(), dev[2].data_ptr(), dev[3].data_ptr(), o.data_ptr(), m, k, stream_ptr()) == 0
            torch.cuda.synchronize()
            got = o.cpu().numpy()[z["dequant_rows"]]
            assert np.array_equal(got.view(np.uint16), z["dequant_sample"])


def test_python_mirror_matches_c_abi():
    import tuna_b200

    m, n, k = 1024, 16, 1024
    host, (xd, qd, sd, cd) = make_case(m, n, k, seed=8)
    o = torch.empty((n, m), dtype=torch.float16, device="cuda")
    tuna_b200.matmul(xd, qd, sd, cd, o, m, n, k)
    torch.cuda.synchronize()
    check_parity(o.cpu().numpy(), orc.matmul_ref(*host, m, n, k), TOL)
    w = torch.empty((m, k), dtype=torch.float16, device="cuda")
    tuna_b200.dequant(qd, sd, cd, w, m, k)
    torch.cuda.synchronize()
    assert np.array_equal(w.cpu().numpy().view(np.uint16), orc.dequant_ref(host[1], host[2], host[3], m, k).view(np.uint16))
    with pytest.raises(TypeError):
        tuna_b200.matmul(xd.float(), qd, sd, cd, o, m, n, k)
    with pytest.raises(ValueError):
        tuna_b200.matmul(xd, qd, sd, cd, o, m, n + 1, k)
    with pytest.raises(ValueError):
        tuna_b200.matmul(xd.cpu(), qd, sd, cd, o, m, n, k)


def test_reference_named_wrappers_match_the_c_abi():
    """`wrapper` / `dequantize_wrapper` with the reference's C++ linkage and argument order."""
    m, n, k = 1024, 16, 2048
    host, dev = make_case(m, n, k, 21)
    xd, qd, sd, cd = dev
    lib = _lib.load()
    out = torch.full((n, m), float("nan"), dtype=torch.float16, device="cuda")
    lib._Z7wrapperPvS_S_S_S_iiiP11CUstream_st(qd.data_ptr(), xd.data_ptr(), cd.data_ptr(), sd.data_ptr(), out.data_ptr(),
                                              m, n, k, stream_ptr())
    assert lib.tuna_last_wrapper_status() == 0
    torch.cuda.synchronize()
    check_parity(out.cpu().numpy(), orc.matmul_ref(*host, m, n, k), TOL)
    w = torch.empty((m, k), dtype=torch.float16, device="cuda")
    lib._Z18dequantize_wrapperPvS_S_S_iiP11CUstream_st(qd.data_ptr(), sd.data_ptr(), cd.data_ptr(), w.data_ptr(), m, k, stream_ptr())
    assert lib.tuna_last_wrapper_status() == 0
    torch.cuda.synchronize()
    assert np.array_equal(w.cpu().numpy().view(np.uint16), orc.dequant_ref(host[1], host[2], host[3], m, k).view(np.uint16))


def test_one_workspace_serves_alternating_shapes_and_kernels():
    """A single zero-initialised workspace, reused across shapes with different tile counts and
    across both kernels: the arrival counters of one call never land on another call's partials."""
    lib = _lib.load()
    shapes = [(4096, 16, 2048), (256, 16, 8192), (8192, 8, 512), (1024, 64, 1024), (512, 16, 4096), (4096, 16, 2048)]
    need = max(int(lib.tuna_matmul_workspace_bytes(m, n, k)) for m, n, k in shapes)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    for rep in range(2):
        for i, (m, n, k) in enumerate(shapes):
            host, dev = make_case(m, n, k, 70 + i)
            st, out, holder = run_matmul(dev, m, n, k, ws=ws)
            assert st == 0
            check_parity(out.cpu().numpy(), orc.matmul_ref(*host, m, n, k), TOL)
            assert holder.guards_intact()


def _sampled_rows_check(m, n, k, seed, code=None, cfg=None):
    """Full-size shapes: the oracle runs on a random sample of 8-row groups (plus first and last)."""
    (x, q, absmax, nf4), dev = make_case(m, n, k, seed=seed)
    if code is not None:
        dev[3] = torch.from_numpy(code).cuda()
    else:
        code = nf4
    st, out, holder = run_matmul(dev, m, n, k, cfg=cfg)
    assert st == 0, _lib.load().tuna_status_string(st)
    assert _lib.load().tuna_check_device_status(stream_ptr()) == 0, "a bounded wait ran out"
    rng = np.random.default_rng(seed)
    rows = np.unique(np.concatenate([rng.integers(0, m // 8, 24), [0, m // 8 - 1]]))
    q3 = q.reshape(m // 8, k // 8, 32)
    ref = orc.matmul_ref(x, q3[rows], absmax.reshape(-1, 8)[rows].ravel(), code, len(rows) * 8, n, k)
    got = out.cpu().numpy().reshape(n, m // 8, 8)[:, rows].reshape(n, -1)
    check_parity(got, ref, TOL)
    assert holder.guards_intact()


# BASELINE config 4: the token sweep on the Llama-70B gate+up shape, default dispatch
# (reference buckets kernel.cu:3034, 3049, 3079, 3109, 3139, 3154)
@pytest.mark.parametrize("n", [1, 64, 256, 1024, 2048])
def test_matmul_llama70b_gateup_token_sweep(n):
    _sampled_rows_check(57344, n, 8192, seed=400 + n)


# the token counts a survey of the reference's buckets suggests, at a full benchmark size
@pytest.mark.parametrize("n", [7, 8, 17, 64, 100, 128])
def test_matmul_mistral_gateup_token_counts(n):
    _sampled_rows_check(28672, n, 4096, seed=500 + n)


# BASELINE config 3: the Mixtral combined-expert shapes
@pytest.mark.parametrize("m,k", [(229376, 4096), (32768, 14336)])
def test_matmul_mixtral_combined_shapes_m16(m, k):
    _sampled_rows_check(m, 16, k, seed=m + k)


# the per-GPU shards of configs 1 and 2 at 2, 4 and 8 GPUs (column-parallel: rows / g; row-parallel: k / g)
SHARD_SHAPES = [
    (14336, 4096), (7168, 4096), (3584, 4096), (4096, 7168), (4096, 3584), (4096, 1792),
    (28672, 8192), (7168, 8192), (8192, 14336), (8192, 3584), (5120, 8192), (1280, 8192), (8192, 4096), (8192, 1024),
]


@pytest.mark.parametrize("m,k", SHARD_SHAPES)
def test_matmul_shard_shapes_m16(m, k):
    _sampled_rows_check(m, 16, k, seed=m * 3 + k)


@pytest.mark.parametrize("m,n,k", [(4096, 16, 4096), (1024, 64, 2048), (520, 5, 264)])
def test_matmul_arbitrary_codebook(m, n, k):
    """The codebook is a run-time argument (test.py:19-40 passes NF4; any 16 values must work)."""
    code = np.random.default_rng(77).standard_normal(16).astype(np.float32)
    _sampled_rows_check(m, n, k, seed=m + n, code=code)


def test_matmul_absmax_only_4_byte_aligned():
    """absmax as a slice of a larger scale buffer, off a 16-byte boundary."""
    m, n, k = 1024, 16, 1024
    host, (xd, qd, sd, cd) = make_case(m, n, k, seed=12)
    big = torch.zeros(m + 8, dtype=torch.float32, device="cuda")
    for off in (1, 3):
        view = big[off:off + m]
        view.copy_(sd)
        assert view.data_ptr() % 16 != 0
        for path in (_lib.PATH_STREAM, _lib.PATH_TSTREAM, _lib.PATH_UMMA):
            st, out, holder = run_matmul((xd, qd, view, cd), m, n, k, cfg=_lib.TunaConfig(path=path))
            assert st == 0
            check_parity(out.cpu().numpy(), orc.matmul_ref(*host, m, n, k), TOL)


def test_wrapper_on_two_streams_uses_separate_scratch():
    """The reference-named `wrapper` may run on different streams at once (as the reference's can):
    each stream gets its own scratch, so overlapping calls do not share arrival counters."""
    m, n, k = 512, 16, 8192  # few tiles, every tile split across CTAs
    lib = _lib.load()
    cases = [make_case(m, n, k, 90 + i) for i in range(2)]
    streams = [torch.cuda.Stream() for _ in range(2)]
    outs = [torch.full((n, m), float("nan"), dtype=torch.float16, device="cuda") for _ in range(2)]
    torch.cuda.synchronize()
    for rep in range(8):
        for i, s in enumerate(streams):
            xd, qd, sd, cd = cases[i][1]
            lib._Z7wrapperPvS_S_S_S_iiiP11CUstream_st(qd.data_ptr(), xd.data_ptr(), cd.data_ptr(), sd.data_ptr(),
                                                      outs[i].data_ptr(), m, n, k, s.cuda_stream)
            assert lib.tuna_last_wrapper_status() == 0
    torch.cuda.synchronize()
    for i in range(2):
        check_parity(outs[i].cpu().numpy(), orc.matmul_ref(*cases[i][0], m, n, k), TOL)


def test_a_bounded_wait_that_runs_out_is_reported_not_spun_on():
    """The time-out path of the in-kernel waits, exercised without a real failure: a one-warp kernel
    waits ~1 ms on a barrier nothing arrives at; the status word then reports the time-out once,
    and the next GEMM on the same context runs normally."""
    lib = _lib.load()
    assert lib.tuna_check_device_status(stream_ptr()) == 0
    assert lib.tuna_selftest_bounded_wait(stream_ptr()) == 0
    assert lib.tuna_check_device_status(stream_ptr()) == -8  # TUNA_ERR_DEVICE_TIMEOUT, and the word is cleared
    assert lib.tuna_check_device_status(stream_ptr()) == 0
    m, n, k = 512, 16, 1024
    host, dev = make_case(m, n, k, seed=77)
    st, out, _ = run_matmul(dev, m, n, k)
    assert st == 0
    check_parity(out.cpu().numpy(), orc.matmul_ref(*host, m, n, k), TOL)
