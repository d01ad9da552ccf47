"""CPU oracle for the FP16 x 4-bit(codebook) GEMM path of TryForefront/tuna.

TEST INFRASTRUCTURE ONLY.  This module restates, on the CPU with numpy, the
arithmetic of the reference's two exported ops and of its offline quantizer so
that the CUDA path can be checked against it.  Nothing in the shipped package
imports it; only the test-suite, the smoke check and the benchmark's
``cpu_baseline`` / reference arm do.

Parity status: the reference ships no golden vectors and no asserting tests
(test.py prints two tensors and times them), so this restatement is pinned in
two other ways: (1) against fixtures under ``tests/golden/`` that were produced
by the reference's own CUDA kernels compiled from its sources and run on a
B200 (see ``tests/golden/make_reference_fixtures.py``), and (2) against a
second, independent restatement in C (``oracle/tuna_oracle.c``).  The quantizer
is pinned by the reference's torch expression evaluated on the CPU
(``tests/golden/make_quantizer_fixture.py``).

Naming follows the reference: ``m`` = output features (rows of W), ``n`` =
tokens, ``k`` = reduction length; ``x`` is ``[n, k]``, ``W`` is ``[m, k]`` and
the output is ``[n, m]``.
"""

from __future__ import annotations

import numpy as np

# The 16-entry NF4 codebook the reference's quantizer emits (test.py:19-40).
# Index 0 is -1.0, index 7 is 0.0, index 15 is 1.0.  It is an input of the ops
# (passed per call as an fp32 tensor), not a constant of the kernels.
NF4_CODE = np.array(
    [
        -1.0,
        -0.6961928009986877,
        -0.5250730514526367,
        -0.39491748809814453,
        -0.28444138169288635,
        -0.18477343022823334,
        -0.09105003625154495,
        0.0,
        0.07958029955625534,
        0.16093020141124725,
        0.24611230194568634,
        0.33791524171829224,
        0.44070982933044434,
        0.5626170039176941,
        0.7229568362236023,
        1.0,
    ],
    dtype=np.float32,
)


# --------------------------------------------------------------------------
# Packed weight layout
# --------------------------------------------------------------------------

def pack_codes(codes: np.ndarray) -> np.ndarray:
    """4-bit codes ``[m, k]`` (uint8, values 0..15) -> packed ``[m/8, k/8, 32]``.

    Follows test.py:55-65: the matrix is cut into 8x8 tiles; inside a tile the
    64 codes are taken row-major two at a time, the first of each pair in the
    HIGH nibble.  Byte ``j`` of tile ``(mt, kt)`` therefore holds
    ``W[8*mt + j//4, 8*kt + 2*(j%4)]`` (high) and ``W[.., 8*kt + 2*(j%4) + 1]``
    (low).
    """
    codes = np.asarray(codes, dtype=np.uint8)
    m, k = codes.shape
    if m % 8 or k % 8:
        raise ValueError("m and k must be multiples of 8")
    t = codes.reshape(m // 8, 8, k // 8, 4, 2).transpose(0, 2, 1, 3, 4)
    t = t.reshape(m // 8, k // 8, 32, 2)
    return (t[..., 0] * 16 + t[..., 1]).astype(np.uint8)


def unpack_codes(q: np.ndarray, m: int, k: int) -> np.ndarray:
    """Inverse of :func:`pack_codes`; cross-checked by how the reference's
    dequant kernel reads a tile (kernel.cu:3218-3228: lane ``l`` of a 32-byte
    tile owns row ``l/4`` and columns ``2*(l%4)``, ``2*(l%4)+1``; high nibble
    first)."""
    q = np.asarray(q, dtype=np.uint8).reshape(m // 8, k // 8, 32)
    hi = q >> 4
    lo = q & 15
    t = np.stack([hi, lo], axis=-1)  # [m/8, k/8, 32, 2]
    t = t.reshape(m // 8, k // 8, 8, 4, 2).transpose(0, 2, 1, 3, 4)
    return np.ascontiguousarray(t.reshape(m, k))


# --------------------------------------------------------------------------
# Dequantisation
# --------------------------------------------------------------------------

def dequant_ref(q, absmax, code, m: int, k: int) -> np.ndarray:
    """The ``dequant`` op: ``W16[r, c] = fp16_rn(fp32(code[nib]) * fp32(absmax[r]))``.

    Follows kernel.cu:3218-3229 (fp32 multiply, one rounding to fp16).  This is
    the BIT-EXACT target for the CUDA ``tuna_dequant`` entry point.
    """
    codes = unpack_codes(q, m, k)
    code = np.asarray(code, dtype=np.float32)
    absmax = np.asarray(absmax, dtype=np.float32).reshape(m, 1)
    return (code[codes] * absmax).astype(np.float16)


def dequant_gemm_internal(q, absmax, code, m: int, k: int) -> np.ndarray:
    """What the reference's GEMM main loop multiplies by (kernel.cu:2162-2193,
    2770, 2800): codebook and absmax are first narrowed to fp16, then multiplied
    in fp16.  Differs from :func:`dequant_ref` by at most one fp16 ulp on a
    fraction of (row, code) pairs.  Kept for documentation and for bounding the
    distance between the two definitions in the tests; not a parity target.
    """
    codes = unpack_codes(q, m, k)
    c16 = np.asarray(code, dtype=np.float32).astype(np.float16)
    a16 = np.asarray(absmax, dtype=np.float32).astype(np.float16).reshape(m, 1)
    return (c16[codes] * a16).astype(np.float16)


# --------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------

def matmul_ref(x, q, absmax, code, m: int, n: int, k: int, accum: str = "f64") -> np.ndarray:
    """The ``matmul`` op restated as dequantize-then-matmul.

    ``out[n, m] = fp16_rn( sum_k x[n, k] * W16[m, k] )`` with ``W16`` from
    :func:`dequant_ref`.  The reference accumulates in fp32 (configs fix
    ``acc_mode`` 32, kernel.cu:54-55) and rounds once to fp16 (kernel.cu:2719);
    ``accum="f32"`` mirrors that with numpy's fp32 matmul, ``accum="f64"`` (the
    default) gives the order-independent value the tolerance is stated against.
    """
    x = np.asarray(x, dtype=np.float16).reshape(n, k)
    w16 = dequant_ref(q, absmax, code, m, k)
    if accum == "f32":
        acc = x.astype(np.float32) @ w16.astype(np.float32).T
    elif accum == "f64":
        acc = x.astype(np.float64) @ w16.astype(np.float64).T
    else:
        raise ValueError(accum)
    return acc.astype(np.float16)


def parity_error(out, ref):
    """The two error figures the parity tests bound.

    Returns ``(max_abs_over_max_ref, worst_mixed)`` where the second is
    ``max(|out-ref| / (|ref| + rms(ref)))``: element-wise relative error with an
    rms floor, because outputs of a zero-mean GEMM have many near-zero entries.
    """
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    diff = np.abs(out - ref)
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    denom = max(float(np.max(np.abs(ref))) if ref.size else 0.0, 1e-30)
    a = float(diff.max()) / denom if ref.size else 0.0
    b = float((diff / (np.abs(ref) + max(rms, 1e-30))).max()) if ref.size else 0.0
    return a, b


# --------------------------------------------------------------------------
# Quantizer (offline)
# --------------------------------------------------------------------------

def quantize_blockwise_dynamic_4bit(w: np.ndarray, code: np.ndarray = NF4_CODE):
    """Row-wise absmax NF4 quantizer + packer (test.py:7-68 with
    ``block_size == k`` and ``preprocess=True``, the only way the reference
    calls it, test.py:81).

    Returns ``(q[m/8,k/8,32] uint8, absmax[m] fp32, code[16] fp32)``.  Ties in
    the nearest-code search go to the lower index, as ``argmin`` does.
    """
    w = np.asarray(w)
    m, k = w.shape
    if w.size % 128:
        raise ValueError("numel must be a multiple of 128")
    wf = w.astype(np.float32)
    absmax = np.abs(wf).max(axis=1).astype(np.float32)
    # test.py:16-18,42: `absmax` is converted to fp32 before `torch.divide(temp, absmax)`, so
    # the fp16 weights are promoted and the quotient is an fp32 division (checked against torch
    # on CPU by tests/golden/make_quantizer_fixture.py).  A row of zeros divides 0 by 0: every
    # candidate distance is NaN and argmin answers index 0.
    with np.errstate(divide="ignore", invalid="ignore"):
        normalized = wf / absmax[:, None]
    codes = np.empty((m, k), dtype=np.uint8)
    rows = max(1, (512 * 1024) // k)
    code32 = np.asarray(code, dtype=np.float32)
    for r0 in range(0, m, rows):
        blk = normalized[r0 : r0 + rows]
        dist = np.abs(blk[..., None] - code32)
        dist = np.where(np.isnan(dist), np.float32(np.inf), dist)  # all-NaN rows: first index, as torch.argmin
        codes[r0 : r0 + rows] = dist.argmin(axis=-1)
    return pack_codes(codes), absmax, code32.copy()


# --------------------------------------------------------------------------
# Seeded synthetic inputs (identical bits on the CPU oracle and on the GPU)
# --------------------------------------------------------------------------

def synth_inputs(m: int, n: int, k: int, seed: int = 0, scale_lo=0.005, scale_hi=0.02):
    """Synthetic operands with the benchmark's distributions.

    ``x ~ N(0,1)`` as fp16 ``[n,k]``; uniform-random 4-bit codes packed in the
    reference layout; per-row scales drawn U[scale_lo, scale_hi], rounded to
    fp16 and stored as fp32 (the reference ABI takes fp32 scales,
    kernel.cu:3014-3015); the NF4 codebook.
    """
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, k), dtype=np.float32).astype(np.float16)
    codes = rng.integers(0, 16, size=(m, k), dtype=np.uint8)
    q = pack_codes(codes)
    absmax = (
        (scale_lo + (scale_hi - scale_lo) * rng.random(m, dtype=np.float32))
        .astype(np.float16)
        .astype(np.float32)
    )
    return x, q, absmax, NF4_CODE.copy()
