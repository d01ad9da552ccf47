"""The device quantizer against the oracle (bit-exact) and the torch-CPU golden fixture."""

from pathlib import Path

import numpy as np
import pytest
import torch

import tuna_b200
from oracle import tuna_oracle as orc
from tests.gpu_util import check_parity

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden"


def _quantize_gpu(w: np.ndarray):
    q, (absmax, code) = tuna_b200.quantize(torch.from_numpy(w).cuda())
    torch.cuda.synchronize()
    return q.cpu().numpy(), absmax.cpu().numpy(), code.cpu().numpy()


def test_fixture_from_the_reference_expression():
    d = np.load(GOLDEN / "quantizer_torch_cpu.npz")
    q, absmax, _ = _quantize_gpu(d["w_bits"].view(np.float16).copy())
    assert np.array_equal(absmax, d["absmax"])
    assert np.array_equal(q, d["q"])


@pytest.mark.parametrize("m,k", [(16, 8), (64, 256), (136, 80), (1024, 4096), (4096, 1000)])
def test_bit_exact_against_the_oracle(m, k):
    rng = np.random.default_rng(m * 131 + k)
    w = (rng.standard_normal((m, k)) * 0.05).astype(np.float16)
    w[m // 2] = 0
    q, absmax, _ = _quantize_gpu(w)
    q_ref, a_ref, _ = orc.quantize_blockwise_dynamic_4bit(w)
    assert np.array_equal(absmax, a_ref)
    assert np.array_equal(q, q_ref)


def test_quantize_then_matmul_matches_the_fp16_product():
    # the reference's own smoke check (test.py:81-88): quantized GEMM next to x @ w.T
    m, n, k = 2048, 16, 4096
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn((n, k), device="cuda", generator=g).half() * 0.1
    w = torch.randn((m, k), device="cuda", generator=g).half() * 0.05
    q, (absmax, code) = tuna_b200.quantize(w)
    out = torch.empty((n, m), dtype=torch.float16, device="cuda")
    tuna_b200.matmul(x, q, absmax, code, out, m, n, k)
    torch.cuda.synchronize()
    # exact check against the oracle on the quantized weights ...
    ref = orc.matmul_ref(x.cpu().numpy(), q.cpu().numpy(), absmax.cpu().numpy(), code.cpu().numpy(), m, n, k)
    check_parity(out.cpu().numpy(), ref, 1e-2)
    # ... and the quantization error itself stays at the 4-bit level
    dense = (x.float() @ w.float().t()).cpu().numpy()
    rel = np.abs(out.cpu().numpy().astype(np.float32) - dense).max() / np.abs(dense).max()
    assert rel < 0.15


def test_rejects_bad_arguments():
    with pytest.raises(ValueError):
        tuna_b200.quantize(torch.zeros((8, 8), dtype=torch.float32, device="cuda"))
    with pytest.raises(tuna_b200.TunaError):
        tuna_b200.quantize(torch.zeros((12, 8), dtype=torch.float16, device="cuda"))
