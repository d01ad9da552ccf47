"""tuna_matmul_batched: several GEMMs of one shape in one call, against the oracle per matrix."""

import numpy as np
import pytest
import torch

import tuna_b200
from oracle import tuna_oracle as orc
from tests.gpu_util import check_parity

pytestmark = pytest.mark.gpu


def _case(batch, m, n, k, seed, shared_x):
    per = [orc.synth_inputs(m, n, k, seed + b) for b in range(batch)]
    code = per[0][3]
    q = np.stack([p[1] for p in per])
    s = np.stack([p[2] for p in per])
    x = per[0][0] if shared_x else np.stack([p[0] for p in per])
    return per, x, q, s, code


@pytest.mark.parametrize("shared_x", [False, True])
@pytest.mark.parametrize("batch,m,n,k", [(3, 512, 16, 1024), (8, 256, 16, 4096), (2, 1032, 5, 520), (5, 64, 1, 64), (2, 512, 40, 1024)])
def test_batched_matches_oracle_per_matrix(batch, m, n, k, shared_x):
    per, x, q, s, code = _case(batch, m, n, k, 300 + batch, shared_x)
    xd, qd, sd, cd = (torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (x, q, s, code))
    out = torch.full((batch, n, m), float("nan"), dtype=torch.float16, device="cuda")
    tuna_b200.matmul_batched(xd, qd, sd, cd, out, m, n, k)
    torch.cuda.synchronize()
    assert tuna_b200._lib.load().tuna_check_device_status(torch.cuda.current_stream().cuda_stream) == 0
    o = out.cpu().numpy()
    for b in range(batch):
        xb = x if shared_x else x[b]
        check_parity(o[b], orc.matmul_ref(xb, per[b][1], per[b][2], code, m, n, k), 1e-2)


def test_batched_equals_separate_calls_bit_for_bit_and_is_repeatable():
    batch, m, n, k = 8, 4096, 16, 2048
    per, x, q, s, code = _case(batch, m, n, k, 900, False)
    xd, qd, sd, cd = (torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in (x, q, s, code))
    out = torch.empty((batch, n, m), dtype=torch.float16, device="cuda")
    tuna_b200.matmul_batched(xd, qd, sd, cd, out, m, n, k)
    first = out.clone()
    for _ in range(3):
        out.fill_(float("nan"))
        tuna_b200.matmul_batched(xd, qd, sd, cd, out, m, n, k)
        assert torch.equal(out, first)
    torch.cuda.synchronize()
    o = first.cpu().numpy()
    for b in range(batch):
        check_parity(o[b], orc.matmul_ref(x[b], per[b][1], per[b][2], code, m, n, k), 1e-2)
