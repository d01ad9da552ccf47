"""One process driving two GPUs: every kernel family must run on the second device after the first
(the opt-in to large dynamic shared memory, the status word and the scratch are per device)."""

import pytest
import torch

from oracle import tuna_oracle as orc
from tuna_b200 import _lib
from tests.gpu_util import check_parity, make_case, run_matmul, stream_ptr

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]


@pytest.mark.parametrize("n", [16, 64, 300])  # weight-streaming tcgen05 kernel, its 64-token tile, the TMA-staged kernel
def test_same_process_second_device(n):
    m, k = 1024, 2048
    for dev in (0, 1, 0):
        with torch.cuda.device(dev):
            host, tensors = make_case(m, n, k, 900 + dev)
            st, out, holder = run_matmul(tensors, m, n, k)
            assert st == 0, _lib.load().tuna_status_string(st)
            assert out.device.index == dev
            check_parity(out.cpu().numpy(), orc.matmul_ref(*host, m, n, k), 1e-2)
            assert holder.guards_intact()
            assert _lib.load().tuna_check_device_status(stream_ptr()) == 0


def test_same_process_second_device_noalloc_and_dequant():
    lib = _lib.load()
    m, n, k = 512, 16, 1024
    for dev in (0, 1):
        with torch.cuda.device(dev):
            host, (xd, qd, sd, cd) = make_case(m, n, k, 910 + dev)
            out = torch.full((n, m), float("nan"), dtype=torch.float16, device="cuda")
            assert lib.tuna_matmul_noalloc(qd.data_ptr(), xd.data_ptr(), cd.data_ptr(), sd.data_ptr(), out.data_ptr(), m, n, k, stream_ptr()) == 0
            w = torch.empty((m, k), dtype=torch.float16, device="cuda")
            assert lib.tuna_dequant(qd.data_ptr(), sd.data_ptr(), cd.data_ptr(), w.data_ptr(), m, k, stream_ptr()) == 0
            torch.cuda.synchronize()
            check_parity(out.cpu().numpy(), orc.matmul_ref(*host, m, n, k), 1e-2)
            x, q, absmax, code = host
            assert (w.cpu().numpy().view("uint16") == orc.dequant_ref(q, absmax, code, m, k).view("uint16")).all()
