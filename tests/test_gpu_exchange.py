"""K-split GEMMs fused with the sum of their partial outputs over the GPUs (`tuna_matmul_sequence_reduce`).

One GPU: an exchange of one rank runs the whole path (slabs, parity regions, flags, reduce kernel)
and must give the bits of the ordinary sequence launch.  Two GPUs: two processes (gloo carries the
IPC handles), each with its K slice of one seeded weight set; every rank's result must equal the
oracle on the full K within the GEMM tolerance and the two ranks' results must be the same bits.
The reduce kernel's bounded wait is made to run out on ONE GPU (a second rank that does not exist:
a flag that nothing sets); no test makes a wait run out across GPUs.
"""

import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import tuna_b200
from oracle import tuna_oracle as orc
from tests.gpu_util import check_parity, make_case

pytestmark = pytest.mark.gpu


def _gemms(shapes, seed0):
    hosts, gemms, refs = [], [], []
    for i, (m, n, k) in enumerate(shapes):
        host, dev = make_case(m, n, k, seed0 + i)
        xd, qd, sd, cd = dev
        o = torch.full((n, m), float("nan"), dtype=torch.float16, device="cuda")
        gemms.append((xd, qd, sd, o, m, n, k))
        hosts.append(host)
        refs.append(orc.matmul_ref(*host, m, n, k))
    return hosts, gemms, refs, cd


def test_single_rank_exchange_gives_the_bits_of_the_plain_sequence():
    shapes = [(1024, 16, 2048), (512, 7, 4096), (2048, 1, 1024), (256, 16, 8192)]
    _, gemms, refs, code = _gemms(shapes, 300)
    plain_out = [torch.empty_like(g[3]) for g in gemms]
    plain = tuna_b200.MatmulSequence([(g[0], g[1], g[2], po, g[4], g[5], g[6]) for g, po in zip(gemms, plain_out)], code)
    plain.run()
    partial = [True, False, True, True]  # the second GEMM is an ordinary one that shares the launch
    ex = tuna_b200.Exchange(tuna_b200.ReduceSequence.exchange_bytes([(m, n, k) for m, n, k in shapes], 1, partial), "cuda")
    seq = tuna_b200.ReduceSequence(gemms, code, ex, partial=partial)
    for rep in range(3):  # both parity regions, and the first one again
        for g in gemms:
            g[3].fill_(float("nan"))
        seq.run()
        torch.cuda.synchronize()
        assert tuna_b200._lib.load().tuna_check_device_status(torch.cuda.current_stream().cuda_stream) == 0
        for g, po, ref in zip(gemms, plain_out, refs):
            got = g[3].cpu().numpy()
            assert np.array_equal(got.view(np.uint16), po.cpu().numpy().view(np.uint16))
            check_parity(got, ref, 1e-2)
    ex.close()


def test_single_rank_exchange_larger_tiles_many_gemms_and_graph_replay():
    shapes = [(256, 40, 512)] + [(128, 16, 256)] * 70  # 64-token tiles in the first launch, two launches
    _, gemms, refs, code = _gemms(shapes, 400)
    ex = tuna_b200.Exchange(tuna_b200.ReduceSequence.exchange_bytes([(m, n, k) for m, n, k in shapes], 1), "cuda")
    seq = tuna_b200.ReduceSequence(gemms, code, ex)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        seq.run()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            seq.run()
        for g in gemms:
            g[3].fill_(float("nan"))
        for _ in range(3):  # the exchange number advances on the device: replays alternate regions
            graph.replay()
        stream.synchronize()
    for g, ref in zip(gemms, refs):
        check_parity(g[3].cpu().numpy(), ref, 1e-2)
    ex.close()


def test_exchange_validation():
    lib = tuna_b200._lib.load()
    shapes = [(256, 16, 512)]
    _, gemms, _, code = _gemms(shapes, 500)
    need = tuna_b200.ReduceSequence.exchange_bytes(shapes, 1)
    assert need == 4096 + 2 * 256 * 16 * 2
    ex = tuna_b200.Exchange(need, "cuda")
    with pytest.raises(ValueError):
        tuna_b200.ReduceSequence([(g[0], g[1], g[2], g[3], g[4], 0, g[6]) for g in gemms], code, ex)
    small = tuna_b200.Exchange(4096 + 512, "cuda")
    with pytest.raises(ValueError):
        tuna_b200.ReduceSequence(gemms, code, small)
    small.close()
    ex.close()
    assert lib.tuna_exchange_bytes(None, 1, 2) == 0


def test_a_peer_that_never_signals_ends_in_a_status_not_a_hang():
    """Rank 0 of a two-rank exchange whose rank 1 does not exist (its buffer is a second local one that
    nobody signals): the reduce kernel's wait runs out after about a second, the device status word
    reports it, the outputs stay untouched and the device keeps working."""
    import ctypes
    import time

    lib = tuna_b200._lib.load()
    shapes = [(256, 16, 512)]
    _, gemms, refs, code = _gemms(shapes, 520)
    need = tuna_b200.ReduceSequence.exchange_bytes(shapes, 2)
    mine, silent = tuna_b200.Exchange(need, "cuda"), tuna_b200.Exchange(need, "cuda")

    class TwoRanks:  # the exchange as rank 0 of 2 sees it
        rank, world, nbytes = 0, 2, need
        struct = tuna_b200._lib.TunaExchange()

    TwoRanks.struct.rank, TwoRanks.struct.world, TwoRanks.struct.bytes = 0, 2, need
    TwoRanks.struct.buffer[0] = mine.struct.buffer[0]
    TwoRanks.struct.buffer[1] = silent.struct.buffer[0]
    seq = tuna_b200.ReduceSequence(gemms, code, TwoRanks)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.tuna_check_device_status(stream) == 0
    t0 = time.time()
    seq.run()
    torch.cuda.synchronize()
    assert time.time() - t0 < 20.0
    assert lib.tuna_check_device_status(stream) == -8   # TUNA_ERR_DEVICE_TIMEOUT, and the word is cleared
    assert lib.tuna_check_device_status(stream) == 0
    assert bool(torch.isnan(gemms[0][3]).all())           # nothing was summed
    # the device and the library are still usable: the same GEMM through the plain sequence
    tuna_b200.MatmulSequence(gemms, code).run()
    torch.cuda.synchronize()
    check_parity(gemms[0][3].cpu().numpy(), refs[0], 1e-2)
    mine.close()
    silent.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_sum_their_k_slices():
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, PYTHONPATH=str(root), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", str(root / "tests" / "exchange_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "exchange worker ok" in r.stdout
