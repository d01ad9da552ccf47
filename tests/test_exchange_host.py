"""Host-side arithmetic and argument checks of the fused GEMM + reduce entry points (no GPU needed:
every case returns before the first CUDA call)."""

import ctypes
import os
import socket

import torch.distributed as dist
import torch.multiprocessing as mp

from tuna_b200 import _lib
from tuna_b200.ops import Exchange, ReduceSequence


def _descs(shapes, flags=None, ptr=0x1000):
    d = (_lib.TunaGemmDesc * len(shapes))()
    for i, (m, n, k) in enumerate(shapes):
        d[i] = _lib.TunaGemmDesc(ptr, ptr, ptr, ptr, m, n, k, _lib.GEMM_PARTIAL if flags is None or flags[i] else 0)
    return d


def test_exchange_bytes():
    # header + two parity regions of world x m x tile_tok fp16 per partial GEMM (tile_tok from the largest n)
    assert ReduceSequence.exchange_bytes([(4096, 16, 1792)] * 3, 8) == 4096 + 2 * 8 * 3 * 4096 * 16 * 2
    assert ReduceSequence.exchange_bytes([(4096, 16, 1792), (1024, 33, 512)], 2) == 4096 + 2 * 2 * (4096 + 1024) * 64 * 2
    # ordinary GEMMs of the launch take no room
    assert ReduceSequence.exchange_bytes([(4096, 16, 1792), (28672, 16, 4096)], 4, [True, False]) == 4096 + 2 * 4 * 4096 * 16 * 2
    # more than 64 GEMMs run as several launches that reuse the regions: the largest launch decides
    assert ReduceSequence.exchange_bytes([(256, 16, 256)] * 100, 2) == 4096 + 2 * 2 * 64 * 256 * 16 * 2
    lib = _lib.load()
    assert lib.tuna_exchange_bytes(_descs([(256, 16, 256)]), 1, 9) == 0  # more ranks than TUNA_MAX_PEERS
    assert lib.tuna_exchange_bytes(_descs([(256, 16, 256)]), 0, 2) == 0


def _exchange(world=2, rank=0, nbytes=1 << 20, ptr=0x10000):
    ex = _lib.TunaExchange()
    ex.rank, ex.world, ex.bytes = rank, world, nbytes
    for j in range(min(world, _lib.MAX_PEERS)):
        ex.buffer[j] = ptr + j * (1 << 24)
    return ex


def test_reduce_sequence_argument_checks():
    lib = _lib.load()
    code = ws = 0x2000
    good = _descs([(256, 16, 256)])
    call = lambda d, n, ex: lib.tuna_matmul_sequence_reduce(d, n, code, ws, 1 << 20, ctypes.byref(ex) if ex is not None else None, None)
    assert call(good, 1, None) == -1
    assert call(good, 0, _exchange()) == -2
    assert call(good, 1, _exchange(world=9)) == -5
    assert call(good, 1, _exchange(world=2, rank=2)) == -5
    ex = _exchange()
    ex.buffer[1] = 0
    assert call(good, 1, ex) == -1
    assert call(good, 1, _exchange(ptr=0x10010)) == -3           # buffers are 256-byte aligned
    assert call(_descs([(256, 0, 256)]), 1, _exchange()) == -2   # every rank runs every GEMM: no empty entries
    assert call(_descs([(256, 65, 256)]), 1, _exchange()) == -9  # one pass of the streaming kernel: at most 64 tokens
    assert call(_descs([(250, 16, 256)]), 1, _exchange()) == -2
    assert call(good, 1, _exchange(nbytes=4096 + 1024)) == -4    # exchange buffers too small for the call


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _exchange_worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # rank 1 asks for a buffer smaller than the header: its creation fails whatever the machine
        try:
            Exchange((1 << 20) if rank == 0 else 16, "cuda:0", group=dist.group.WORLD)
            ret[rank] = "created"
        except RuntimeError as exc:
            ret[rank] = str(exc)
    finally:
        dist.destroy_process_group()


def test_exchange_setup_fails_on_every_rank_together():
    """One rank cannot create its buffer: no rank hangs in a collective, all raise."""
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_exchange_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert set(ret.keys()) == {0, 1}
    assert all("could not allocate" in ret[r] for r in (0, 1)), dict(ret)
