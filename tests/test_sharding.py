"""N-split / K-split of the packed format, and the tensor-parallel layers on two CPU ranks
(gloo) with the oracle standing in for the CUDA GEMM."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import tuna_oracle as orc
from tuna_b200 import sharding


def test_column_shard_is_a_row_slice():
    m, k, world = 64, 48, 4
    _, q, absmax, code = orc.synth_inputs(m, 1, k, 3)
    codes = orc.unpack_codes(q, m, k)
    for rank in range(world):
        qs, ss, ms = sharding.shard_columns(torch.from_numpy(q), torch.from_numpy(absmax), m, k, world, rank)
        assert ms == m // world
        assert np.array_equal(orc.unpack_codes(qs.numpy(), ms, k), codes[rank * ms:(rank + 1) * ms])
        assert np.array_equal(ss.numpy(), absmax[rank * ms:(rank + 1) * ms])


def test_k_shard_is_a_column_slice_after_repack():
    m, k, world = 32, 128, 4
    _, q, absmax, code = orc.synth_inputs(m, 1, k, 4)
    codes = orc.unpack_codes(q, m, k)
    for rank in range(world):
        qs, ks = sharding.shard_k(torch.from_numpy(q), m, k, world, rank)
        assert ks == k // world and qs.is_contiguous()
        assert np.array_equal(orc.unpack_codes(qs.numpy(), m, ks), codes[:, rank * ks:(rank + 1) * ks])


def test_uneven_split_is_refused():
    _, q, absmax, _ = orc.synth_inputs(24, 1, 64, 0)
    with pytest.raises(ValueError):
        sharding.shard_columns(torch.from_numpy(q), torch.from_numpy(absmax), 24, 64, 2, 0)  # 12 rows: not % 8
    with pytest.raises(ValueError):
        sharding.shard_k(torch.from_numpy(q), 24, 64, 3, 0)


def _oracle_matmul(x, q, s, c, o, m, n, k):
    o.copy_(torch.from_numpy(orc.matmul_ref(x.numpy(), q.numpy(), s.numpy(), c.numpy(), m, n, k)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k, q, absmax, code, x, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        col = sharding.ColumnParallelLinear(q, absmax, code, m, k, matmul_fn=_oracle_matmul)
        out_col = col.forward(x)
        row = sharding.RowParallelLinear(q, absmax, code, m, k, matmul_fn=_oracle_matmul, reduce_dtype=torch.float32)
        out_row = row.forward(row.slice_input(x))
        if rank == 0:
            ret["col"] = out_col.numpy().copy()
            ret["row"] = out_row.numpy().copy()
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_layers_two_gloo_ranks():
    m, n, k, world = 64, 5, 128, 2
    x, q, absmax, code = orc.synth_inputs(m, n, k, 21)
    ref = orc.matmul_ref(x, q, absmax, code, m, n, k)
    mgr = mp.Manager()
    ret = mgr.dict()
    args = (world, _free_port(), m, n, k, torch.from_numpy(q), torch.from_numpy(absmax),
            torch.from_numpy(code), torch.from_numpy(x), ret)
    mp.spawn(_worker, args=args, nprocs=world, join=True)
    # column-parallel: every output column is computed by exactly one rank -> identical to the oracle
    assert np.array_equal(ret["col"].view(np.uint16), ref.view(np.uint16))
    # row-parallel: two fp16-rounded partials summed in fp32, rounded again
    a, b = orc.parity_error(ret["row"], ref)
    assert a < 2e-3 and b < 4e-3
