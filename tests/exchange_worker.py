"""One rank of the two-GPU test of `ReduceSequence` (launched by tests/test_gpu_exchange.py under
torch.distributed.run; gloo carries the IPC handles and the comparison between the ranks)."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

import tuna_b200
from oracle import tuna_oracle as orc
from tuna_b200 import sharding


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("gloo")
    dev = torch.device("cuda", torch.cuda.current_device())
    shapes = [(1024, 16, 4096), (512, 5, 2048), (4096, 16, 1792 * world), (256, 33, 1024)]
    gemms, refs = [], []
    code = None
    for i, (m, n, k) in enumerate(shapes):
        x, q, absmax, codebook = orc.synth_inputs(m, n, k, 700 + i)  # the same full problem on every rank
        refs.append(orc.matmul_ref(x, q, absmax, codebook, m, n, k))
        qd = torch.from_numpy(q).to(dev)
        q_shard, ks = sharding.shard_k(qd, m, k, world, rank)
        x_shard = torch.from_numpy(np.ascontiguousarray(x[:, rank * ks:(rank + 1) * ks])).to(dev)
        o = torch.full((n, m), float("nan"), dtype=torch.float16, device=dev)
        gemms.append((x_shard, q_shard.reshape(-1), torch.from_numpy(absmax).to(dev), o, m, n, ks))
        code = torch.from_numpy(codebook).to(dev)
    # plus one ordinary (not K-split) GEMM in the same launch: every rank computes it in full
    m, n, k = 512, 16, 1024
    x, q, absmax, codebook = orc.synth_inputs(m, n, k, 799)
    refs.append(orc.matmul_ref(x, q, absmax, codebook, m, n, k))
    gemms.append((torch.from_numpy(x).to(dev), torch.from_numpy(q).to(dev), torch.from_numpy(absmax).to(dev),
                  torch.full((n, m), float("nan"), dtype=torch.float16, device=dev), m, n, k))
    partial = [True] * len(shapes) + [False]
    ex = tuna_b200.Exchange(tuna_b200.ReduceSequence.exchange_bytes([(g[4], g[5], g[6]) for g in gemms], world, partial), dev,
                            group=dist.group.WORLD)
    seq = tuna_b200.ReduceSequence(gemms, code, ex, partial=partial)
    lib = tuna_b200._lib.load()
    for rep in range(4):
        for g in gemms:
            g[3].fill_(float("nan"))
        seq.run()
        torch.cuda.synchronize()
        status = lib.tuna_check_device_status(torch.cuda.current_stream().cuda_stream)
        assert status == 0, f"rank {rank}: device status {status}"
        for g, ref in zip(gemms, refs):
            got = g[3].cpu().numpy()
            err = np.abs(got.astype(np.float32) - ref).max() / np.abs(ref).max()
            assert err <= 1e-2, f"rank {rank} rep {rep}: max-norm error {err}"
            theirs = [None] * world
            dist.all_gather_object(theirs, got.view(np.uint16).tobytes())
            assert all(t == theirs[0] for t in theirs), f"rep {rep}: the ranks' sums differ"
    # a captured step, replayed: the exchange number advances on the device
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            seq.run()
        dist.barrier()
        for _ in range(5):
            graph.replay()
        stream.synchronize()
    assert lib.tuna_check_device_status(stream.cuda_stream) == 0
    for g, ref in zip(gemms, refs):
        got = g[3].cpu().numpy()
        assert np.abs(got.astype(np.float32) - ref).max() / np.abs(ref).max() <= 1e-2
    # the tensor-parallel layer class with the fused sum instead of its all-reduce
    m, n, k = 1024, 16, 4096
    x, q, absmax, codebook = orc.synth_inputs(m, n, k, 900)
    layer = sharding.RowParallelLinear(torch.from_numpy(q).to(dev), torch.from_numpy(absmax).to(dev), code, m, k, exchange=ex)
    xs = layer.slice_input(torch.from_numpy(x).to(dev))
    out = torch.full((n, m), float("nan"), dtype=torch.float16, device=dev)
    for _ in range(2):
        layer.forward(xs, out)
    torch.cuda.synchronize()
    ref = orc.matmul_ref(x, q, absmax, codebook, m, n, k)
    assert np.abs(out.cpu().numpy().astype(np.float32) - ref).max() / np.abs(ref).max() <= 1e-2
    dist.barrier()
    ex.close()
    dist.barrier()
    if rank == 0:
        print("exchange worker ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
