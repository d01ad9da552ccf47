"""`HostSequence`: a list of GEMMs whose activations and outputs live in pinned host memory."""

import numpy as np
import pytest
import torch

import tuna_b200
from oracle import tuna_oracle as orc
from tests.gpu_util import check_parity

pytestmark = pytest.mark.gpu

SHAPES = [(1024, 16, 2048), (512, 7, 4096), (256, 16, 1024), (2048, 3, 512), (512, 16, 512), (128, 16, 256), (768, 9, 1024)]


def _problem(shapes, seed0, slab_outputs):
    """Device weights, pinned host activations and outputs (outputs either one tensor each or views of
    one pinned slab per pool, back to back in GEMM order), oracle results."""
    gemms, refs, pools = [], [], [i % 2 for i in range(len(shapes))]
    slabs = {pid: torch.empty(sum(n * m for (m, n, k), p in zip(shapes, pools) if p == pid), dtype=torch.float16).pin_memory() for pid in (0, 1)}
    used = {0: 0, 1: 0}
    code = None
    for i, (m, n, k) in enumerate(shapes):
        x, q, absmax, codebook = orc.synth_inputs(m, n, k, seed0 + i)
        refs.append(orc.matmul_ref(x, q, absmax, codebook, m, n, k))
        xh = torch.from_numpy(x).pin_memory()
        if slab_outputs:
            oh = slabs[pools[i]][used[pools[i]]:used[pools[i]] + n * m].view(n, m)
            used[pools[i]] += n * m
        else:
            oh = torch.empty((n, m), dtype=torch.float16).pin_memory()
        oh.fill_(float("nan"))
        gemms.append((xh, torch.from_numpy(q).cuda(), torch.from_numpy(absmax).cuda(), oh, m, n, k))
        code = torch.from_numpy(codebook).cuda()
    return gemms, refs, pools, code


@pytest.mark.parametrize("slab_outputs", [False, True])
@pytest.mark.parametrize("groups", [1, 3])
def test_host_sequence_matches_the_oracle(groups, slab_outputs):
    gemms, refs, pools, code = _problem(SHAPES, 600, slab_outputs)
    hs = tuna_b200.HostSequence(gemms, code, groups=groups, pool_ids=pools)
    if slab_outputs:  # neighbouring outputs of a pool leave as one copy
        assert sum(len(g["copies_out"]) for g in hs._groups) < len(gemms)
    for rep in range(2):
        for g in gemms:
            g[3].fill_(float("nan"))
        hs.run()
        torch.cuda.synchronize()
        for g, ref in zip(gemms, refs):
            check_parity(g[3].numpy(), ref, 1e-2)


def test_host_sequence_after_group_sees_one_tensor_per_pool():
    gemms, refs, pools, code = _problem(SHAPES, 620, True)
    seen = []

    def hook(p):
        seen.append({pid: t.numel() for pid, t in p.items()})
        if 1 in p:
            p[1].mul_(2)  # stands in for a collective on the pool's outputs

    hs = tuna_b200.HostSequence(gemms, code, groups=2, after_group=hook, pool_ids=pools)
    hs.run()
    torch.cuda.synchronize()
    assert len(seen) == 2 and all(set(s) <= {0, 1} for s in seen)
    for g, ref, pid in zip(gemms, refs, pools):
        check_parity(g[3].numpy(), ref * (2 if pid == 1 else 1), 1e-2)


def test_host_sequence_with_a_one_rank_exchange_and_graph_replay():
    """The groups as fused-reduce launches (an exchange of one rank: the sum of one slab), captured and replayed."""
    gemms, refs, pools, code = _problem(SHAPES, 640, True)
    partial = [p == 1 for p in pools]
    need = tuna_b200.ReduceSequence.exchange_bytes([(m, n, k) for m, n, k in SHAPES], 1, partial)
    ex = tuna_b200.Exchange(need, "cuda")
    hs = tuna_b200.HostSequence(gemms, code, groups=2, pool_ids=pools, exchange=ex, partial=partial)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        hs.run()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            hs.run()
        for g in gemms:
            g[3].fill_(float("nan"))
        for _ in range(3):
            graph.replay()
        stream.synchronize()
    assert tuna_b200._lib.load().tuna_check_device_status(stream.cuda_stream) == 0
    for g, ref in zip(gemms, refs):
        check_parity(g[3].numpy(), ref, 1e-2)
    ex.close()


def test_host_sequence_rejects_pageable_memory():
    gemms, _, pools, code = _problem(SHAPES[:2], 660, False)
    xh, q, s, oh, m, n, k = gemms[0]
    gemms[0] = (xh.clone(), q, s, oh, m, n, k)  # a pageable copy
    with pytest.raises(ValueError):
        tuna_b200.HostSequence(gemms, code)
