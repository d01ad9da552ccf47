"""HostPipeline (host activations and outputs, copies overlapped with the GEMMs) against the oracle."""

import numpy as np
import pytest
import torch

import tuna_b200
from oracle import tuna_oracle as orc
from tests.gpu_util import check_parity, to_dev

pytestmark = pytest.mark.gpu


def test_pipeline_matches_oracle_with_slot_reuse():
    # 7 GEMMs of two shapes through 2 staging slots: every slot is reused several times and
    # consecutive calls have different activations, so a missing ordering edge shows as a wrong result
    shapes = [(512, 16, 1024), (256, 5, 2048)]
    weights = []
    for i, (m, n, k) in enumerate(shapes):
        x, q, absmax, code = orc.synth_inputs(m, n, k, 40 + i)
        weights.append((q, absmax, code) + tuple(to_dev(q, absmax, code)))
    pipe = tuna_b200.HostPipeline("cuda", max(n * k for _, n, k in shapes), max(n * m for m, n, _ in shapes), depth=2)
    rng = np.random.default_rng(5)
    calls = []
    for j in range(7):
        m, n, k = shapes[j % 2]
        q, absmax, code, qd, sd, cd = weights[j % 2]
        xh = torch.from_numpy(rng.standard_normal((n, k)).astype(np.float16)).pin_memory()
        oh = torch.full((n, m), float("nan"), dtype=torch.float16).pin_memory()
        pipe.matmul(xh, qd, sd, cd, oh, m, n, k)
        calls.append((xh, oh, q, absmax, code, m, n, k))
    pipe.join()
    torch.cuda.synchronize()
    for xh, oh, q, absmax, code, m, n, k in calls:
        check_parity(oh.numpy(), orc.matmul_ref(xh.numpy(), q, absmax, code, m, n, k), 1e-2)


def test_pipeline_rejects_pageable_and_oversized():
    pipe = tuna_b200.HostPipeline("cuda", 64, 64, depth=2)
    d = torch.zeros(8, dtype=torch.uint8, device="cuda")
    f = torch.zeros(16, dtype=torch.float32, device="cuda")
    with pytest.raises(ValueError):
        pipe.matmul(torch.zeros((1, 8), dtype=torch.float16), d, f, f, torch.zeros((1, 8), dtype=torch.float16), 8, 1, 8)
    big = torch.zeros((16, 64), dtype=torch.float16).pin_memory()
    with pytest.raises(ValueError):
        pipe.matmul(big, d, f, f, big, 64, 16, 64)


def test_pipeline_sequence_replays_from_a_cuda_graph():
    m, n, k = 512, 16, 1024
    x, q, absmax, code = orc.synth_inputs(m, n, k, 77)
    qd, sd, cd = to_dev(q, absmax, code)
    pipe = tuna_b200.HostPipeline("cuda", n * k, n * m, depth=2)
    xs = [torch.zeros((n, k), dtype=torch.float16).pin_memory() for _ in range(3)]
    os_ = [torch.zeros((n, m), dtype=torch.float16).pin_memory() for _ in range(3)]
    ws = tuna_b200.workspace_for(m, n, k, torch.device("cuda"))
    stream = torch.cuda.Stream()

    def sequence():
        pipe.begin()
        for xh, oh in zip(xs, os_):
            pipe.matmul(xh, qd, sd, cd, oh, m, n, k, workspace=ws)
        pipe.join()

    with torch.cuda.stream(stream):
        sequence()
        stream.synchronize()
        torch.cuda.synchronize()
        pipe.reset()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            sequence()
        rng = np.random.default_rng(9)
        for rep in range(2):  # new host contents before every replay
            for xh in xs:
                xh.copy_(torch.from_numpy(rng.standard_normal((n, k)).astype(np.float16)))
            graph.replay()
            stream.synchronize()
            for xh, oh in zip(xs, os_):
                check_parity(oh.numpy(), orc.matmul_ref(xh.numpy(), q, absmax, code, m, n, k), 1e-2)
