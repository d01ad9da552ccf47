"""Evolutionary tuner for the shape -> launch-configuration table.

The reference ships a table tuned by an evolutionary search on an RTX A6000
(README.md:5,32) but not the tuner itself; its `make_configs.py` only renders
`param_map.json` into `configs.cu` (make_configs.py:85-132).  This module is the
missing half for Blackwell: it searches the launch parameters of
`tuna_config` (include/tuna_b200.h) on the local GPU and rewrites
`param_map.json` in the same `"{m}_{n}_{k}"` key format.

    python -m tuna_b200.tuner --shapes 28672x4096 4096x14336 --tokens 16 [--generations 6]

Fitness is the median time of the GEMM over weight buffers that rotate through
more than twice the L2 capacity, measured with CUDA events around CUDA-graph
replays (so host launch overhead is not part of it).  The search is seeded and
resumable: the population and every measurement are written to a state file
after each generation.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import random
import statistics
from pathlib import Path

from . import _lib, make_configs

L2_BYTES = 126 << 20

# the search space, per kernel family
STREAM_SPACE = {
    "rows_per_warp": (1, 2),
    "warps_m": (1, 2, 4, 8, 16),
    "warps_k": (1, 2, 4, 8, 16),
    "k_steps": (4, 8, 16, 32, 64),
}
TSTREAM_SPACE = {
    "row_blocks": (1, 2, 4),
    "k_steps": (4, 8),
}
# The TMA-staged kernel is measured with its own defaults only (0 = default): two searches over
# its stage counts, dequant warps and accumulator split ended in a launch failure on 57344x8192
# (64- and 256-token tiles) with combinations no GPU test exercises, so the tuner does not explore them.
UMMA_SPACE = {
    "row_blocks": (0,),
    "stages_w": (0,),
    "stages_x": (0,),
    "dequant_warps": (0,),
    "k_accs": (0,),
}


PATH_IDS = {"stream": _lib.PATH_STREAM, "umma": _lib.PATH_UMMA, "tstream": _lib.PATH_TSTREAM}


def space_for(path: str) -> dict:
    return {"stream": STREAM_SPACE, "tstream": TSTREAM_SPACE, "umma": UMMA_SPACE}[path]


def candidate_paths(n: int) -> tuple:
    """Kernel families worth measuring for a token count: the path is part of what is tuned
    (the reference's table has one kernel and tunes its tile per bucket, kernel.cu:3022-3155)."""
    if n <= 32:
        return ("tstream", "stream")
    return ("tstream", "umma")  # above 64 tokens the streaming kernel runs passes of 128 tokens


def tile_tok_for(path: str, n: int) -> int:
    if path == "stream":
        return 8 if n <= 8 else 16 if n <= 16 else 32
    if path == "tstream":
        return 16 if n <= 16 else 32 if n <= 32 else 64 if n <= 64 else 128
    return min(make_configs.token_bucket(n), 256)


def random_genome(rng: random.Random, path: str) -> dict:
    return {k: rng.choice(v) for k, v in space_for(path).items()}


def mutate(rng: random.Random, g: dict, path: str, rate: float = 0.3) -> dict:
    out = dict(g)
    for k, v in space_for(path).items():
        if rng.random() < rate:
            out[k] = rng.choice(v)
    return out


def crossover(rng: random.Random, a: dict, b: dict) -> dict:
    return {k: (a if rng.random() < 0.5 else b)[k] for k in a}


def to_config(path: str, tile_tok: int, genome: dict) -> _lib.TunaConfig:
    cfg = _lib.TunaConfig(path=PATH_IDS[path], tile_tok=tile_tok)
    for k, v in genome.items():
        setattr(cfg, k, int(v))
    return cfg


def is_valid(lib, m: int, n: int, k: int, cfg: _lib.TunaConfig) -> bool:
    """Host-side validation only: the launcher rejects inconsistent configurations before any
    CUDA call when given null device pointers."""
    buf = ctypes.create_string_buffer(128)
    p = ctypes.c_void_p((ctypes.addressof(buf) + 63) & ~63)
    st = lib.tuna_matmul_cfg(p, p, p, p, p, m, n, k, p, 16, None, ctypes.byref(cfg))
    return st == -4  # everything fine except the (deliberately tiny) workspace


class Bench:
    """Times one (m, n, k) GEMM for arbitrary configurations on the current device."""

    def __init__(self, m: int, n: int, k: int, seed: int = 0):
        import torch

        self.torch = torch
        self.m, self.n, self.k = m, n, k
        dev = torch.device("cuda")
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)
        nbuf = max(2, -(-(2 * L2_BYTES + 1) // (m * k // 2)))
        self.qs = [torch.randint(0, 256, (m * k // 2,), dtype=torch.uint8, device=dev, generator=gen) for _ in range(nbuf)]
        self.x = torch.randn((n, k), device=dev, generator=gen).half()
        self.s = (0.005 + 0.015 * torch.rand(m, device=dev, generator=gen)).half().float()
        from .codebooks import nf4_tensor

        self.c = nf4_tensor(dev)
        self.o = torch.empty((n, m), dtype=torch.float16, device=dev)
        self.ws = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
        self.stream = torch.cuda.Stream()
        self.lib = _lib.load()

    def _call(self, cfg, i):
        q = self.qs[i % len(self.qs)]
        return self.lib.tuna_matmul_cfg(q.data_ptr(), self.x.data_ptr(), self.c.data_ptr(), self.s.data_ptr(),
                                        self.o.data_ptr(), self.m, self.n, self.k, self.ws.data_ptr(),
                                        self.ws.numel(), self.stream.cuda_stream, ctypes.byref(cfg))

    def time_us(self, cfg, reps: int = 5) -> float | None:
        torch = self.torch
        nb = len(self.qs)
        with torch.cuda.stream(self.stream):
            for i in range(nb):
                if self._call(cfg, i) != 0:
                    return None
            self.stream.synchronize()
            if self.lib.tuna_check_device_status(self.stream.cuda_stream) != 0:
                return None
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.stream):
                for i in range(nb):
                    self._call(cfg, i)
            times = []
            for _ in range(reps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self.stream)
                graph.replay()
                e1.record(self.stream)
                self.stream.synchronize()
                times.append(e0.elapsed_time(e1) * 1e3 / nb)
        return statistics.median(times)


def tune_shape(m: int, n: int, k: int, path: str, generations: int, population: int, seed: int,
               state_path: Path, log=print, bench=None) -> tuple[dict, float]:
    lib = _lib.load()
    rng = random.Random(seed * 1000003 + m * 31 + k * 17 + n)
    tile_tok = tile_tok_for(path, n)
    key = f"{m}_{make_configs.token_bucket(n)}_{k}"
    state = json.loads(state_path.read_text()) if state_path.exists() else {}
    entry = state.setdefault(f"{key}/{path}", {"measured": {}, "generation": 0, "population": []})
    bench = bench or Bench(m, n, k, seed)
    space = space_for(path)
    size = 1
    for v in space.values():
        size *= len(v)
    enumerate_all = size <= population  # a space this small is simply enumerated
    def fitness(g: dict) -> float:
        gk = json.dumps(g, sort_keys=True)
        if gk not in entry["measured"]:
            cfg = to_config(path, tile_tok, g)
            us = bench.time_us(cfg) if is_valid(lib, m, n, k, cfg) else None
            entry["measured"][gk] = us if us is not None else float("inf")
        return entry["measured"][gk]

    if enumerate_all:
        import itertools

        pop = [dict(zip(space, vals)) for vals in itertools.product(*space.values())]
        pop.sort(key=fitness)
        entry["population"], entry["generation"] = pop, generations
        state_path.write_text(json.dumps(state))
        log(f"  {key} {path}: best of {len(pop)} enumerated {fitness(pop[0]):.2f} us {pop[0]}")
        return pop[0], fitness(pop[0])
    pop = entry["population"] or [random_genome(rng, path) for _ in range(population)]
    for gen in range(entry["generation"], generations):
        pop.sort(key=fitness)
        elite = pop[: max(2, population // 4)]
        log(f"  {key} gen {gen}: best {fitness(elite[0]):.2f} us {elite[0]}")
        children = list(elite)
        while len(children) < population:
            a, b = rng.sample(elite, 2)
            children.append(mutate(rng, crossover(rng, a, b), path))
        pop = children
        entry["population"], entry["generation"] = pop, gen + 1
        state_path.write_text(json.dumps(state))
    pop.sort(key=fitness)
    return pop[0], fitness(pop[0])


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shapes", nargs="+", required=True, help="MxK pairs, e.g. 28672x4096")
    ap.add_argument("--tokens", nargs="+", type=int, default=[16])
    ap.add_argument("--path", choices=["auto", "stream", "tstream", "umma"], default="auto",
                    help="auto: measure every kernel family that suits the token count and keep the fastest")
    ap.add_argument("--generations", type=int, default=5)
    ap.add_argument("--population", type=int, default=12)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--state", type=Path, default=Path("tuner_state.json"))
    ap.add_argument("--param-map", type=Path, default=make_configs.PARAM_MAP)
    args = ap.parse_args(argv)
    pm = make_configs.load(args.param_map) if args.param_map.exists() else {}
    for shape in args.shapes:
        m, k = (int(v) for v in shape.lower().split("x"))
        for n in args.tokens:
            paths = (args.path,) if args.path != "auto" else candidate_paths(n)
            bench = Bench(m, n, k, args.seed)
            results = []
            for path in paths:
                best, us = tune_shape(m, n, k, path, args.generations, args.population, args.seed, args.state, bench=bench)
                if us != float("inf"):
                    results.append((us, path, best))
            if not results:
                print(f"{m}x{k} n={n}: no valid configuration found")
                continue
            us, path, best = min(results, key=lambda r: r[0])
            note = ", ".join(f"{p_} {u:.2f} us" for u, p_, _ in sorted(results, key=lambda r: r[0]))
            pm[f"{m}_{make_configs.token_bucket(n)}_{k}"] = {"path": path, "tile_tok": tile_tok_for(path, n), **best, "us": round(us, 2),
                                                             "note": note}
            print(f"{m}x{k} n={n}: {path} {us:.2f} us {best}   [{note}]", flush=True)
            args.param_map.write_text(json.dumps(pm, indent=1, sort_keys=True))
    make_configs.generate(args.param_map)


if __name__ == "__main__":
    main()
