"""Benchmark of the FP16 x 4-bit(codebook) GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--no-extras]

Headline workload (default `mistral7b_mlp_m16`): the Mistral-7B MLP GEMMs at 16 tokens -
fused gate+up K=4096 -> N=28672, then down K=14336 -> N=4096 - for 32 layers
with DISTINCT synthetic weights per layer (2.7 GB of packed codes, far larger
than L2, so every step streams from HBM).  One step = one pass over the 32
layers = 64 GEMMs.  With N GPUs the layers are tensor-parallel: ONE seeded weight set is
sharded through tuna_b200.sharding - gate+up by output columns (no collective), down along K
with an NCCL all-reduce of the partial outputs; total work is fixed ("strong").

The metric is the reference README's: time per 16-token GEMM, expressed as
effective HBM bandwidth = algorithmic bytes / time, with
    bytes(m, n, k) = m*k/2 + 4*m + 64 + 2*n*k + 2*n*m.
`value` is measured with inputs resident on the device (CUDA-graph replay of
the step, repeated so that the timed region lasts about a second); `e2e` calls the op with HOST
activations and outputs (pinned memory, copies inside the timed region); `roofline` times the
dominant kernel alone; `extras` (one GPU) holds the other BASELINE configurations: the Llama-70B
80-layer sweep, the Mixtral combined-expert GEMMs and the token sweep on the Llama-70B gate+up
shape.  `--impl reference` runs the reference's own CUDA kernels (oracle/_ref, compiled from the
reference tree where it lies) on the same workload when that library travelled with the tree,
else the CPU restatement of dequantize-then-matmul; `cpu_baseline` is that CPU restatement
timed on the host cores.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (layers, [(kind, m, k)], tokens)
    "mistral7b_mlp_m16": (32, [("col", 28672, 4096), ("row", 4096, 14336)], 16),
    "llama70b_layer_m16": (80, [("col", 10240, 8192), ("row", 8192, 8192), ("col", 57344, 8192), ("row", 8192, 28672)], 16),
    "mistral7b_qkv_m16": (32, [("col", 6144, 4096)], 16),
    # Mixtral-8x7B expert projections as the reference benchmarks them: one combined GEMM per
    # projection over all 8 experts (make_configs.py:105-106, README.md:18)
    "mixtral8x7b_combined_m16": (8, [("col", 229376, 4096), ("row", 32768, 14336)], 16),
    # token-count sweep of the largest Llama-70B GEMM (one layer each; tensor-core regime from 256 up)
    "llama70b_gateup_m256": (2, [("col", 57344, 8192)], 256),
    "llama70b_gateup_m2048": (2, [("col", 57344, 8192)], 2048),
}
FALLBACK_HBM_GBS = 6650.0
NOMINAL_FP16_TFLOPS = 2250.0
TARGET_TIMED_SECONDS = 1.0
KERNEL_NAMES = {1: "gemm_stream_kernel (mma.sync)", 2: "gemm_w4a16_umma_kernel (tcgen05, TMA-staged)",
                3: "gemm_w4a16_tstream_kernel (tcgen05 weight streaming)"}


def alg_bytes(m: int, n: int, k: int) -> int:
    return m * k // 2 + 4 * m + 64 + 2 * n * k + 2 * n * m


def measured_peak(key: str = "hbm_gbs", fallback: float = FALLBACK_HBM_GBS):
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())[key]), "measured"
        except Exception:
            pass
    return fallback, "fallback"


class ClockSampler:
    """Samples SM clocks, power and throttle reasons with nvidia-smi; `stop()` summarises the samples
    whose time stamps lie inside the timed regions that were registered with `window()`."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    SETTLE_S = 0.15  # a sample this soon after the start of a region may still show the idle state

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.windows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, bufsize=1)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def window(self, t0: float, t1: float):
        """Registers a timed region by its wall-clock start and end (time.time())."""
        self.windows.append((t0, t1))

    @staticmethod
    def _stamp(text):
        import datetime
        return datetime.datetime.strptime(text, "%Y/%m/%d %H:%M:%S.%f").timestamp()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"], "samples": 0}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, watts, reasons, seen = [], [], [], set(), 0
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in list(self.samples):
            f = [t.strip() for t in s.split(",")]
            if len(f) < 8:
                continue
            try:
                t = self._stamp(f[0])
                clock, cmax = float(f[1]), float(f[2])
            except ValueError:
                continue
            seen += 1
            mx.append(cmax)
            if not any(t0 + self.SETTLE_S <= t <= t1 for t0, t1 in self.windows):
                continue
            sm.append(clock)
            try:
                watts.append(float(f[3]))
            except ValueError:
                pass
            for name, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "power_w": statistics.median(watts) if watts else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_outside_timed_regions": seen - len(sm),
                "what": "nvidia-smi every 50 ms; only the samples inside the timed region of the headline step count"}


# --------------------------------------------------------------------------- reference arms

def host_threads() -> int:
    """All the host cores this process may use, whatever OMP_NUM_THREADS a launcher set."""
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def load_oracle_lib():
    os.environ["OMP_NUM_THREADS"] = str(host_threads())  # before the OpenMP runtime of the library starts
    so = ROOT / "oracle" / "libtuna_oracle.so"
    if not so.exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "oracle"], check=True, capture_output=True)
    return ctypes.CDLL(str(so))


def cpu_reference_step(shapes, tokens, reps, oracle, layers=1):
    """dequantize (C oracle, all host threads) + torch.matmul (fp16, CPU) for each GEMM of `layers`
    layers with distinct weights.  Returns (seconds per pass list, algorithmic bytes per pass, threads)."""
    from oracle import tuna_oracle as orc

    torch.set_num_threads(host_threads())
    rng = np.random.default_rng(0)
    cases = []
    for _layer in range(layers):
        for _kind, m, k in shapes:
            q = rng.integers(0, 256, size=m * k // 2, dtype=np.uint8)
            absmax = (0.005 + 0.015 * rng.random(m, dtype=np.float32)).astype(np.float16).astype(np.float32)
            x = torch.from_numpy(rng.standard_normal((tokens, k), dtype=np.float32).astype(np.float16))
            cases.append((m, k, q, absmax, x))
    scratch = {(m, k): np.empty((m, k), dtype=np.uint16) for _, m, k in shapes}
    code = orc.NF4_CODE.copy()
    vp = ctypes.c_void_p

    def one_pass():
        for m, k, q, absmax, x in cases:
            w = scratch[(m, k)]
            oracle.oracle_dequant(q.ctypes.data_as(vp), absmax.ctypes.data_as(vp), code.ctypes.data_as(vp),
                                  w.ctypes.data_as(vp), m, k)
            wt = torch.from_numpy(w.view(np.float16))
            torch.matmul(x, wt.t())

    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
    nbytes = layers * sum(alg_bytes(m, tokens, k) for _, m, k in shapes)
    return times, nbytes, torch.get_num_threads()


def cpu_baseline_record(layers, shapes, tokens):
    oracle = load_oracle_lib()
    sample_layers = min(layers, 8)
    times, nbytes, threads = cpu_reference_step(shapes, tokens, 4, oracle, sample_layers)
    sec = statistics.median(times[1:])
    return {"value": nbytes / sec / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{sample_layers} of {layers} layers with distinct weights ({sample_layers * len(shapes)} GEMMs, "
                      f"{nbytes / 1e6:.1f} MB algorithmic), median of 3 after 1 warm-up: C restatement of the "
                      "reference's dequant (all host threads) + torch.matmul fp16 on CPU",
            "seconds_per_sample": sec}


REF_GAP = 4 << 20  # the reference's loaders prefetch past a tensor's end without bounds checks: keep reads in owned memory


def reference_gpu_arm(args, layers, shapes, tokens):
    """The reference's own kernels (kernel.cu compiled where it lies into oracle/_ref/libtuna_ref.so),
    launched through its `wrapper` (kernel.cu:3009) on the same workload: full-size layers on ONE GPU
    (the reference has no multi-GPU code and silently launches nothing for shapes outside its table,
    kernel.cu:3022-3155, which all sharded sub-shapes are).  Its output must be zero-filled before every
    call (kernel.cu:2739-2745); that memset is part of what a caller pays and is inside the timed region."""
    so = ROOT / "oracle" / "_ref" / "libtuna_ref.so"
    if not so.exists() or not torch.cuda.is_available():
        return None
    ref = ctypes.CDLL(str(so))
    vp, ci = ctypes.c_void_p, ctypes.c_int
    ref.tuna_ref_matmul.argtypes = [vp] * 5 + [ci] * 3 + [vp]
    from tuna_b200.codebooks import nf4_tensor

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1000)

    def carve(nbytes):
        slab = torch.zeros(nbytes + 2 * REF_GAP, dtype=torch.uint8, device=dev)
        return slab, slab[REF_GAP:REF_GAP + nbytes]

    keep, gemms = [], []
    cslab, cview = carve(64)
    cview.view(torch.float32).copy_(nf4_tensor(dev))
    keep.append(cslab)
    for _layer in range(layers):
        per = []
        for _kind, m, k in shapes:
            qs, qv = carve(m * k // 2)
            qv.copy_(torch.randint(0, 256, (m * k // 2,), dtype=torch.uint8, device=dev, generator=gen))
            ss, sv = carve(m * 4)
            sv.view(torch.float32).copy_((0.005 + 0.015 * torch.rand(m, device=dev, generator=gen)).half().float())
            keep += [qs, ss]
            per.append((m, k, qv, sv))
        gemms.append(per)
    xs, os_, xh, oh = [], [], [], []
    xgen = torch.Generator(device="cpu")
    xgen.manual_seed(7)
    for _kind, m, k in shapes:
        x_host = torch.randn((tokens, k), generator=xgen).half().pin_memory()
        s1, xv = carve(tokens * k * 2)
        xv.view(torch.float16).view(tokens, k).copy_(x_host)
        s2, ov = carve(tokens * m * 2)
        keep += [s1, s2]
        xs.append(xv)
        os_.append(ov)
        xh.append(x_host)
        oh.append(torch.empty((tokens, m), dtype=torch.float16).pin_memory())
    stream = torch.cuda.Stream(device=dev)

    def step(e2e: bool):
        for per in gemms:
            for i, (m, k, qv, sv) in enumerate(per):
                if e2e:
                    xs[i].view(torch.float16).view(tokens, k).copy_(xh[i], non_blocking=True)
                os_[i].zero_()
                ref.tuna_ref_matmul(qv.data_ptr(), xs[i].data_ptr(), cview.data_ptr(), sv.data_ptr(), os_[i].data_ptr(),
                                    m, tokens, k, stream.cuda_stream)
                if e2e:
                    oh[i].copy_(os_[i].view(torch.float16).view(tokens, m), non_blocking=True)

    def timed(e2e):
        with torch.cuda.stream(stream):
            for _ in range(args.warmup):
                step(e2e)
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(args.steps):
                step(e2e)
            e1.record(stream)
            stream.synchronize()
        return e0.elapsed_time(e1) / args.steps

    with torch.cuda.stream(stream):
        step(False)
        stream.synchronize()
        nz = float((os_[0].view(torch.float16) != 0).float().mean())
    if nz < 0.5:
        return None  # the reference launched nothing for this shape
    ms, ms_e2e = timed(False), timed(True)
    return ms, ms_e2e, nz


def run_reference_arm(args, layers, shapes, tokens):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # rank 0 alone runs the reference; the other ranks exit 0 without work
    total = layers * sum(alg_bytes(m, tokens, k) for _, m, k in shapes)
    cpu = None
    try:
        cpu = cpu_baseline_record(layers, shapes, tokens)
    except Exception as exc:
        cpu = {"value": None, "unit": "GB/s", "cores": host_threads(), "kind": "port", "sample": f"failed: {type(exc).__name__}"}
    gpu = None
    try:
        gpu = reference_gpu_arm(args, layers, shapes, tokens)
    except Exception as exc:  # the library is test infrastructure: fall back to the CPU port
        gpu = None
        print(json.dumps({"note": f"reference GPU arm failed: {type(exc).__name__}: {exc}"}), file=sys.stderr)
    base = {
        "impl": "reference", "metric": "m16_gemm_effective_hbm_bandwidth", "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16*u4->f32", "data": "synthetic", "cpu_baseline": cpu,
    }
    if gpu is not None:
        ms, ms_e2e, nz = gpu
        h2d = layers * sum(tokens * k * 2 for _, _m, k in shapes)
        d2h = layers * sum(tokens * m * 2 for _, m, _k in shapes)
        line = dict(base, value=total / (ms * 1e-3) / 1e9, ms_per_step=ms,
                    config={"workload": args.workload, "tokens": tokens, "layers": layers,
                            "step": "the full workload on ONE GPU (the reference cannot shard: unknown shapes are silent no-ops)",
                            "timing": "CUDA events, eager launches through the reference's wrapper(), output zero-fill included",
                            "kind": "reference: its own kernel.cu compiled for sm_100 into oracle/_ref (A6000-tuned table, mma.sync)"},
                    e2e={"value": total / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e,
                         "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                         "how": "per GEMM: pinned-host x -> device, zero-fill o, wrapper(), o -> pinned host, one stream"},
                    gpu_launches=layers * len(shapes) * args.steps, nonzero_output_fraction=nz)
        print(json.dumps(line), flush=True)
        return
    if cpu is None or cpu.get("value") is None:
        print(json.dumps({"impl": "reference", "unavailable": "neither oracle/_ref nor the CPU port could run here"}), flush=True)
        return
    gbs = cpu["value"]
    line = dict(base, value=gbs, ms_per_step=cpu["seconds_per_sample"] * 1e3,
                config={"workload": args.workload, "tokens": tokens, "step": "bounded sample: " + cpu["sample"], "timing": "host wall clock"},
                e2e={"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, gpu_launches=0)
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm helpers

def make_timer(stream, world, dev):
    import torch.distributed as dist

    def timed(fn, steps, warmup, inner=1, sampler=None):
        """ms per call of fn: `warmup` untimed calls, then steps * inner timed ones between events.
        With `sampler` the region's wall-clock bounds are registered with it."""
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                fn()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            wall0 = time.time()
            e0.record(stream)
            for _ in range(steps * inner):
                fn()
            e1.record(stream)
            stream.synchronize()
            torch.cuda.synchronize()
            if sampler is not None:
                sampler.window(wall0, time.time())
            if world > 1:
                dist.barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / (steps * inner)

    def inner_for(fn, steps):
        """Repeats per timed step so that the timed region lasts about TARGET_TIMED_SECONDS."""
        ms = timed(fn, 1, 2, 1)
        inner = max(1, int(round(TARGET_TIMED_SECONDS * 1e3 / (ms * steps))))
        if world > 1:
            t = torch.tensor([inner], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            inner = int(t.item())
        return inner

    return timed, inner_for


def roofline_record(m, tokens, k, us, path, timing):
    flops = 2.0 * m * tokens * k
    nbytes = alg_bytes(m, tokens, k)
    hbm, hkind = measured_peak()
    tpeak, tkind = measured_peak("bf16_tflops", 1590.0)
    tf = flops / (us * 1e-6) / 1e12
    gbs = nbytes / (us * 1e-6) / 1e9
    rec = {"shape": {"m": m, "n": tokens, "k": k}, "kernel": KERNEL_NAMES.get(path, str(path)), "us_per_launch": us,
           "gbs": gbs, "frac_hbm": gbs / hbm, "tflops": tf, "frac_tensor_burst": tf / tpeak, "frac_tensor_nominal": tf / NOMINAL_FP16_TFLOPS,
           "bound": "tensor" if tf / tpeak > gbs / hbm else "hbm", "timing": timing,
           "peaks": {"hbm_gbs": hbm, "hbm_source": hkind, "bf16_tflops_burst": tpeak, "tensor_source": tkind, "fp16_tflops_nominal": NOMINAL_FP16_TFLOPS}}
    return rec


def run_extras(dev, stream, timed, code, steps):
    """The other BASELINE configurations on one GPU: per-GEMM times over distinct weights
    (more than twice the L2 capacity per shape, or the whole layer sweep)."""
    import tuna_b200

    lib_ws = torch.zeros(int(96 << 20), dtype=torch.uint8, device=dev)
    out = {}

    def gemm_set(m, k, count, gen):
        qs = [torch.randint(0, 256, (m * k // 2,), dtype=torch.uint8, device=dev, generator=gen) for _ in range(count)]
        s = (0.005 + 0.015 * torch.rand(m, device=dev, generator=gen)).half().float()
        return qs, s

    # ---- layer sweeps: every layer its own weights, one CUDA graph per sweep
    for name in ("llama70b_layer_m16", "mixtral8x7b_combined_m16"):
        layers, shapes, tokens = WORKLOADS[name]
        gen = torch.Generator(device=dev)
        gen.manual_seed(4242)
        sets = [gemm_set(m, k, layers, gen) for _, m, k in shapes]
        xs = [torch.randn((tokens, k), device=dev, generator=gen).half() for _, _m, k in shapes]
        os_ = [torch.empty((tokens, m), dtype=torch.float16, device=dev) for _, m, _k in shapes]

        def sweep(only=None):
            for li in range(layers):
                for i, (_, m, k) in enumerate(shapes):
                    if only is None or only == i:
                        tuna_b200.matmul(xs[i], sets[i][0][li], sets[i][1], code, os_[i], m, tokens, k, workspace=lib_ws)

        # the sweep through the sequence API: every GEMM its own output
        o_all = [[torch.empty((tokens, m), dtype=torch.float16, device=dev) for _, m, _k in shapes] for _ in range(layers)]
        seq = tuna_b200.MatmulSequence([(xs[i], sets[i][0][li], sets[i][1], o_all[li][i], m, tokens, k)
                                        for li in range(layers) for i, (_, m, k) in enumerate(shapes)], code)
        with torch.cuda.stream(stream):
            seq.run()
            stream.synchronize()
            gs = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gs, stream=stream):
                seq.run()
            sweep()
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                sweep()
        ms_seq = timed(gs.replay, max(3, steps // 4), 2, max(1, int(50 / max(1.0, layers * len(shapes) * 0.02))))
        ms = timed(g.replay, max(3, steps // 4), 2)
        total = layers * sum(alg_bytes(m, tokens, k) for _, m, k in shapes)
        per_shape = []
        for i, (_, m, k) in enumerate(shapes):
            us = timed(lambda i=i: sweep(i), 3, 1) * 1e3 / layers
            cfg = tuna_b200.lookup_config(m, tokens, k)
            per_shape.append(roofline_record(m, tokens, k, us, cfg.path, "that GEMM alone (tuna_matmul) over the layers' distinct weights, eager back-to-back launches"))
        hbm, _ = measured_peak()
        out[name] = {"layers": layers, "tokens": tokens, "gemms": layers * len(shapes), "bytes_per_sweep": total,
                     "sequence": {"ms_per_sweep": ms_seq, "gbs": total / (ms_seq * 1e-3) / 1e9, "frac_hbm": total / (ms_seq * 1e-3) / 1e9 / hbm,
                                  "api": "tuna_matmul_sequence (persistent launches of up to 64 GEMMs), CUDA graph replay"},
                     "per_call": {"ms_per_sweep": ms, "gbs": total / (ms * 1e-3) / 1e9, "frac_hbm": total / (ms * 1e-3) / 1e9 / hbm,
                                  "api": "tuna_matmul, one launch per GEMM, CUDA graph replay of the whole sweep"},
                     "gemms_alone": per_shape}
        del sets, g, gs, seq, o_all
        torch.cuda.empty_cache()

    # ---- Mixtral's experts as separate GEMMs with per-expert token lists (the reference benchmarks one combined
    # GEMM over all experts instead, make_configs.py:105-106): 16 tokens routed to 2 of 8 experts each
    layers, counts = 4, [7, 5, 4, 4, 3, 3, 3, 3]
    gen = torch.Generator(device=dev)
    gen.manual_seed(99)
    gemms, total = [], 0
    for _ in range(layers):
        for m, k in ((28672, 4096), (4096, 14336)):  # gate+up, down of every expert
            for n_e in counts:
                q = torch.randint(0, 256, (m * k // 2,), dtype=torch.uint8, device=dev, generator=gen)
                sc = (0.005 + 0.015 * torch.rand(m, device=dev, generator=gen)).half().float()
                x = torch.randn((n_e, k), device=dev, generator=gen).half()
                o = torch.empty((n_e, m), dtype=torch.float16, device=dev)
                gemms.append((x, q, sc, o, m, n_e, k))
                total += alg_bytes(m, n_e, k)
    seq = tuna_b200.MatmulSequence(gemms, code)
    with torch.cuda.stream(stream):
        seq.run()
        stream.synchronize()
        gs = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gs, stream=stream):
            seq.run()
    ms_seq = timed(gs.replay, max(3, steps // 4), 2, 20)
    hbm, _ = measured_peak()
    out["mixtral8x7b_experts_m16"] = {"layers": layers, "experts": 8, "tokens_per_expert": counts, "gemms": len(gemms), "bytes_per_sweep": total,
                                      "sequence": {"ms_per_sweep": ms_seq, "gbs": total / (ms_seq * 1e-3) / 1e9, "frac_hbm": total / (ms_seq * 1e-3) / 1e9 / hbm,
                                                   "api": "tuna_matmul_sequence with one entry per expert (its own token count), CUDA graph replay"}}
    del gemms, seq, gs
    torch.cuda.empty_cache()

    # ---- token sweep on the Llama-70B gate+up shape (BASELINE config 4)
    m, k = 57344, 8192
    gen = torch.Generator(device=dev)
    gen.manual_seed(77)
    qs, s = gemm_set(m, k, 3, gen)  # 3 x 235 MB: every launch streams its weights from HBM
    rows = []
    for tokens in (1, 16, 64, 256, 1024, 2048, 4096):
        x = torch.randn((tokens, k), device=dev, generator=gen).half()
        o = torch.empty((tokens, m), dtype=torch.float16, device=dev)

        def rot():
            for q in qs:
                tuna_b200.matmul(x, q, s, code, o, m, tokens, k, workspace=lib_ws)

        reps = 3 if tokens >= 1024 else 5
        us = timed(rot, reps, 2) * 1e3 / len(qs)
        cfg = tuna_b200.lookup_config(m, tokens, k)
        rows.append(roofline_record(m, tokens, k, us, cfg.path, "rotating over 3 weight sets (705 MB), eager back-to-back launches"))
        del x, o
    out["llama70b_gateup_token_sweep"] = rows
    return out


# --------------------------------------------------------------------------- GPU arm

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mistral7b_mlp_m16", choices=sorted(WORKLOADS))
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of CUDA-graph replay")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-groups", type=int, default=4, help="groups the end-to-end step is cut into (copy-in / launch / copy-out pipeline)")
    ap.add_argument("--no-fused", action="store_true", help="N > 1: skip the fused GEMM + reduce step (tuna_matmul_sequence_reduce)")
    ap.add_argument("--no-extras", action="store_true", help="skip the sub-records of the other BASELINE configurations")
    ap.add_argument("--layers", type=int, default=0, help="use only the first N layers (profiling captures); 0 = all")
    ap.add_argument("--inner", type=int, default=0, help="repeats of the step inside one timed step (0 = fill about a second)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else max(args.warmup, 1)
    layers, shapes, tokens = WORKLOADS[args.workload]
    if args.layers > 0:
        layers = min(layers, args.layers)

    if args.impl == "reference":
        run_reference_arm(args, layers, shapes, tokens)
        return

    import torch.distributed as dist

    import tuna_b200
    from oracle import tuna_oracle as orc
    from tuna_b200 import _lib, sharding
    from tuna_b200.codebooks import nf4_tensor

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        # a rank that stops answering must not hold the whole job: give up after a bounded time
        limit = float(os.environ.get("TUNA_BENCH_WATCHDOG_S", "600"))

        def _give_up():
            print(json.dumps({"error": f"rank {rank}: multi-GPU bench exceeded {limit:.0f} s, aborted"}), flush=True)
            os._exit(2)

        watchdog = threading.Timer(limit, _give_up)
        watchdog.daemon = True
        watchdog.start()
    lib = _lib.load()

    # ---- ONE seeded synthetic weight set (uniform-random codes, scales U[0.005, 0.02] rounded to fp16):
    # every rank generates the same full layer on its GPU and keeps its shard (tuna_b200.sharding)
    code = nf4_tensor(dev)
    gemms = []   # per layer: list of dicts with this rank's shard
    full0 = None  # layer 0 in full, for the parity check
    for layer in range(layers):
        gen = torch.Generator(device=dev)
        gen.manual_seed(1000 + layer)
        per, full = [], []
        for kind, m, k in shapes:
            q = torch.randint(0, 256, (m * k // 2,), dtype=torch.uint8, device=dev, generator=gen)
            s = (0.005 + 0.015 * torch.rand(m, device=dev, generator=gen)).half().float()
            if kind == "col":
                qs, ss, ms = sharding.shard_columns(q, s, m, k, world, rank)
                per.append(dict(kind=kind, m=ms, k=k, q=qs.contiguous().view(-1) if world > 1 else q, s=ss.contiguous() if world > 1 else s))
            else:
                qs, ks = sharding.shard_k(q, m, k, world, rank)
                per.append(dict(kind=kind, m=m, k=ks, q=qs.view(-1) if world > 1 else q, s=s))
            if layer == 0:
                full.append((q, s))
            else:
                del q
        gemms.append(per)
        if layer == 0:
            full0 = full
    xgen = torch.Generator(device="cpu")
    xgen.manual_seed(7)
    x_full, x_host, x_dev, o_dev, o_host = [], [], [], [], []
    for i, (kind, m, k) in enumerate(shapes):
        g0 = gemms[0][i]
        xh = torch.randn((tokens, k), generator=xgen).half()
        x_full.append(xh)
        if kind == "row" and world > 1:
            xh = xh[:, rank * g0["k"]:(rank + 1) * g0["k"]].contiguous()
        x_host.append(xh.pin_memory())
        x_dev.append(xh.to(dev))
        o_dev.append(torch.empty((tokens, g0["m"]), dtype=torch.float16, device=dev))
        o_host.append(torch.empty((tokens, g0["m"]), dtype=torch.float16).pin_memory())
    ws_bytes = max(int(lib.tuna_matmul_workspace_bytes(g["m"], tokens, g["k"])) for g in gemms[0])
    ws = torch.zeros(max(ws_bytes, 1 << 20), dtype=torch.uint8, device=dev)
    stream = torch.cuda.Stream(device=dev)
    timed, inner_for = make_timer(stream, world, dev)

    # ---- parity of the sharded layer 0 against the oracle, outside every timed region
    parity = None
    if True:
        rec = {}
        rng = np.random.default_rng(5)
        with torch.cuda.stream(stream):
            for i, (kind, m, k) in enumerate(shapes):
                g0 = gemms[0][i]
                tuna_b200.matmul(x_dev[i], g0["q"], g0["s"], code, o_dev[i], g0["m"], tokens, g0["k"], workspace=ws)
                if kind == "col":
                    if world > 1:
                        gathered = torch.empty((world * tokens, g0["m"]), dtype=torch.float16, device=dev)
                        dist.all_gather_into_tensor(gathered, o_dev[i])
                        full_o = gathered.view(world, tokens, g0["m"]).permute(1, 0, 2).reshape(tokens, m)
                    else:
                        full_o = o_dev[i]
                else:
                    full_o = o_dev[i].clone()
                    if world > 1:
                        dist.all_reduce(full_o)
                stream.synchronize()
                if rank == 0:
                    qf, sf = full0[i]
                    groups = np.unique(np.concatenate([rng.integers(0, m // 8, 24), [0, m // 8 - 1]]))
                    gi = torch.from_numpy(groups).to(dev)
                    q3 = qf.view(m // 8, k // 8, 32)[gi].cpu().numpy()
                    sc = sf.view(-1, 8)[gi].reshape(-1).cpu().numpy()
                    ref = orc.matmul_ref(x_full[i].numpy(), q3, sc, orc.NF4_CODE, len(groups) * 8, tokens, k)
                    got = full_o.view(tokens, m // 8, 8)[:, gi].reshape(tokens, -1).cpu().numpy()
                    a, b = orc.parity_error(got, ref)
                    rec[f"{kind}_{m}x{k}"] = {"max_norm_err": float(a), "mixed_err": float(b)}
        if rank == 0:
            # column-parallel shards are exact per column; row-parallel sums world fp16-rounded partials
            tol = 1e-2
            parity = {"checked": "layer 0, sampled 8-row groups, sharded result (all-gather / all-reduce) vs the CPU oracle",
                      "tolerance": tol, "results": rec, "ok": all(v["max_norm_err"] <= tol and v["mixed_err"] <= tol for v in rec.values())}
    full0 = None
    torch.cuda.empty_cache()

    # K-split layers: every layer has its own output so that its all-reduce (NCCL's stream) can stay
    # in flight under the next layers' GEMMs; the step ends when the last reduction has finished
    o_layer = None
    if world > 1:
        o_layer = [[torch.empty_like(o_dev[i]) if g["kind"] == "row" else None for i, g in enumerate(per)] for per in gemms]

    # The step through the sequence API: every GEMM of the step (all layers) in persistent launches
    # of up to 64 GEMMs (tuna_matmul_sequence); every GEMM has its own output.  The all-reduces of
    # the K-split layers follow the launch (asynchronously, joined at the end of the step).
    # (the K-split layers' outputs lie back to back in one buffer, so ONE all-reduce sums them all)
    n_row = sum(1 for per in gemms for g in per if g["kind"] == "row")
    row_elems = max([tokens * g["m"] for g in gemms[0] if g["kind"] == "row"], default=0)
    o_rows = torch.empty((max(n_row, 1), max(row_elems, 1)), dtype=torch.float16, device=dev)
    o_seq, r = [], 0
    for per in gemms:
        outs = []
        for g in per:
            if g["kind"] == "row":
                outs.append(o_rows[r, :tokens * g["m"]].view(tokens, g["m"]))
                r += 1
            else:
                outs.append(torch.empty((tokens, g["m"]), dtype=torch.float16, device=dev))
        o_seq.append(outs)
    seq_gemms = [(x_dev[i], g["q"], g["s"], o_seq[li][i], g["m"], tokens, g["k"]) for li, per in enumerate(gemms) for i, g in enumerate(per)]
    seq = tuna_b200.MatmulSequence(seq_gemms, code)
    ws = seq.workspace  # sized for the sequence and for every GEMM of it on its own

    def step_device(collectives=True):
        seq.run()
        if collectives and world > 1 and n_row:
            dist.all_reduce(o_rows)

    # The same step with the K-split layers' sum fused into the launch (tuna_matmul_sequence_reduce):
    # the epilogue stores finished rows into every rank's exchange buffer over NVLink while the
    # weights stream, a small kernel per launch exchanges flags and adds the slabs; no collective.
    fused, fused_note, o_fused = None, None, None
    if world > 1 and n_row and not args.no_fused:
        try:
            o_fused = [[torch.empty_like(o) for o in outs] for outs in o_seq]
            fg = [(x_dev[i], g["q"], g["s"], o_fused[li][i], g["m"], tokens, g["k"]) for li, per in enumerate(gemms) for i, g in enumerate(per)]
            partial = [g["kind"] == "row" for per in gemms for g in per]
            need = tuna_b200.ReduceSequence.exchange_bytes([(g[4], g[5], g[6]) for g in fg], world, partial)
            exchange = tuna_b200.Exchange(need, dev, group=dist.group.WORLD)
            fused = tuna_b200.ReduceSequence(fg, code, exchange, partial=partial)
        except Exception as exc:  # e.g. no CUDA IPC between the ranks' processes: the collective path stays
            fused, fused_note = None, f"{type(exc).__name__}: {exc}"
        ok = torch.tensor([1 if fused is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)  # all ranks or none
        if int(ok.item()) == 0:
            fused = None

    # The same step GEMM by GEMM (tuna_matmul, one launch each): reported beside the headline
    def step_per_call(collectives=True):
        pending = []
        for li, per in enumerate(gemms):
            for i, g in enumerate(per):
                out = o_layer[li][i] if (o_layer is not None and o_layer[li][i] is not None) else o_dev[i]
                tuna_b200.matmul(x_dev[i], g["q"], g["s"], code, out, g["m"], tokens, g["k"], workspace=ws)
                if collectives and g["kind"] == "row" and world > 1:
                    pending.append(dist.all_reduce(out, async_op=True))
        for h in pending:
            h.wait()

    # end to end: every GEMM takes its activations from pinned HOST memory and returns its output
    # there, through the package's host-buffer API: the sequence in 4 groups, group j's copy-in,
    # group j-1's launch and group j-2's copy-out overlapping on three streams; the step ends when
    # the last output has reached the host
    # host activations: every GEMM has its own buffer (a copy of its shape's activations), all of them back to
    # back in one pinned slab in GEMM order, so that HostSequence can bring in a group with one copy
    x_slab_host = torch.empty(layers * sum(t.numel() for t in x_host), dtype=torch.float16).pin_memory()
    x_host_l, pos = [], 0
    for per in gemms:
        row = []
        for i, _ in enumerate(per):
            v = x_slab_host[pos:pos + x_host[i].numel()].view_as(x_host[i])
            v.copy_(x_host[i])
            pos += x_host[i].numel()
            row.append(v)
        x_host_l.append(row)
    # host outputs: one pinned slab per pool (column-parallel / K-split outputs), the GEMMs' outputs back to
    # back in it, so that HostSequence can return neighbouring outputs with one copy
    slab_elems = {0: 0, 1: 0}
    for per in gemms:
        for g in per:
            slab_elems[1 if g["kind"] == "row" else 0] += tokens * g["m"]
    host_slab = {pid: torch.empty(max(n_, 1), dtype=torch.float16).pin_memory() for pid, n_ in slab_elems.items()}
    used = {0: 0, 1: 0}
    o_host_l = []
    for per in gemms:
        outs = []
        for g in per:
            pid = 1 if g["kind"] == "row" else 0
            outs.append(host_slab[pid][used[pid]:used[pid] + tokens * g["m"]].view(tokens, g["m"]))
            used[pid] += tokens * g["m"]
        o_host_l.append(outs)
    host_gemms = [(x_host_l[li][i], g["q"], g["s"], o_host_l[li][i], g["m"], tokens, g["k"]) for li, per in enumerate(gemms) for i, g in enumerate(per)]
    pool_ids = [1 if g["kind"] == "row" else 0 for per in gemms for g in per]  # pool 1: outputs that need the all-reduce

    def reduce_rows(pools):
        if 1 in pools:
            dist.all_reduce(pools[1])

    hseq, e2e_reduce = None, ("NCCL all-reduce per group" if world > 1 else None)
    if fused is not None:
        try:  # the end-to-end step with the fused sum as well: its own exchange buffers, sized for a group's launch
            exchange2 = tuna_b200.Exchange(exchange.nbytes, dev, group=dist.group.WORLD)
            hseq = tuna_b200.HostSequence(host_gemms, code, groups=args.e2e_groups, pool_ids=pool_ids, exchange=exchange2,
                                          partial=[g["kind"] == "row" for per in gemms for g in per])
            e2e_reduce = "fused (tuna_matmul_sequence_reduce per group)"
        except Exception:
            hseq = None
        ok = torch.tensor([1 if hseq is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            hseq, e2e_reduce = None, "NCCL all-reduce per group"
    if hseq is None:
        hseq = tuna_b200.HostSequence(host_gemms, code, groups=args.e2e_groups, after_group=reduce_rows if world > 1 else None, pool_ids=pool_ids)

    def step_e2e():
        hseq.run()

    launches_per_step = -(-(layers * len(shapes)) // 64)  # persistent launches of up to 64 GEMMs
    gemms_per_step = layers * len(shapes)
    total_bytes = layers * sum(alg_bytes(m, tokens, k) for _, m, k in shapes)

    def capture(fn):
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                fn()
        return g

    # ---- device-resident number: CUDA-graph replay of one step (or eager with --no-graph)
    graph = None if args.no_graph else capture(step_device)
    run_dev = graph.replay if graph is not None else step_device
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    inner = args.inner if args.inner > 0 else inner_for(run_dev, args.steps)
    ms_step = timed(run_dev, args.steps, args.warmup, inner, sampler if rank == 0 else None)
    ms_eager = timed(step_device, max(args.steps // 4, 3), 2) if graph is not None else ms_step
    pc_graph = None if args.no_graph else capture(step_per_call)
    ms_per_call = timed(pc_graph.replay if pc_graph is not None else step_per_call, args.steps, args.warmup, max(1, inner // 2))
    ms_gemm_only = None
    ms_fused, fused_err = None, None
    if world > 1:
        g2 = None if args.no_graph else capture(lambda: step_device(False))
        ms_gemm_only = timed(g2.replay if g2 is not None else (lambda: step_device(False)), args.steps, args.warmup, inner)
        if fused is not None:
            g3 = None if args.no_graph else capture(fused.run)
            ms_fused = timed(g3.replay if g3 is not None else fused.run, args.steps, args.warmup, inner)
            # the fused sums against the all-reduced ones (both sum fp16 partials; the order of the adds differs)
            with torch.cuda.stream(stream):
                step_device()
                stream.synchronize()
            worst = 0.0
            r = 0
            for li, per in enumerate(gemms):
                for i, g in enumerate(per):
                    if g["kind"] != "row":
                        continue
                    a, b = o_fused[li][i].float(), o_seq[li][i].float()
                    worst = max(worst, float((a - b).abs().max() / b.abs().max().clamp_min(1e-6)))
            fused_err = worst
            if lib.tuna_check_device_status(stream.cuda_stream) != 0:
                fused_err = float("inf")
    # the same host-buffer sequence captured once and replayed: the host only pays one graph launch per step
    e2e_graph, e2e_launch = None, "eager calls"
    if not args.no_graph:
        try:
            with torch.cuda.stream(stream):
                step_e2e()
                stream.synchronize()
                torch.cuda.synchronize()
                e2e_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(e2e_graph, stream=stream):
                    step_e2e()
            e2e_launch = "CUDA graph replay of the captured call sequence"
        except Exception as exc:  # capture not possible on this stack: time the eager calls
            e2e_graph = None
            e2e_launch = f"eager calls (capture failed: {type(exc).__name__})"
            torch.cuda.synchronize()
    run_e2e = e2e_graph.replay if e2e_graph is not None else step_e2e
    inner_e2e = args.inner if args.inner > 0 else inner_for(run_e2e, args.steps)
    ms_e2e = timed(run_e2e, args.steps, args.warmup, inner_e2e)

    # ---- roofline of the dominant kernel: the largest GEMM of the step, timed alone with CUDA events
    dom = max(range(len(shapes)), key=lambda i: gemms[0][i]["m"] * gemms[0][i]["k"])
    gd = gemms[0][dom]

    def dom_pass():
        for per in gemms:
            g = per[dom]
            tuna_b200.matmul(x_dev[dom], g["q"], g["s"], code, o_dev[dom], g["m"], tokens, g["k"], workspace=ws)

    dom_graph = None if args.no_graph else capture(dom_pass)
    run_dom = dom_graph.replay if dom_graph is not None else dom_pass
    inner_dom = max(1, int(round(0.5e3 / (timed(run_dom, 1, 2) * max(args.steps, 5)))))
    ms_dom = timed(run_dom, max(args.steps, 5), args.warmup, inner_dom) / layers
    allgather_us = None
    if world > 1:
        col = next((i for i, g in enumerate(gemms[0]) if g["kind"] == "col"), None)
        if col is not None:
            gathered = torch.empty((world * tokens, gemms[0][col]["m"]), dtype=torch.float16, device=dev)
            allgather_us = timed(lambda: dist.all_gather_into_tensor(gathered, o_dev[col]), 50, 10) * 1e3
    clocks = sampler.stop() if rank == 0 else None

    # N > 1: the step is the faster of the two ways to sum the K-split layers (both are reported)
    ms_allreduce = ms_step
    reduce_kind = "NCCL all-reduce after the launch" if world > 1 else None
    if ms_fused is not None and fused_err is not None and fused_err <= 1e-2 and ms_fused < ms_step:
        ms_step = ms_fused
        reduce_kind = "fused: peer stores from the GEMM epilogue + one reduce kernel per launch (tuna_matmul_sequence_reduce)"

    dom_bytes = alg_bytes(gd["m"], tokens, gd["k"])
    peak, peak_kind = measured_peak()
    cfg = tuna_b200.lookup_config(gd["m"], tokens, gd["k"])
    kernel_name = KERNEL_NAMES.get(cfg.path, str(cfg.path))
    if tokens >= 256:
        # tensor-bound regime: flops per launch against the measured cuBLAS bf16 burst figure
        flops = 2.0 * gd["m"] * tokens * gd["k"]
        tpeak, tkind = measured_peak("bf16_tflops", 1590.0)
        roofline = {
            "bound": "tensor", "achieved": flops / (ms_dom * 1e-3) / 1e12, "peak": tpeak, "unit": "TFLOP/s",
            "frac": flops / (ms_dom * 1e-3) / 1e12 / tpeak, "traffic": None,
            "frac_of_nominal_fp16_2250": flops / (ms_dom * 1e-3) / 1e12 / NOMINAL_FP16_TFLOPS,
            "kernel": kernel_name, "shape": {"m": gd["m"], "n": tokens, "k": gd["k"]}, "us_per_launch": ms_dom * 1e3,
            "flops_per_launch": flops, "peak_source": f"{tkind} cuBLAS bf16 burst throughput",
            "timing": "that GEMM alone over the layers' distinct weights, CUDA-graph replay, CUDA events",
        }
    else:
        traffic = DRAM_TRAFFIC_PER_LAUNCH.get((gd["m"], tokens, gd["k"], cfg.path))
        roofline = {
            "bound": "hbm", "achieved": dom_bytes / (ms_dom * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
            "frac": dom_bytes / (ms_dom * 1e-3) / 1e9 / peak, "traffic": traffic[0] if traffic else None,
            "traffic_source": traffic[1] if traffic else None,
            "kernel": kernel_name, "shape": {"m": gd["m"], "n": tokens, "k": gd["k"]}, "us_per_launch": ms_dom * 1e3,
            "algorithmic_bytes_per_launch": dom_bytes, "peak_source": f"{peak_kind} copy bandwidth",
            "timing": "that GEMM alone over the layers' distinct weights, CUDA-graph replay, CUDA events",
        }

    # the launch that dominates the timed region is the sequence kernel itself: one launch = one step
    roofline_single = roofline
    rank_bytes = sum(alg_bytes(g["m"], tokens, g["k"]) for per in gemms for g in per)  # this GPU's share of the step
    if tokens < 256:
        seq_traffic = DRAM_TRAFFIC_PER_LAUNCH.get(("sequence", args.workload, world))
        roofline = {
            "bound": "hbm", "achieved": rank_bytes / (ms_step * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
            "frac": rank_bytes / (ms_step * 1e-3) / 1e9 / peak,
            "traffic": seq_traffic[0] if seq_traffic else None, "traffic_source": seq_traffic[1] if seq_traffic else None,
            "kernel": "gemm_w4a16_tstream_kernel (tcgen05 weight streaming), one persistent launch over the step's %d GEMMs" % gemms_per_step,
            "us_per_launch": ms_step * 1e3 / launches_per_step, "algorithmic_bytes_per_launch": rank_bytes / launches_per_step,
            "per": "GPU (one rank's launch over its shards; with N GPUs the step also contains the all-reduce)",
            "peak_source": f"{peak_kind} copy bandwidth", "timing": "CUDA events around the timed region (graph replays of the step), divided by the launches in it",
        }

    extras = None
    if world == 1 and not args.no_extras and args.workload == "mistral7b_mlp_m16" and args.layers == 0:
        gemms, graph, dom_graph, e2e_graph, pc_graph, seq, hseq, seq_gemms, host_gemms = (None,) * 9  # free the headline's weights first
        torch.cuda.empty_cache()
        try:
            extras = run_extras(dev, stream, timed, code, args.steps)
        except Exception as exc:
            extras = {"error": f"{type(exc).__name__}: {exc}"}

    # Every rank is done with the process group at the same point, before rank 0 goes on alone.
    # The group is not destroyed: tearing down a communicator that a live CUDA graph still refers
    # to blocks, so the processes leave with os._exit once their output is flushed.
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
    if rank != 0:
        sys.stdout.flush()
        os._exit(0)  # nothing left to do; skip the interpreter's teardown of CUDA graphs and NCCL state

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_record(layers, shapes, tokens)

    h2d = layers * sum(t.numel() * 2 for t in x_host)
    d2h = layers * sum(t.numel() * 2 for t in o_host)
    gbs = total_bytes / (ms_step * 1e-3) / 1e9
    line = {
        "metric": "m16_gemm_effective_hbm_bandwidth", "value": gbs, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16*u4->f32", "data": "synthetic",
        "config": {
            "workload": args.workload, "tokens": tokens, "layers": layers,
            "gemms_per_layer": [{"kind": k_, "m": m, "k": k} for k_, m, k in shapes],
            "parallelism": "single GPU" if world == 1 else f"tp{world}: one seeded weight set sharded by tuna_b200.sharding - column-parallel N-split + row-parallel K-split; sum of the K-split partials: {reduce_kind}",
            "l2": "inputs larger than L2: every layer has its own weights (%.2f GB per step per job)" % (total_bytes / 1e9),
            "launch": "CUDA graph replay" if graph is not None or not args.no_graph else "eager",
            "timed_region": f"{args.steps} steps x {inner} back-to-back replays of the step = {args.steps * inner * ms_step / 1e3:.2f} s; ms_per_step is per replay",
        },
        "inner_repeats": inner,
        "us_per_gemm_avg": ms_step * 1e3 / gemms_per_step,
        "api": "tuna_matmul_sequence: the step's GEMMs as persistent launches of up to 64 GEMMs; `per_call` is the same step through tuna_matmul, one launch per GEMM",
        "per_call": {"ms_per_step": ms_per_call, "value": total_bytes / (ms_per_call * 1e-3) / 1e9, "unit": "GB/s", "launch": "CUDA graph replay of 64 tuna_matmul calls"},
        "pct_of_8tbs": gbs / 8000.0 * 100.0,
        "eager_ms_per_step": ms_eager,
        "roofline": roofline,
        "roofline_single_gemm": roofline_single,
        "cpu_baseline": cpu,
        "e2e": {"value": total_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "inner_repeats": inner_e2e, "sum_of_k_split_partials": e2e_reduce,
                "how": "tuna_b200.HostSequence: pinned HOST activations and outputs of every GEMM, the step in %d groups (copy-in of a group, launch of the previous one, copy-out of the one before on three streams)" % args.e2e_groups + "; weights resident (they are parameters)", "launch": e2e_launch},
        # the library's own kernels in the timed region (the fused step adds one reduce kernel per launch)
        "gpu_launches": launches_per_step * (2 if ms_step is ms_fused else 1) * args.steps * inner,
        "clocks": clocks,
        "parity": parity,
    }
    if world > 1:
        line["multi_gpu"] = {"gemm_only_ms_per_step": ms_gemm_only, "gemm_plus_allreduce_ms_per_step": ms_allreduce,
                             "fused_gemm_reduce_ms_per_step": ms_fused, "fused_vs_allreduce_max_rel_diff": fused_err,
                             "fused_unavailable": fused_note, "step_uses": reduce_kind,
                             "gemm_only_gbs": total_bytes / (ms_gemm_only * 1e-3) / 1e9 if ms_gemm_only else None,
                             "allgather_us": allgather_us,
                             "note": "the K-split layers' partial outputs lie in one buffer and are summed by ONE all-reduce after the step's launch (per group of the sequence in the end-to-end path); the all-gather that would reassemble a column-parallel output is timed alone, it is not part of the MLP step"}
    if extras is not None:
        line["extras"] = extras
    print(json.dumps(line), flush=True)
    if world > 1:
        sys.stdout.flush()
        os._exit(0)


# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel: (bytes, where they come from).
# The full-size launch (64 GEMMs, 2.9 GB) is too large to capture under `ncu --set full`; the figure is the
# capture of the same kernel over 4 layers (8 GEMMs: 356.87 MB read + 8.1 MB written for 359.40 MB
# algorithmic), scaled by the layers - traffic grows in proportion, every layer has its own weights.
DRAM_TRAFFIC_PER_LAUNCH: dict = {
    ("sequence", "mistral7b_mlp_m16", 1): (8 * (356.87e6 + 8.14e6), "ncu capture of `python bench.py --layers 4 --steps 1 --warmup 3 "
                                            "--no-cpu-baseline --no-extras --inner 1` (one sequence launch; kernel as of commit 8564eba), scaled x8 to the 32 layers"),
}

if __name__ == "__main__":
    main()
