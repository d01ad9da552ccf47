"""Benchmark of the FP16 x 4-bit(codebook) GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workload (default `mistral7b_mlp_m16`): the Mistral-7B MLP GEMMs at 16 tokens -
fused gate+up K=4096 -> N=28672, then down K=14336 -> N=4096 - for 32 layers
with DISTINCT synthetic weights per layer (2.7 GB of packed codes, far larger
than L2, so every step streams from HBM).  One step = one pass over the 32
layers = 64 GEMMs.  With N GPUs the layers are tensor-parallel: gate+up is
split by output columns (no collective), down is split along K and its partial
outputs are summed with an NCCL all-reduce; total work is fixed ("strong").

The metric is the reference README's: time per 16-token GEMM, expressed as
effective HBM bandwidth = algorithmic bytes / time, with
    bytes(m, n, k) = m*k/2 + 4*m + 64 + 2*n*k + 2*n*m.
`value` is measured with inputs resident on the device (CUDA-graph replay of
the step); `e2e` calls the op with HOST activations and outputs (pinned memory,
copies inside the timed region); `roofline` times the dominant kernel alone;
`cpu_baseline` / `--impl reference` time the CPU restatement of the reference's
dequantize-then-matmul on the host cores (the reference has no CPU path and no
CUDA-free build).
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
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [t.strip() for t in s.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- CPU reference arm

def cpu_reference_step(shapes, tokens, reps, oracle, layers=1):
    """dequantize (C oracle, all host threads) + torch.matmul (fp16, CPU) for each GEMM of `layers`
    layers with distinct weights.  Returns (seconds per pass list, algorithmic bytes per pass, threads)."""
    from oracle import tuna_oracle as orc

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


def load_oracle_lib():
    so = ROOT / "oracle" / "libtuna_oracle.so"
    if not so.exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "oracle"], check=True, capture_output=True)
    return ctypes.CDLL(str(so))


def run_reference_arm(args, layers, shapes, tokens):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # rank 0 alone runs the CPU reference; the other ranks exit 0 without work
    oracle = load_oracle_lib()
    sample_layers = min(layers, 8)
    times, nbytes, threads = cpu_reference_step(shapes, tokens, args.warmup + args.steps, oracle, sample_layers)
    timed = times[args.warmup:]
    sec = sum(timed) / len(timed)
    gbs = nbytes / sec / 1e9
    sample = (f"{sample_layers} of {layers} layers per step, distinct weights ({sample_layers * len(shapes)} GEMMs, {nbytes / 1e6:.1f} MB "
              "algorithmic): C dequant (all host threads) + torch.matmul fp16 on CPU")
    line = {
        "impl": "reference", "metric": "m16_gemm_effective_hbm_bandwidth", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16*u4->f32", "data": "synthetic",
        "config": {"workload": args.workload, "tokens": tokens, "step": f"bounded sample: {sample_layers} layers", "timing": "host wall clock"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


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
    ap.add_argument("--layers", type=int, default=0, help="use only the first N layers (profiling captures); 0 = all")
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
    from tuna_b200 import _lib
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
        limit = float(os.environ.get("TUNA_BENCH_WATCHDOG_S", "420"))

        def _give_up():
            print(json.dumps({"error": f"rank {rank}: multi-GPU bench exceeded {limit:.0f} s, aborted"}), flush=True)
            os._exit(2)

        watchdog = threading.Timer(limit, _give_up)
        watchdog.daemon = True
        watchdog.start()
    lib = _lib.load()

    # ---- synthetic weights: uniform-random codes (random bytes), scales U[0.005, 0.02] rounded to fp16
    gen = torch.Generator(device=dev)
    gen.manual_seed(1000 + rank)
    code = nf4_tensor(dev)
    gemms = []   # per layer: list of dicts
    for _layer in range(layers):
        per = []
        for kind, m, k in shapes:
            ms, ks = (m // world, k) if kind == "col" else (m, k // world)
            q = torch.randint(0, 256, (ms * ks // 2,), dtype=torch.uint8, device=dev, generator=gen)
            s = (0.005 + 0.015 * torch.rand(ms, device=dev, generator=gen)).half().float()
            per.append(dict(kind=kind, m=ms, k=ks, q=q, s=s))
        gemms.append(per)
    xgen = torch.Generator(device="cpu")
    xgen.manual_seed(7)
    x_host, x_dev, o_dev, o_host = [], [], [], []
    for kind, m, k in shapes:
        ms, ks = (m // world, k) if kind == "col" else (m, k // world)
        xh = torch.randn((tokens, k), generator=xgen).half()
        if kind == "row":
            xh = xh[:, rank * ks:(rank + 1) * ks].contiguous()
        x_host.append(xh.pin_memory())
        x_dev.append(xh.to(dev))
        o_dev.append(torch.empty((tokens, ms), dtype=torch.float16, device=dev))
        o_host.append(torch.empty((tokens, ms), dtype=torch.float16).pin_memory())
    ws_bytes = max(int(lib.tuna_matmul_workspace_bytes(g["m"], tokens, g["k"])) for g in gemms[0])
    ws = torch.zeros(max(ws_bytes, 1 << 20), dtype=torch.uint8, device=dev)
    stream = torch.cuda.Stream(device=dev)

    # K-split layers: every layer has its own output so that its all-reduce (NCCL's stream) can stay
    # in flight under the next layers' GEMMs; the step ends when the last reduction has finished
    o_layer = None
    if world > 1:
        o_layer = [[torch.empty_like(o_dev[i]) if g["kind"] == "row" else None for i, g in enumerate(per)] for per in gemms]

    def step_device():
        pending = []
        for li, per in enumerate(gemms):
            for i, g in enumerate(per):
                out = o_layer[li][i] if (o_layer is not None and o_layer[li][i] is not None) else o_dev[i]
                tuna_b200.matmul(x_dev[i], g["q"], g["s"], code, out, g["m"], tokens, g["k"], workspace=ws)
                if g["kind"] == "row" and world > 1:
                    pending.append(dist.all_reduce(out, async_op=True))
        for h in pending:
            h.wait()

    # end to end: every GEMM takes its activations from pinned HOST memory and returns its output
    # there, through the package's host-buffer API (copies on their own streams, overlapped with
    # the neighbouring GEMMs); the step ends when the last output has reached the host
    pipe = tuna_b200.HostPipeline(dev, max(t.numel() for t in x_host), max(t.numel() for t in o_host), depth=4)

    def step_e2e():
        pipe.begin()
        for per in gemms:
            for i, g in enumerate(per):
                reduce = (lambda od: dist.all_reduce(od)) if (g["kind"] == "row" and world > 1) else None
                pipe.matmul(x_host[i], g["q"], g["s"], code, o_host[i], g["m"], tokens, g["k"], workspace=ws, after_gemm=reduce)
        pipe.join()

    launches_per_step = layers * len(shapes)
    total_bytes = layers * sum(alg_bytes(m, tokens, k) for _, m, k in shapes)

    def timed(fn, steps, warmup):
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                fn()
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            stream.synchronize()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    # ---- device-resident number: CUDA-graph replay of one step (or eager with --no-graph)
    graph = None
    if not args.no_graph:
        with torch.cuda.stream(stream):
            step_device()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step_device()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_step = timed(graph.replay if graph is not None else step_device, args.steps, args.warmup)
    ms_eager = timed(step_device, args.steps, args.warmup) if graph is not None else ms_step
    # the same sequence captured once and replayed: the host only pays one graph launch per step
    e2e_graph, e2e_launch = None, "eager calls"
    if not args.no_graph and world == 1:
        try:
            with torch.cuda.stream(stream):
                step_e2e()
                stream.synchronize()
                torch.cuda.synchronize()
                pipe.reset()
                e2e_graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(e2e_graph, stream=stream):
                    step_e2e()
            e2e_launch = "CUDA graph replay of the captured call sequence"
        except Exception as exc:  # capture not possible on this stack: time the eager calls
            e2e_graph = None
            e2e_launch = f"eager calls (capture failed: {type(exc).__name__})"
            torch.cuda.synchronize()
    ms_e2e = timed(e2e_graph.replay if e2e_graph is not None else step_e2e, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None

    # ---- roofline of the dominant kernel: the largest GEMM of the step, timed alone with CUDA events
    dom = max(range(len(shapes)), key=lambda i: gemms[0][i]["m"] * gemms[0][i]["k"])
    gd = gemms[0][dom]

    def dom_pass():
        for per in gemms:
            g = per[dom]
            tuna_b200.matmul(x_dev[dom], g["q"], g["s"], code, o_dev[dom], g["m"], tokens, g["k"], workspace=ws)

    ms_dom = timed(dom_pass, max(args.steps, 5), args.warmup) / layers
    dom_bytes = alg_bytes(gd["m"], tokens, gd["k"])
    peak, peak_kind = measured_peak()
    cfg = tuna_b200.lookup_config(gd["m"], tokens, gd["k"])
    kernel_name = {1: "gemm_stream_kernel (mma.sync)", 2: "gemm_w4a16_umma_kernel (tcgen05)"}[cfg.path]
    if tokens >= 256:
        # tensor-bound regime: flops per launch against the measured cuBLAS bf16 burst figure
        flops = 2.0 * gd["m"] * tokens * gd["k"]
        tpeak, tkind = measured_peak("bf16_tflops", 1590.0)
        roofline = {
            "bound": "tensor", "achieved": flops / (ms_dom * 1e-3) / 1e12, "peak": tpeak, "unit": "TFLOP/s",
            "frac": flops / (ms_dom * 1e-3) / 1e12 / tpeak, "traffic": None,
            "kernel": kernel_name, "shape": {"m": gd["m"], "n": tokens, "k": gd["k"]}, "us_per_launch": ms_dom * 1e3,
            "flops_per_launch": flops, "peak_source": f"{tkind} cuBLAS bf16 burst throughput",
            "timing": "isolated back-to-back launches over the layers' distinct weights, CUDA events",
        }
    else:
        roofline = {
            "bound": "hbm", "achieved": dom_bytes / (ms_dom * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
            "frac": dom_bytes / (ms_dom * 1e-3) / 1e9 / peak, "traffic": DRAM_TRAFFIC_PER_LAUNCH.get((gd["m"], tokens, gd["k"])),
            "kernel": kernel_name, "shape": {"m": gd["m"], "n": tokens, "k": gd["k"]}, "us_per_launch": ms_dom * 1e3,
            "algorithmic_bytes_per_launch": dom_bytes, "peak_source": f"{peak_kind} copy bandwidth",
            "timing": "isolated back-to-back launches over the layers' distinct weights, CUDA events",
        }

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
        oracle = load_oracle_lib()
        sample_layers = min(layers, 8)
        times, nbytes, threads = cpu_reference_step(shapes, tokens, 4, oracle, sample_layers)
        sec = statistics.median(times[1:])
        cpu = {"value": nbytes / sec / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": f"{sample_layers} of {layers} layers with distinct weights ({sample_layers * len(shapes)} GEMMs, "
                         f"{nbytes / 1e6:.1f} MB algorithmic), median of 3 after 1 warm-up: C restatement of the "
                         "reference's dequant (all host threads) + torch.matmul fp16 on CPU",
               "seconds_per_sample": sec}

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
            "parallelism": "single GPU" if world == 1 else f"tp{world}: column-parallel N-split + row-parallel K-split with NCCL all-reduce",
            "l2": "inputs larger than L2: every layer has its own weights (%.2f GB per step per job)" % (total_bytes / 1e9),
            "launch": "CUDA graph replay" if graph is not None else "eager",
        },
        "us_per_gemm_avg": ms_step * 1e3 / launches_per_step,
        "pct_of_8tbs": gbs / 8000.0 * 100.0,
        "eager_ms_per_step": ms_eager,
        "roofline": roofline,
        "cpu_baseline": cpu,
        "e2e": {"value": total_bytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "how": "every GEMM called through tuna_b200.HostPipeline with pinned HOST activations and outputs (copy-in, GEMM and copy-out on three streams, 4 staging slots); weights resident (they are parameters)", "launch": e2e_launch},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        sys.stdout.flush()
        os._exit(0)


# dram__bytes_read.sum + dram__bytes_write.sum per launch from ncu captures of the dominant kernel
# (profiles/gemm_stream_mistral_mlp_16tok.md), keyed by (m, n, k); None for shapes not captured.
DRAM_TRAFFIC_PER_LAUNCH: dict = {
    (28672, 16, 4096): 59.009536e6 + 0.886272e6,
    (4096, 16, 14336): 29.875200e6,
}

if __name__ == "__main__":
    main()
