"""Generates tests/golden/ref_*.npz by running the REFERENCE's own CUDA kernels.

Run on a GPU box (sm_100) after `make -C oracle ref` has produced
oracle/_ref/libtuna_ref.so from the reference tree (compiled where it lies,
nothing copied).  For each case the seeded inputs of oracle.synth_inputs are
fed to the reference's `wrapper` (kernel.cu:3009) and `dequantize_wrapper`
(kernel.cu:3243) through the C shim, and the outputs are stored.  The
fixtures pin the CPU oracle (tests/test_oracle.py) and the CUDA path
(tests/test_gpu_parity.py) to what the reference itself computes.

Every device tensor is carved out of one large zero-filled slab with wide gaps:
the reference's loaders prefetch a few tiles past the end of a K range and read
scales for a whole row tile without bounds checks, so reads a little outside a
tensor are expected and must land in owned memory.

    python tests/golden/make_reference_fixtures.py [outdir]
"""

import ctypes
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import tuna_oracle as orc  # noqa: E402

# (m, n, k, seed): shapes the reference's table supports (kernel.cu:3022-3035), token counts that
# pick its "_1" and "_16" buckets
CASES = [(4096, 16, 4096, 101), (6144, 1, 4096, 102), (4096, 16, 14336, 103), (6144, 16, 4096, 104)]
GAP = 4 << 20


def main(outdir: Path):
    ref = ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libtuna_ref.so"))
    vp, ci = ctypes.c_void_p, ctypes.c_int
    ref.tuna_ref_matmul.argtypes = [vp] * 5 + [ci] * 3 + [vp]
    ref.tuna_ref_dequant.argtypes = [vp] * 4 + [ci] * 2 + [vp]
    stream = torch.cuda.current_stream().cuda_stream
    for (m, n, k, seed) in CASES:
        x, q, absmax, code = orc.synth_inputs(m, n, k, seed)
        sizes = [x.nbytes, q.nbytes, absmax.nbytes, code.nbytes, n * m * 2, m * k * 2]
        slab = torch.zeros(sum(s + GAP for s in sizes) + GAP, dtype=torch.uint8, device="cuda")
        views, off = [], GAP
        for s in sizes:
            views.append(slab[off:off + s])
            off += (s + GAP + 255) // 256 * 256
        for v, a in zip(views[:4], (x, q, absmax, code)):
            v.copy_(torch.from_numpy(a.view(np.uint8).ravel()))
        xd, qd, sd, cd, od, wd = views
        od.zero_()  # the reference accumulates split-K partials into the output (kernel.cu:2739-2745)
        ref.tuna_ref_matmul(qd.data_ptr(), xd.data_ptr(), cd.data_ptr(), sd.data_ptr(), od.data_ptr(), m, n, k, stream)
        ref.tuna_ref_dequant(qd.data_ptr(), sd.data_ptr(), cd.data_ptr(), wd.data_ptr(), m, k, stream)
        torch.cuda.synchronize()
        out = od.cpu().numpy().view(np.uint16).reshape(n, m)
        w16 = wd.cpu().numpy().view(np.uint16).reshape(m, k)
        rows = np.unique(np.concatenate([np.arange(4), np.random.default_rng(seed).integers(0, m, 4), [m - 1]]))
        nz = float((out != 0).mean())
        print(f"case m={m} n={n} k={k}: nonzero outputs {nz:.3f}")
        if nz < 0.5:
            raise SystemExit("reference launched nothing for this shape")
        np.savez_compressed(outdir / f"ref_m{m}_n{n}_k{k}.npz", m=m, n=n, k=k, seed=seed, matmul=out,
                            dequant_rows=rows, dequant_sample=w16[rows])


if __name__ == "__main__":
    out = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).parent
    out.mkdir(parents=True, exist_ok=True)
    main(out)
