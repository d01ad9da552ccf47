"""Helpers shared by the GPU tests: device buffers with guard bands, calls through the C ABI."""

import ctypes

import numpy as np
import torch

from oracle import tuna_oracle as orc
from tuna_b200 import _lib

GUARD = 4096  # bytes of 0xFF either side of an output buffer


class Guarded:
    """A device buffer with canary bands: `view` is the usable middle part."""

    def __init__(self, nbytes: int, dtype, shape, device="cuda"):
        self.raw = torch.full((nbytes + 2 * GUARD,), 0xFF, dtype=torch.uint8, device=device)
        self.nbytes = nbytes
        self.view = self.raw[GUARD:GUARD + nbytes].view(dtype).view(*shape)

    def guards_intact(self) -> bool:
        return bool((self.raw[:GUARD] == 0xFF).all() and (self.raw[GUARD + self.nbytes:] == 0xFF).all())


def to_dev(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]


def make_case(m, n, k, seed):
    x, q, absmax, code = orc.synth_inputs(m, n, k, seed)
    return (x, q, absmax, code), to_dev(x, q, absmax, code)


def stream_ptr():
    return torch.cuda.current_stream().cuda_stream


def run_matmul(dev, m, n, k, cfg=None, out=None, ws=None):
    """Call tuna_matmul[_cfg] through the C ABI; returns (status, out tensor, guarded holder)."""
    lib = _lib.load()
    xd, qd, sd, cd = dev
    holder = None
    if out is None:
        holder = Guarded(n * m * 2, torch.float16, (n, m))
        out = holder.view
    if ws is None:
        if cfg is None:
            need = lib.tuna_matmul_workspace_bytes(m, n, k)
        else:
            need = 64 << 20
        ws = torch.zeros(max(int(need), 256), dtype=torch.uint8, device="cuda")
    args = (qd.data_ptr(), xd.data_ptr(), cd.data_ptr(), sd.data_ptr(), out.data_ptr(), m, n, k,
            ws.data_ptr(), ws.numel(), stream_ptr())
    st = lib.tuna_matmul(*args) if cfg is None else lib.tuna_matmul_cfg(*args, ctypes.byref(cfg))
    torch.cuda.synchronize()
    return st, out, holder


def check_parity(out, ref, tol=1e-2):
    """|out-ref| <= tol*|ref| + tol*rms(ref) element-wise and max|out-ref| <= tol*max|ref|.
    Both operands are fp16 values of a fp32-accumulated GEMM; the expected error is one fp16
    rounding (~5e-4)."""
    a, b = orc.parity_error(out, ref)
    assert a <= tol and b <= tol, f"parity error {a:.3e} / {b:.3e} exceeds {tol}"
    return a, b
