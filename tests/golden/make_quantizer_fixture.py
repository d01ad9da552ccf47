"""Golden vectors for the quantizer: the reference's `quantize_blockwise_dynamic_4bit`
(test.py:7-68, block_size = k, preprocess=True) restated with the same torch operations on the
CPU (the reference module itself cannot be imported without its CUDA extension and pins its
codebook to "cuda", test.py:2,38).  Run once in the build container:

    python tests/golden/make_quantizer_fixture.py

writes tests/golden/quantizer_torch_cpu.npz (fp16 weights as raw bits, packed codes, absmax).
"""

from pathlib import Path

import numpy as np
import torch

NF4 = [-1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
       -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
       0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941,
       0.7229568362236023, 1.0]


def quantize_like_reference(inp: torch.Tensor):
    m, k = inp.shape
    temp = inp.clone().flatten().reshape(m, -1)                      # block_size = k: one block per row
    absmax = torch.max(temp.abs(), dim=1)[0].float()
    code = torch.tensor(NF4, dtype=torch.float)
    normalized = torch.divide(temp, absmax.unsqueeze(-1)).flatten()  # fp16 / fp32 -> fp32
    candidates = torch.sub(normalized.unsqueeze(0), code.unsqueeze(-1)).abs()
    results = torch.argmin(candidates, keepdim=True, dim=0).flatten().to(torch.uint8)
    results = results.reshape(-1, m // 8, 8, k // 8, 4, 2).permute(0, 1, 3, 2, 4, 5).reshape(-1, m // 8, k // 8, 32, 2)
    results = results[..., 0] * 16 + results[..., 1]
    return results.reshape(m // 8, k // 8, 32), absmax


def main():
    g = torch.Generator().manual_seed(20240)
    m, k = 64, 256
    w = (torch.randn(m, k, generator=g) * 0.05).half()
    w[3] = 0                      # a row of zeros: 0/0, every distance NaN
    w[5, :16] = w[5, 16:32]       # repeated values
    w[7] = w[7].abs().max()       # a constant row: every quotient is exactly 1
    # exact midpoints between neighbouring codes, scaled by a power of two (ties go to the lower index)
    mids = torch.tensor([(NF4[i] + NF4[i + 1]) / 2 for i in range(15)]).half()
    w[9, :15] = mids * 0.5
    w[9, 15] = 0.5
    q, absmax = quantize_like_reference(w)
    out = Path(__file__).with_name("quantizer_torch_cpu.npz")
    np.savez_compressed(out, w_bits=w.numpy().view(np.uint16), q=q.numpy(), absmax=absmax.numpy())
    print("wrote", out, q.shape, absmax.shape)


if __name__ == "__main__":
    main()
