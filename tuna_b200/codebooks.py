"""Codebooks for the 4-bit weight format.

The GEMM takes the 16-entry codebook as an fp32 tensor per call; this module
only provides the one the reference's quantizer emits (test.py:19-40), the
"NormalFloat4" levels: index 0 is -1.0, index 7 is 0.0, index 15 is 1.0.
"""

NF4 = (
    -1.0,
    -0.6961928009986877,
    -0.5250730514526367,
    -0.39491748809814453,
    -0.28444138169288635,
    -0.18477343022823334,
    -0.09105003625154495,
    0.0,
    0.07958029955625534,
    0.16093020141124725,
    0.24611230194568634,
    0.33791524171829224,
    0.44070982933044434,
    0.5626170039176941,
    0.7229568362236023,
    1.0,
)


def nf4_tensor(device=None):
    import torch

    return torch.tensor(NF4, dtype=torch.float32, device=device)
