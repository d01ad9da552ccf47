"""tuna_b200 — B200-native FP16 x 4-bit(codebook) GEMM behind tuna's op surface.

`matmul` and `dequant` keep the signatures of the reference's torch extension
(extension.cpp:26-49): same argument order, same tensor layouts, same meaning
of m (output features), n (tokens) and k (reduction).  They call hand-written
sm_100a kernels through the C ABI of libtuna_b200.so; there is no other
implementation behind them.
"""

from .ops import Exchange, HostPipeline, HostSequence, MatmulSequence, ReduceSequence, dequant, matmul, matmul_batched, matmul_sequence, quantize, workspace_for, lookup_config  # noqa: F401
from ._lib import TunaConfig, TunaError, PATH_AUTO, PATH_STREAM, PATH_UMMA, PATH_TSTREAM  # noqa: F401

__all__ = [
    "matmul", "matmul_batched", "matmul_sequence", "MatmulSequence", "ReduceSequence", "Exchange", "HostSequence", "dequant", "quantize", "HostPipeline", "workspace_for", "lookup_config",
    "TunaConfig", "TunaError", "PATH_AUTO", "PATH_STREAM", "PATH_UMMA", "PATH_TSTREAM",
]
