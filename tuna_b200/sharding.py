"""Sharding of the packed weight format across GPUs, and the two tensor-parallel
layer kinds built on the GEMM.

The reference is single-GPU (no collective, no process group anywhere in its
tree); this module adds what the benchmark configurations ask for on one
8-GPU node:

* column-parallel (QKV, gate+up): output features are split into contiguous
  blocks.  In the packed layout `[m/8, k/8, 32]` (test.py:55-65) that is a
  contiguous slice of the leading dimension, so a shard is a view.  The GEMM
  needs no collective; an all-gather reassembles the output.
* row-parallel (attention out, down): the reduction dimension is split.  K
  tiles are the middle dimension of the packed layout, so a shard has to be
  repacked once into a contiguous `[m/8, (k/g)/8, 32]` tensor; partial outputs
  are summed with an all-reduce (or reduce-scatter).

The GEMM callable is a parameter so that the collective logic can be exercised
on CPU ranks (gloo) with a stand-in; the default is the CUDA op.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def _split_even(total: int, parts: int, align: int, what: str) -> int:
    if total % (parts * align):
        raise ValueError(f"{what}={total} does not split into {parts} shards of a multiple of {align}")
    return total // parts


def shard_columns(q: torch.Tensor, absmax: torch.Tensor, m: int, k: int, world: int, rank: int):
    """Output-feature (N-split) shard: returns (q_shard view, absmax_shard view, m_shard)."""
    ms = _split_even(m, world, 8, "m")
    q3 = q.reshape(m // 8, k // 8, 32)
    lo = rank * ms
    return q3[lo // 8 : (lo + ms) // 8], absmax[lo : lo + ms], ms


def shard_k(q: torch.Tensor, m: int, k: int, world: int, rank: int):
    """Reduction-dimension (K-split) shard, repacked contiguous: returns (q_shard, k_shard)."""
    ks = _split_even(k, world, 8, "k")
    q3 = q.reshape(m // 8, k // 8, 32)
    lo = rank * ks
    return q3[:, lo // 8 : (lo + ks) // 8, :].contiguous(), ks


def _default_matmul():
    from .ops import matmul

    return matmul


class ColumnParallelLinear:
    """o[n, m] = x[n, k] W^T with W's rows split across the group; optional all-gather."""

    def __init__(self, q, absmax, code, m: int, k: int, group=None,
                 matmul_fn: Optional[Callable] = None, gather_output: bool = True):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.m, self.k = m, k
        qs, ss, self.m_shard = shard_columns(q, absmax, m, k, self.world, self.rank)
        self.q = qs.contiguous()
        self.absmax = ss.contiguous()
        self.code = code
        self.matmul_fn = matmul_fn or _default_matmul()
        self.gather_output = gather_output and self.world > 1

    def forward(self, x: torch.Tensor, out_shard: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x.shape[0]
        if out_shard is None:
            out_shard = torch.empty((n, self.m_shard), dtype=torch.float16, device=x.device)
        self.matmul_fn(x, self.q, self.absmax, self.code, out_shard, self.m_shard, n, self.k)
        if not self.gather_output:
            return out_shard
        # all_gather_into_tensor concatenates along dim 0: gather [world * n, m_shard], then
        # interleave to [n, m].
        gathered = torch.empty((self.world * n, self.m_shard), dtype=out_shard.dtype, device=x.device)
        dist.all_gather_into_tensor(gathered, out_shard, group=self.group)
        return gathered.view(self.world, n, self.m_shard).permute(1, 0, 2).reshape(n, self.m)


class RowParallelLinear:
    """o[n, m] = sum over ranks of x[:, k-slice] W[:, k-slice]^T; all-reduce of the partials.

    Partials travel as fp16, like the fp16 split-K partials of the reference
    (kernel.cu:2719, 2742); `reduce_dtype=torch.float32` keeps them in fp32.
    With `exchange` (a `tuna_b200.Exchange` over the same group, at least
    `ReduceSequence.exchange_bytes([(m, 64, k_shard)], world)` bytes) and up to 64 tokens the
    sum is fused into the launch instead (`tuna_matmul_sequence_reduce`): no collective.
    """

    def __init__(self, q, absmax, code, m: int, k: int, group=None,
                 matmul_fn: Optional[Callable] = None, reduce_dtype=torch.float16, exchange=None):
        self.group = group
        self.exchange = exchange
        self._fused = {}  # (x pointer, out pointer, n) -> ReduceSequence
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.m, self.k = m, k
        self.q, self.k_shard = shard_k(q, m, k, self.world, self.rank)
        self.absmax = absmax
        self.code = code
        self.matmul_fn = matmul_fn or _default_matmul()
        self.reduce_dtype = reduce_dtype

    def slice_input(self, x_full: torch.Tensor) -> torch.Tensor:
        lo = self.rank * self.k_shard
        return x_full[:, lo : lo + self.k_shard].contiguous()

    def forward(self, x_shard: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x_shard.shape[0]
        if out is None:
            out = torch.empty((n, self.m), dtype=torch.float16, device=x_shard.device)
        if self.exchange is not None and n <= 64:
            from .ops import ReduceSequence

            key = (x_shard.data_ptr(), out.data_ptr(), n)
            seq = self._fused.get(key)
            if seq is None:  # a sequence holds addresses: one per (input, output) pair that was seen
                seq = ReduceSequence([(x_shard, self.q.reshape(-1), self.absmax, out, self.m, n, self.k_shard)], self.code, self.exchange)
                self._fused = {key: seq}
            seq.run()
            return out
        self.matmul_fn(x_shard, self.q, self.absmax, self.code, out, self.m, n, self.k_shard)
        if self.world > 1:
            if self.reduce_dtype == torch.float16:
                dist.all_reduce(out, group=self.group)
            else:
                acc = out.to(self.reduce_dtype)
                dist.all_reduce(acc, group=self.group)
                out.copy_(acc)
        return out
