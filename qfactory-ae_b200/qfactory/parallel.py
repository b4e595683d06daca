"""Tensor-parallel use of the quantized linear layer, one process per GPU.

The reference's own code has no parallelism; its vLLM hook is shard-agnostic and relies on
vLLM's ColumnParallelLinear (no collective) and RowParallelLinear (all-reduce after the local
matmul) (reference: third_party/vllm-bitblas/vllm/model_executor/layers/linear.py:382-394,
1100-1124).  This module gives the same two shardings for GPTQ-style tensors:

  column parallel  split N: every rank owns N/p output features with their scales and zeros;
                   outputs are disjoint, no collective
  row parallel     split K: every rank owns K/p input features (a whole number of quantisation
                   groups); the full-width partial results are summed with ONE all-reduce

The collective here is `torch.distributed.all_reduce` (NCCL over NVLink on GPUs, gloo in the CPU
tests); the decoder's decode steps use the peer-memory kernel of comm.py instead.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_columns(q, s, z, rank: int, world: int):
    """Column-parallel shard of codes [K,N], scales [G,N], zeros [G,N] (zeros may be None)."""
    N = q.shape[1]
    assert N % world == 0, f"N={N} not divisible by world size {world}"
    n0, n1 = rank * N // world, (rank + 1) * N // world
    return (q[:, n0:n1].contiguous(), None if s is None else s[:, n0:n1].contiguous(),
            None if z is None else z[:, n0:n1].contiguous())


def shard_rows(q, s, z, rank: int, world: int, group_size: int):
    """Row-parallel shard along K; K/world must be a whole number of groups (and of 64)."""
    K = q.shape[0]
    assert K % world == 0, f"K={K} not divisible by world size {world}"
    ks = K // world
    assert ks % 64 == 0, f"K shard {ks} must be a multiple of 64"
    k0 = rank * ks
    if group_size == -1:
        return q[k0 : k0 + ks].contiguous(), None, None
    assert ks % group_size == 0, f"K shard {ks} must hold whole groups of {group_size}"
    g0, g1 = k0 // group_size, (k0 + ks) // group_size
    return (q[k0 : k0 + ks].contiguous(), s[g0:g1].contiguous(), None if z is None else z[g0:g1].contiguous())


def all_reduce_sum(t: torch.Tensor, group=None) -> torch.Tensor:
    """In-place sum over ranks; a no-op without an initialised process group or with one rank."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t
