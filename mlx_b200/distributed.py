"""N-sharded quantized linear over one process per GPU (NCCL through torch.distributed).

Mirrors the reference's tensor-parallel layer for quantized weights
(python/mlx/nn/layers/distributed.py:40-93 `_shard`/`_all_to_sharded`, :357-455
`QuantizedAllToShardedLinear`) and its all_gather primitive
(mlx/distributed/ops.cpp:62-84, mlx/distributed/nccl/nccl.cpp:346-358):

* rank r keeps rows [r*N/R, (r+1)*N/R) of `weight`, `scales` and `biases`; the packed
  layout is row-major, so a shard is a contiguous slice and is never repacked;
* x is replicated; every rank computes y_r [.., M, N/R] with its local rows;
* `all_gather` concatenates the shards.  The reference gathers on axis 0; `gather_output`
  returns the row-major [.., M, N] a caller of an unsharded layer would see.

torch.distributed only carries the collective; the matmul is libb200q.so.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from . import ops


def shard_bounds(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Row range of `rank` when n rows are split evenly (n must divide: the reference
    raises for uneven splits, nn/layers/distributed.py:75-83)."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"invalid rank {rank} for world size {world}")
    if n % world != 0:
        raise ValueError(f"cannot shard {n} rows evenly across {world} ranks")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """The slice of a [.., N, C] tensor owned by `rank` (axis max(ndim-2, 0))."""
    axis = max(t.ndim - 2, 0)
    lo, hi = shard_bounds(t.shape[axis], rank, world)
    return t.narrow(axis, lo, hi - lo).contiguous()


class QuantizedAllToShardedLinear:
    """y_r = x @ dequant(W_r)^T with the rows of W split across the ranks of `group`."""

    def __init__(self, weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                 group_size: int = 64, bits: int = 4, group: Optional[dist.ProcessGroup] = None,
                 rank: Optional[int] = None, world: Optional[int] = None, already_sharded: bool = False):
        if rank is None or world is None:
            rank = dist.get_rank(group) if dist.is_initialized() else 0
            world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.group, self.rank, self.world = group, rank, world
        self.group_size, self.bits = group_size, bits
        if already_sharded:
            self.weight, self.scales, self.biases = weight, scales, biases
        else:
            self.weight = shard_rows(weight, rank, world)
            self.scales = shard_rows(scales, rank, world)
            self.biases = shard_rows(biases, rank, world)
        self.n_local = self.weight.shape[-2]
        self._gather_buf = None

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return ops.quantized_matmul(x, self.weight, self.scales, self.biases, transpose=True,
                                    group_size=self.group_size, bits=self.bits)

    def gather_output(self, y_local: torch.Tensor) -> torch.Tensor:
        """all_gather of the per-rank outputs -> [.., M, N] row-major."""
        return all_gather_columns(y_local, self.group, self.world, cache=self)


def all_gather_columns(y_local: torch.Tensor, group=None, world: Optional[int] = None, cache=None) -> torch.Tensor:
    """Concatenate per-rank [.., M, n] blocks along the last axis."""
    if world is None:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return y_local
    y_local = y_local.contiguous()
    shape = (world,) + tuple(y_local.shape)
    buf = getattr(cache, "_gather_buf", None) if cache is not None else None
    if buf is None or tuple(buf.shape) != shape or buf.dtype != y_local.dtype or buf.device != y_local.device:
        buf = torch.empty(shape, dtype=y_local.dtype, device=y_local.device)
        if cache is not None:
            cache._gather_buf = buf
    # axis-0 gather, exactly the reference's AllGather ([R*d0, ...] == [R, d0, ...])
    if y_local.is_cuda:
        dist.all_gather_into_tensor(buf, y_local, group=group)
    else:  # CPU process groups (gloo) gather into a list of views of the same buffer
        dist.all_gather([buf[r] for r in range(world)], y_local, group=group)
    # [R, .., M, n] -> [.., M, R*n]
    nd = buf.ndim
    perm = tuple(range(1, nd - 1)) + (0, nd - 1)
    out = buf.permute(perm)
    return out.reshape(tuple(y_local.shape[:-1]) + (world * y_local.shape[-1],))


def expert_bounds(n_experts: int, rank: int, world: int) -> Tuple[int, int]:
    """Experts owned by `rank` in the expert-parallel layout (contiguous blocks)."""
    return shard_bounds(n_experts, rank, world)
