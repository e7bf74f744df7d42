"""Batch sharding of the scan across the GPUs of one node.

Every (batch, channel) column of the scan is independent, so the path shards
by batch with no data-path collective: rank r of n owns a block of consecutive
batch rows and runs the ordinary single-GPU kernels on its own ``[T, B_r, D]``
tensors. The only communication is an optional gather of the (small) results
for validation: bit-packed spikes and the final membrane state.

Works with any ``torch.distributed`` backend (NCCL on GPUs, gloo on CPU).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def batch_shard(total_batch: int, world_size: int, rank: int) -> tuple[int, int]:
    """(first batch row, number of rows) of ``rank``. Rows are split as evenly as
    possible; the first ``total_batch % world_size`` ranks get one extra row."""
    if world_size < 1 or not 0 <= rank < world_size or total_batch < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(total_batch, world_size)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return start, count


def shard_time_major(t: torch.Tensor, world_size: int, rank: int) -> torch.Tensor:
    """The rank's contiguous ``[T, B_r, ...]`` block of a ``[T, B, ...]`` tensor."""
    start, count = batch_shard(t.shape[1], world_size, rank)
    return t[:, start:start + count].contiguous()


def gather_batch(local: torch.Tensor, total_batch: int, batch_dim: int, group=None) -> torch.Tensor:
    """All-gathers per-rank blocks along ``batch_dim`` (blocks may differ by one
    row; they are padded to the largest block for the collective)."""
    world = dist.get_world_size(group)
    sizes = [batch_shard(total_batch, world, r)[1] for r in range(world)]
    biggest = max(sizes)
    pad_shape = list(local.shape)
    pad_shape[batch_dim] = biggest
    padded = local.new_zeros(pad_shape)
    padded.narrow(batch_dim, 0, local.shape[batch_dim]).copy_(local)
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p.narrow(batch_dim, 0, n) for p, n in zip(parts, sizes)], dim=batch_dim)


def gather_packed_spikes(packed_local: torch.Tensor, local_shape, total_batch: int,
                         group=None) -> torch.Tensor:
    """Gathers bit-packed spikes of all ranks and returns them as a dense uint8
    ``[T, total_batch, *channels]`` tensor. ``packed_local`` is int32
    ``[T, ceil(B_r*D/32)]`` as produced by the packed scans; ``local_shape`` is the
    rank's ``(B_r, *channels)``."""
    T = packed_local.shape[0]
    cols = 1
    for s in local_shape:
        cols *= s
    bits = torch.arange(32, device=packed_local.device, dtype=torch.int32)
    dense = ((packed_local.unsqueeze(-1) >> bits) & 1).reshape(T, -1)[:, :cols]
    dense = dense.to(torch.uint8).reshape(T, *local_shape)
    return gather_batch(dense, total_batch, 1, group)
