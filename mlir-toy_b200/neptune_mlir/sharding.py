"""Partitioning of the hot path over the GPUs of one node (one process per GPU).

Attention, batched decode and both scans shard over independent units -- (batch, head) pairs,
sequences, channels, heads -- with no data-path collective: each rank runs the same kernels on its
slice.  The one exchange step is the single-sequence decode whose KV cache is split along the
sequence: every rank reduces its slice to one partial (o, m, l) per query head, the partials are
all-gathered (``gather_partials``; 16 640 bytes per rank for 32 heads of 128) and merged by the same
log-sum-exp combine kernel that merges the splits of one GPU, with the rank index playing the role
of the split index (``gathered_strides``).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(n_units: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced [start, end) of ``n_units`` for ``rank``; the first n % world ranks get one more."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def gather_partials(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather per-rank partials [rows, D+2] (fp32) into [world, rows, D+2]."""
    if local.dtype != torch.float32 or local.dim() != 2 or not local.is_contiguous():
        raise ValueError("gather_partials expects a contiguous fp32 [rows, D+2] tensor")
    world = dist.get_world_size(group)
    rows, width = local.shape
    out = torch.empty((world * rows, width), dtype=local.dtype, device=local.device)  # concatenated along dim 0
    dist.all_gather_into_tensor(out, local, group=group)
    return out.view(world, rows, width)


def gathered_strides(rows: int, width: int) -> tuple[int, int]:
    """(row_stride, split_stride) in floats that address a [world, rows, width] gather as rows x splits."""
    return width, rows * width
