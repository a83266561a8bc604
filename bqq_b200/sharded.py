"""Column-parallel (output-row patch) sharding of BinaryQuadratic layers.

Row patches never interact (out feature o = i*P + p depends on row patch i only), so rank g
of G keeps the row patches [g*rw/G, (g+1)*rw/G), needs the whole activation and produces the
output columns [g*out/G, (g+1)*out/G).  The only exchange is an all-gather of those columns;
no reduction is involved, and because the decode kernel's work split does not depend on the
number of row patches the gathered result is bit-identical to the single-GPU output.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from .bqq_modules import BinaryQuadratic, shard_rows


def row_patch_range(row_width: int, rank: int, world: int):
    """Row patches [lo, hi) owned by `rank`; row_width must divide evenly."""
    if row_width % world != 0:
        raise ValueError(f'row_width {row_width} is not divisible by world size {world}')
    per = row_width // world
    return rank * per, (rank + 1) * per


def gather_columns(y_local: torch.Tensor, group=None, out: torch.Tensor | None = None, peer=None) -> torch.Tensor:
    """All-gather column shards: y_local [..., n] on every rank -> [..., world*n], rank-major.

    With `peer` (a bqq_b200.peer.PeerGatherGroup of the same ranks) the gather is one kernel of this
    library that stores the slice into the peers' buffers over NVLink; otherwise it is the process
    group's all_gather_into_tensor, for which `out`, if given, is a reusable [world, rows, n] buffer
    (same dtype/device)."""
    if peer is not None:
        return peer.gather(y_local)
    world = dist.get_world_size(group)
    lead, n = y_local.shape[:-1], y_local.shape[-1]
    flat = y_local.reshape(-1, n).contiguous()
    if out is None:
        out = torch.empty((world,) + tuple(flat.shape), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(out.view(-1), flat.view(-1), group=group)
    return out.permute(1, 0, 2).reshape(*lead, world * n)


class ColumnParallelBinaryQuadratic(nn.Module):
    """One rank's shard of a BinaryQuadratic layer plus the all-gather of its outputs.

    forward(X) takes the full activation [..., in] and returns the full output [..., out]
    (gather=True) or only this rank's columns (gather=False, for consumers that are sharded
    the same way, e.g. attention heads or the SwiGLU product)."""

    def __init__(self, full: BinaryQuadratic, rank: int, world: int, group=None, gather: bool = True, peer=None):
        super().__init__()
        self.rank, self.world, self.group, self.gather, self.peer = rank, world, group, gather, peer
        self.out_features = full.row_width * full.y_row
        self.shard = shard_rows(full, rank, world)

    def forward(self, X):
        if self.gather and self.world > 1 and self.peer is not None:
            return self.shard.forward_gathered(X, self.peer)      # decode kernel sends its row patches itself
        y = self.shard(X)
        if not self.gather or self.world == 1:
            return y
        return gather_columns(y, self.group)
