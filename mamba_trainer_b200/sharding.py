"""Sharding of the scan over the GPUs of one box.

Every (batch, head) pair is an independent recurrence (all reference ops on the path batch or
broadcast over those two axes, src/ssm/scan.rs:116-291), so the path shards with NO collective
inside it: contiguous batch slices first, and heads only once there are more ranks than
sequences.  The only cross-shard quantities are the per-head parameter gradients (a_log, D),
which are partial sums per shard; collectives below exist for verification and for those sums.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    batch: slice
    heads: slice

    @property
    def n_batch(self) -> int:
        return self.batch.stop - self.batch.start

    @property
    def n_heads(self) -> int:
        return self.heads.stop - self.heads.start


def _split(n: int, parts: int, i: int) -> slice:
    base, extra = divmod(n, parts)
    lo = i * base + min(i, extra)
    return slice(lo, lo + base + (1 if i < extra else 0))


def shard_plan(batch: int, heads: int, world: int, rank: int) -> Shard:
    """Batch slices when there are enough sequences; otherwise batch x head blocks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if world <= batch:
        return Shard(rank, world, _split(batch, world, rank), slice(0, heads))
    if world % batch:
        raise ValueError(f"with more ranks than sequences, world ({world}) must be a multiple of batch ({batch})")
    per = world // batch
    if heads % per:
        raise ValueError(f"heads ({heads}) must split evenly over {per} ranks per sequence")
    b, hpart = divmod(rank, per)
    return Shard(rank, world, slice(b, b + 1), _split(heads, per, hpart))


_PER_TOKEN = ("x", "b", "c", "dt", "lam", "theta", "dy")     # [B, T, H, ...]
_PER_HEAD = ("a_log", "d_skip")                              # [H]
_STATE = ("h0", "last_u0", "angle0")                         # [B, H, ...]


def shard_inputs(t: Dict[str, Optional[torch.Tensor]], shard: Shard) -> Dict[str, Optional[torch.Tensor]]:
    """This rank's contiguous copy of every scan input."""
    out = {}
    for k, v in t.items():
        if v is None:
            out[k] = None
        elif k in _PER_TOKEN:
            out[k] = v[shard.batch, :, shard.heads].contiguous()
        elif k in _PER_HEAD:
            out[k] = v[shard.heads].contiguous()
        elif k in _STATE:
            out[k] = v[shard.batch, shard.heads].contiguous()
        else:
            out[k] = v
    return out


def gather_per_token(local: torch.Tensor, batch: int, heads: int, group=None) -> torch.Tensor:
    """All-gather shards of a [B_s, T, H_s, ...] tensor back into [B, T, H, ...] (verification only)."""
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    pieces = [None] * world
    dist.all_gather_object(pieces, local.cpu(), group=group)
    full = torch.empty((batch, local.shape[1], heads) + tuple(local.shape[3:]), dtype=local.dtype)
    for r, piece in enumerate(pieces):
        s = shard_plan(batch, heads, world, r)
        full[s.batch, :, s.heads] = piece
    return full


def reduce_per_head(local: torch.Tensor, heads: int, shard: Shard, group=None) -> torch.Tensor:
    """Sum the shards' partial per-head gradients into the full [H] vector (what the trainer's
    data-parallel all-reduce does for a_log and D)."""
    import torch.distributed as dist
    full = torch.zeros(heads, dtype=local.dtype, device=local.device)
    full[shard.heads] = local
    dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
    return full
