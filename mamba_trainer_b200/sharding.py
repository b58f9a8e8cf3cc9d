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


def shard_reverse_heads(heads: int, reverse_heads: int, shard: Shard) -> int:
    """How many of a shard's heads walk time right to left, when the last `reverse_heads` of all
    `heads` do (the bidirectional scan): those of the shard's head range that fall in the reversed
    tail, which is again a tail of the shard because head ranges are contiguous."""
    first_reversed = heads - reverse_heads
    return max(0, shard.heads.stop - max(shard.heads.start, first_reversed))


def shard_inputs(t: Dict[str, Optional[torch.Tensor]], shard: Shard) -> Dict[str, Optional[torch.Tensor]]:
    """This rank's contiguous copy of every scan input.  A bidirectional scan passes
    `shard_reverse_heads(...)` as the shard's own `reverse_heads`."""
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
    """All-gather shards of a [B_s, T, H_s, ...] tensor back into [B, T, H, ...] (verification only).
    The pieces travel as tensors on the device they live on - NCCL between GPUs, gloo between CPU
    ranks - one broadcast-free `all_gather` of equally sized, padded pieces; a shard's own tensor is
    the only memory any rank's kernels ever read."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    shards = [shard_plan(batch, heads, world, r) for r in range(world)]
    nb, nh = max(s.n_batch for s in shards), max(s.n_heads for s in shards)
    tail = tuple(local.shape[3:])
    padded = torch.zeros((nb, local.shape[1], nh) + tail, dtype=local.dtype, device=local.device)
    padded[:local.shape[0], :, :local.shape[2]] = local
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded, group=group)
    full = torch.empty((batch, local.shape[1], heads) + tail, dtype=local.dtype, device=local.device)
    for s, piece in zip(shards, pieces):
        full[s.batch, :, s.heads] = piece[:s.n_batch, :, :s.n_heads]
    return full


def reduce_per_head(local: torch.Tensor, heads: int, shard: Shard, group=None) -> torch.Tensor:
    """Sum the shards' partial per-head gradients into the full [H] vector (what the trainer's
    data-parallel all-reduce does for a_log and D)."""
    import torch.distributed as dist
    full = torch.zeros(heads, dtype=local.dtype, device=local.device)
    full[shard.heads] = local
    dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
    return full
