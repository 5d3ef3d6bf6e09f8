"""Batch x head sharding of the chunk prefill over the GPUs of one node.

Every (batch, head) pair is an independent recurrence and every scale tensor is indexed by head, so a rank takes a
contiguous block of the flattened (b, h) index with no exchange step: split the batch first (inputs stay dense), then
heads within a batch element, slicing the scale dictionary with the heads. The reference is single-GPU
(``bench/mamba2_model.py:86``); this is the multi-GPU mode of the new implementation."""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Shard:
    b0: int
    b1: int
    h0: int
    h1: int

    @property
    def units(self):
        return (self.b1 - self.b0) * (self.h1 - self.h0)


def plan(B, H, world, rank):
    """Shard of ``rank``. world <= B: whole batch elements, as even as possible. world > B: world must be a multiple
    of B and H divisible by world // B; each batch element's heads are split over world // B ranks."""
    assert 0 <= rank < world
    if world <= B:
        base, extra = divmod(B, world)
        b0 = rank * base + min(rank, extra)
        return Shard(b0, b0 + base + (1 if rank < extra else 0), 0, H)
    assert world % B == 0, f"world size {world} must be a multiple of the batch {B} to split heads"
    per = world // B
    assert H % per == 0, f"{H} heads do not split over {per} ranks"
    hs = H // per
    b, part = divmod(rank, per)
    return Shard(b, b + 1, part * hs, (part + 1) * hs)


def take(shard, *tensors):
    """Slices [B,T,H,...] tensors (None passes through) to the shard, contiguous."""
    return tuple(None if t is None else t[shard.b0:shard.b1, :, shard.h0:shard.h1].contiguous() for t in tensors)


def take_scales(shard, scales):
    """Head-sliced copy of a kernel scale dictionary (every entry has the head as its first axis)."""
    return {k: (v if v is None else v[shard.h0:shard.h1].contiguous()) for k, v in scales.items()}


def gather_output(local, shard, B, H, group=None):
    """All ranks receive the full [B,T,H,V] output (outside any timed region; plain ``all_gather_object``-free path:
    equal-shaped shards go through ``all_gather``, ragged ones through a padded gather)."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    T, V = local.shape[1], local.shape[-1]
    shards = [plan(B, H, world, r) for r in range(world)]
    mb = max(s.b1 - s.b0 for s in shards)
    mh = max(s.h1 - s.h0 for s in shards)
    pad = local.new_zeros(mb, T, mh, V)
    pad[: local.shape[0], :, : local.shape[2]] = local
    bufs = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(bufs, pad, group=group)
    out = local.new_empty(B, T, H, V)
    for s, buf in zip(shards, bufs):
        out[s.b0:s.b1, :, s.h0:s.h1] = buf[: s.b1 - s.b0, :, : s.h1 - s.h0]
    return out
