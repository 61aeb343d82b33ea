"""Token (and, for dense calls, sequence) sharding for multi-GPU runs: every query token is independent (no cross-token reduction),
so a batch splits into contiguous token ranges, one per rank, with the caches replicated (or
batch-partitioned by the caller) and NO collective on the data path.  Outputs stay on the rank
that owns the tokens; ``gather_outputs`` is a convenience for harnesses that want one tensor."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

TOKEN_KEYS = ("q", "swa_indices", "swa_lens", "extra_indices", "extra_lens")


def token_range(num_tokens: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous [start, stop) of rank `rank`; the first ``num_tokens % world_size`` ranks get one more."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} / world size {world_size}")
    base, rem = divmod(num_tokens, world_size)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def shard_tokens(kwargs: Dict[str, object], world_size: int, rank: int) -> Dict[str, object]:
    """Slice the per-token arguments of a sparse-MLA call to this rank's token range; cache, scale
    and attn_sink arguments are passed through untouched (replicated)."""
    T = kwargs["q"].shape[0]
    a, b = token_range(T, world_size, rank)
    out = dict(kwargs)
    for k in TOKEN_KEYS:
        v = kwargs.get(k)
        if v is not None:
            if v.shape[0] != T:
                raise ValueError(f"{k} has {v.shape[0]} rows, expected {T}")
            out[k] = v[a:b]
    return out


SEQUENCE_KEYS = ("q", "block_table", "cache_seqlens")


def shard_sequences(kwargs: Dict[str, object], world_size: int, rank: int) -> Dict[str, object]:
    """The same for a dense call (``flash_mla_with_kvcache``): q [b, s_q, h, d], block_table [b, pages] and
    cache_seqlens [b] are cut to this rank's contiguous range of sequences; the paged cache is passed through
    (replicated, or holding this rank's pages: the block table names them)."""
    B = kwargs["q"].shape[0]
    a, b = token_range(B, world_size, rank)
    out = dict(kwargs)
    for k in SEQUENCE_KEYS:
        v = kwargs[k]
        if v.shape[0] != B:
            raise ValueError(f"{k} has {v.shape[0]} rows, expected {B}")
        out[k] = v[a:b]
    return out


def gather_outputs(local_out: torch.Tensor, num_tokens: int, group=None) -> torch.Tensor:
    """The token shards of all ranks as one [num_tokens, H, 512] tensor on every rank (a convenience
    for harnesses, outside any timed region; the data path itself needs no collective)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    me = dist.get_rank(group)
    shards = []
    for r in range(world):
        a, b = token_range(num_tokens, world, r)
        shards.append(torch.empty((b - a,) + tuple(local_out.shape[1:]), dtype=local_out.dtype,
                                  device=local_out.device))
    if len({s.shape for s in shards}) == 1:
        dist.all_gather(shards, local_out.contiguous(), group=group)
    else:
        # ragged shards (num_tokens not a multiple of the world size): one broadcast per rank
        shards[me].copy_(local_out)
        for r in range(world):
            src = dist.get_global_rank(group, r) if group is not None else r
            dist.broadcast(shards[r], src=src, group=group)
    return torch.cat(shards, dim=0)
