"""How the path shards over the GPUs of one box: independent batch rows, or -- for the
un-mixed middle of the sequence mixer -- independent channels.  No collective is needed
on the data path; `gather_*` exist for verification only.

The reference has no multi-GPU code on this path (its data parallelism lives in the
external Composer trainer, bert/main.py:229-260).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(n: int, rank: int, world: int):
    """[lo, hi) of `n` units owned by `rank`; the first n % world ranks own one extra."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    lo, hi = shard_range(x.shape[0], rank, world)
    return x[lo:hi]


def mixer_channel_shard_state(sd: dict, d_model: int, lo: int, hi: int, prefix: str = "") -> dict:
    """State dict of a mixer that owns channels [lo, hi) of the un-mixed middle of the
    sequence mixer (short conv, gates, long convolutions).

    in_linear keeps all input features but only the output rows c, D+c, 2D+c of the owned
    channels; short_filter, the filters' last Linear, bias and modulation deltas are sliced
    the same way; the small filter-MLP layers and positional embeddings are replicated.
    out_linear is NOT part of a channel shard: it mixes channels, so the shard's result is
    the (B, L, hi-lo) tensor out_linear would consume.
    """
    D = d_model
    rows = torch.cat([torch.arange(g * D + lo, g * D + hi) for g in range(3)])
    out = {}
    for k, v in sd.items():
        if not k.startswith(prefix):
            continue
        name = k[len(prefix):]
        if name in ("in_linear.weight", "in_linear.bias", "short_filter.weight", "short_filter.bias"):
            out[k] = v[rows]
        elif name.startswith("out_linear."):
            continue
        elif name.endswith(".6.weight") or name.endswith(".bias") and name.count(".") == 1:
            out[k] = v[lo:hi]
        elif name.endswith("modulation.deltas"):
            out[k] = v[..., lo:hi]
        else:
            out[k] = v
    return out


def gather_batch(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather equal-sized batch shards along dim 0 (verification only)."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=0)


def gather_channels(local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather equal-sized channel shards along the last dim (verification only)."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=-1)
